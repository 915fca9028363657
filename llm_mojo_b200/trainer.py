"""Training loop: the public API behind the ``train_gpt2`` CLI and ``bench.py``.

Parity: ``train_gpt2.mojo:6020-6086`` (TrainArgs and defaults), ``:6161-6613`` (``train``: grad
accumulation, val loss, sampling, checkpoint cadence, per-step line with loss / norm z-scores,
lr, ms, MFU, EMA tok/s), ``:6130-6147`` (resume from the newest ``model_N.bin``).

One process drives one GPU.  ``Trainer.train_step()`` is one optimizer step: ``grad_accum``
micro-steps (pinned-host batch → async H2D → forward → backward, the next batch being read on a
worker thread meanwhile), gradient reduction (ZeRO engine), global-norm clip computed on the
device, AdamW.  The only host synchronisation is the loss read at the end of the step.

Failure handling (``train_gpt2.mojo:6871-6876``, ``llmm/zero.mojo:73-108``): every step starts by polling the
job's sticky abort key, and the loss read also reads the status word that kernels with bounded waits set when a
wait expires.  A non-zero status means this step's collectives did not complete: the rank re-arms its
communication state, sets the abort key and raises ``DeviceWaitExpired`` instead of returning a loss, and every
peer raises ``PeerAborted`` at its next step or barrier, so a supervisor can restart the job from the last
checkpoint.  Phases in which ranks do different amounts of host work (checkpoint write, validation, sampling) end
with a host barrier, so no rank enters the bounded device waits of the next step while another is still busy.
"""
from __future__ import annotations

import math
import os
import time
from dataclasses import dataclass, field
from typing import List, Optional

import torch

from .config import GPT2Config, Precision
from .models.gpt2 import GPT2
from .utils import checkpointing as ckpt
from .utils.dataloader import DataLoader, resolve_data_files
from .utils.logger import OutlierDetector, TokenRateEMA, format_step_line
from .utils.mfu import estimate_mfu
from .utils.profiler import TraceProfiler
from .utils.sampler import SamplerRNG, sample_softmax
from .utils.scheduler import LRScheduler
from .utils.tokenizer import Tokenizer


@dataclass
class TrainArgs:
    """llm.c-style configuration; field ↔ CLI flag (``train_gpt2.mojo:6020-6052``)."""
    train_data_pattern: str = "./data/.tinyshakespeare/tiny_shakespeare_train.bin"   # -i
    val_data_pattern: str = "./data/.tinyshakespeare/tiny_shakespeare_val.bin"       # -j
    load_filename: str = "gpt2_124M.bin"      # -e  checkpoint, .safetensors or descriptor
    output_log_dir: str = ""                  # -o
    checkpoint_every: int = 0                 # -n
    resume: int = 0                           # -y
    batch_size: int = 4                       # -b
    seq_len: int = 1024                       # -t
    total_batch_size: int = -1                # -d
    learning_rate: float = 3e-4               # -l
    lr_scheduler_type: str = "cosine"         # -k
    warmup_iterations: int = 0                # -u
    final_learning_rate_frac: float = 1.0     # -q
    weight_decay: float = 0.0                 # -c
    val_loss_every: int = 20                  # -v
    val_max_steps: int = 20                   # -m
    sample_every: int = 20                    # -s
    gen_tokens: int = 64                      # -g
    overfit_single_batch: int = 0             # -a
    max_steps: int = -1                       # -x
    zero_stage: int = 0                       # -z
    # runtime axes that are compile-time defines in the reference
    precision: str = "bf16"
    grad_clip: float = 1.0
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    recompute: bool = False
    device: str = ""
    synthetic: bool = False                   # uniform random tokens instead of files
    comm_backend: str = "auto"                # auto | p2p | nccl | gloo
    tokenizer_path: str = "gpt2_tokenizer.bin"
    fp8_static_scales: str = ""               # JSON table from calibrate_fp8_scales.py: static instead of delayed scaling


class DeviceWaitExpired(RuntimeError):
    """A bounded device-side wait (peer flag or mbarrier) gave up during the step: its results are not valid."""


class SyntheticLoader:
    """Uniform tokens in [0, V): inputs and targets (inputs shifted by one), pinned host memory."""

    def __init__(self, B: int, T: int, vocab: int, rank: int = 0, seed: int = 1234, pin: Optional[bool] = None,
                 distinct_batches: int = 4):
        g = torch.Generator().manual_seed(seed + rank)
        pin = torch.cuda.is_available() if pin is None else pin
        self._batches = []
        for _ in range(distinct_batches):
            toks = torch.randint(0, vocab, (B * T + 1,), generator=g, dtype=torch.int32)
            x = torch.empty(B * T, dtype=torch.int32, pin_memory=pin)
            y = torch.empty(B * T, dtype=torch.int32, pin_memory=pin)
            x.copy_(toks[:-1]); y.copy_(toks[1:])
            self._batches.append((x, y))
        self._i = 0
        self.num_tokens = B * T * distinct_batches
        self.inputs, self.targets = self._batches[0]

    def next_batch(self):
        self.inputs, self.targets = self._batches[self._i % len(self._batches)]
        self._i += 1
        return self.inputs, self.targets

    def prefetch(self):
        pass

    def mark_consumed(self):
        pass                                  # batches are never rewritten

    def reset(self):
        self._i = 0

    def state(self):
        return {"should_shuffle": 0, "shuffle_draws": 0, "current_shard_idx": 0, "current_sample_idx": self._i}

    def restore(self, should_shuffle, shuffle_draws, current_shard_idx, current_sample_idx):
        self._i = current_sample_idx


class Trainer:
    def __init__(self, args: TrainArgs, rank: int = 0, world_size: int = 1, local_rank: Optional[int] = None,
                 dist_ctx=None):
        self.args, self.rank, self.world_size = args, rank, world_size
        if args.device:
            self.device = torch.device(args.device)
        elif torch.cuda.is_available() and not os.environ.get("LLMM_USE_CPU"):
            lr_ = rank if local_rank is None else local_rank
            self.device = torch.device("cuda", lr_ % torch.cuda.device_count())
            torch.cuda.set_device(self.device)
        else:
            self.device = torch.device("cpu")
        precision = args.precision if self.device.type == "cuda" else "fp32"
        self.precision = Precision(precision)
        B, T = args.batch_size, args.seq_len
        tokens_per_fwdbwd = B * T * world_size
        total = args.total_batch_size if args.total_batch_size > 0 else tokens_per_fwdbwd
        if total % tokens_per_fwdbwd:
            raise ValueError("total batch size must be divisible by B*T*world_size")
        self.grad_accum = total // tokens_per_fwdbwd
        self.total_batch_size = total

        self.dist_ctx = dist_ctx
        self.coord = dist_ctx.coord if dist_ctx is not None else None
        if self.coord is None and world_size > 1 and torch.distributed.is_available() and torch.distributed.is_initialized():
            from .parallel.runtime import Coordinator
            store = torch.distributed.distributed_c10d._get_default_store()
            self.coord = Coordinator(store, rank, world_size, prefix=f"llmb/{os.environ.get('TORCHELASTIC_RUN_ID', 'job')}/trainer")
        self.zero = None
        if world_size > 1 or args.zero_stage > 0:
            from .parallel.zero import ZeroEngine
            self.zero = ZeroEngine(args.zero_stage, rank, world_size, self.device, dist_ctx=dist_ctx,
                                   backend=args.comm_backend)
        self.model = GPT2(args.load_filename, self.precision, self.device, zero=self.zero, recompute=args.recompute,
                          fp8_static_scales=args.fp8_static_scales or None)
        cfg = self.model.config
        if args.synthetic:
            self.train_loader = SyntheticLoader(B, T, cfg.vocab_size, rank)
            self.val_loader = None
        else:
            self.train_loader = DataLoader(resolve_data_files(args.train_data_pattern), B, T, rank, world_size,
                                           should_shuffle=True)
            self.val_loader = DataLoader(resolve_data_files(args.val_data_pattern), B, T, rank, world_size) \
                if args.val_data_pattern else None
        self.train_num_batches = args.max_steps if args.max_steps >= 0 else \
            self.train_loader.num_tokens // self.total_batch_size
        self.scheduler = LRScheduler(args.lr_scheduler_type, args.learning_rate, args.warmup_iterations,
                                     max(self.train_num_batches, 1), args.final_learning_rate_frac)
        self.tokenizer = Tokenizer(args.tokenizer_path) if os.path.exists(args.tokenizer_path) else Tokenizer()
        self.sampler_rng = SamplerRNG(1337)
        self.loss_outliers, self.norm_outliers = OutlierDetector(), OutlierDetector()
        self.ema = TokenRateEMA()
        self.tracer = TraceProfiler(pid=rank)
        self.step = 0
        self.last_norm = 0.0
        self._nanscan = os.environ.get("LLMM_DEBUG_TENSOR_NANSCAN", "") not in ("", "0")
        self._ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) \
            if self.device.type == "cuda" else None
        if args.resume and args.output_log_dir:
            s = ckpt.find_max_step(args.output_log_dir)
            if s >= 0:
                self.load(s)
        self.model.print_memory_report()

    # ------------------------------------------------------------------ one optimizer step
    def train_step(self, read_loss: bool = True) -> dict:
        """One optimizer step.  Returns loss / norm / lr / device_ms (CUDA events) / host ms."""
        a, m = self.args, self.model
        t0 = time.perf_counter()
        if self.coord is not None:
            self.coord.raise_if_aborted()               # a peer failed: stop before entering device-side waits
        if self._ev:
            self._ev[0].record()
        for micro in range(self.grad_accum):
            if a.overfit_single_batch and (self.step > 0 or micro > 0):
                x, y = self.train_loader.inputs, self.train_loader.targets
            else:
                x, y = self.train_loader.next_batch()
            last = micro == self.grad_accum - 1
            if not (last and a.overfit_single_batch):
                self.train_loader.prefetch()
            with self.tracer.cuda_span("forward"):
                m.forward(x, y, self.grad_accum, B=a.batch_size, T=a.seq_len,
                          on_inputs_copied=self.train_loader.mark_consumed)
            with self.tracer.cuda_span("backward"):
                m.backward(self.grad_accum, micro)
        if self._nanscan:                               # LLMM_DEBUG_TENSOR_NANSCAN=1: census of the accumulated gradients
            bad = m.debug_nan_scan("grads")
            if bad:
                print(f"step {self.step}: non-finite gradients (nan, inf): {bad}", flush=True)
        lr = self.scheduler.get_learning_rate(self.step)
        with self.tracer.cuda_span("grad_norm"):
            norm = m.calculate_grad_norm()
        scale = m.clip_scale_from_norm(norm, a.grad_clip) if a.grad_clip > 0 else None
        with self.tracer.cuda_span("update"):
            m.update(self.step + 1, lr, a.weight_decay, 1.0, a.beta1, a.beta2, a.eps, dev_scale=scale)
        if self._ev:
            self._ev[1].record()
        out = {"lr": lr, "step": self.step}
        if read_loss:
            loss = m.read_loss()                       # the step's only host synchronisation
            self._check_device_status()
            if self.zero is not None:
                loss = self.zero.mean_scalar(loss)
            out["loss"] = loss
            out["norm"] = float(norm.item())
            self.last_norm = out["norm"]
            if self._ev:
                out["device_ms"] = self._ev[0].elapsed_time(self._ev[1])
        out["ms"] = (time.perf_counter() - t0) * 1e3
        self.step += 1
        return out

    # ------------------------------------------------------------------ failure handling
    def _check_device_status(self) -> None:
        """Read the status word right after the loss (the stream is idle, so this is one 4-byte copy).  Non-zero:
        some bounded wait expired, i.e. a peer stalled or died and this step's reductions are not valid."""
        if self.device.type != "cuda":
            return
        from .ops import _lib
        status = _lib.read_status(self.device)
        if _lib.BOUNDS_CHECK:                      # checked build: data-dependent indices and scratch canaries
            from . import ops
            bad = _lib.bounds_report()
            if bad:
                self.abort(f"out-of-range index in step {self.step}: {bad}")
                raise _lib.KernelError(f"rank {self.rank}: out-of-range data-dependent index in step {self.step}: {bad}")
            ops.verify_scratch_canaries()
        if status == 0:
            return
        _lib.status_word(self.device).zero_()
        if self.zero is not None:
            self.zero.rearm_after_timeout()
        why = f"a bounded device wait expired in step {self.step} (status {status})"
        self.abort(why)
        raise DeviceWaitExpired(f"rank {self.rank}: {why}")

    def abort(self, reason: str) -> None:
        """Make every peer's next step / barrier raise ``PeerAborted``."""
        if self.coord is not None:
            self.coord.abort(reason)

    def host_barrier(self) -> None:
        """Ranks meet on the host (sticky-abort barrier) after a phase of uneven host work."""
        if self.coord is not None:
            if self.device.type == "cuda":
                torch.cuda.synchronize(self.device)
            self.coord.barrier()

    # ------------------------------------------------------------------ evaluation / sampling
    @torch.no_grad()
    def validate(self) -> float:
        a, m = self.args, self.model
        if self.val_loader is None:
            return float("nan")
        self.val_loader.reset()
        n = min(a.val_max_steps, max(1, self.val_loader.num_tokens // (a.batch_size * a.seq_len * self.world_size)))
        m.loss_acc.zero_()
        for _ in range(n):
            x, y = self.val_loader.next_batch()
            m.forward(x, y, n, B=a.batch_size, T=a.seq_len, on_inputs_copied=self.val_loader.mark_consumed)
        loss = m.read_loss()
        self._check_device_status()
        return self.zero.mean_scalar(loss) if self.zero is not None else loss

    @torch.no_grad()
    def sample(self, gen_tokens: int) -> List[int]:
        """Autoregressive sampling by re-running the forward pass per token, as the reference
        trainer does (``train_gpt2.mojo:6427-6465``); every rank runs it so collectives line up."""
        a, m = self.args, self.model
        B, T = a.batch_size, a.seq_len
        toks = torch.full((B, T), self.tokenizer.eot_token, dtype=torch.int32)
        V = m.config.vocab_size
        out = []
        for t in range(1, min(gen_tokens, T)):
            m.forward(toks, None, B=B, T=T)
            logits = m.acts["logits"][0, t - 1, :V].float().cpu().numpy()
            nxt = sample_softmax(logits, self.sampler_rng.random_f32())
            toks[0, t] = nxt
            out.append(nxt)
        return out

    # ------------------------------------------------------------------ checkpoints
    def save(self, step: int) -> None:
        a = self.args
        os.makedirs(a.output_log_dir, exist_ok=True)
        st = self.train_loader.state()
        state = ckpt.TrainingState(step=step, num_processes=self.world_size, process_rank=self.rank,
                                   should_shuffle=st["should_shuffle"], sampler_rng_state=self.sampler_rng.state,
                                   shuffle_rng_state=st["shuffle_draws"], current_shard_idx=st["current_shard_idx"],
                                   current_sample_idx=st["current_sample_idx"])
        self.model.write_checkpoint(ckpt.model_path(a.output_log_dir, step),
                                    ckpt.state_path(a.output_log_dir, step, self.rank), state, self.rank)

    def load(self, step: int) -> None:
        a = self.args
        state = self.model.load_checkpoint(ckpt.model_path(a.output_log_dir, step),
                                           ckpt.state_path(a.output_log_dir, step, self.rank))
        if state.num_processes != self.world_size or state.process_rank != self.rank:
            raise ValueError("Checkpoint error: state was written with a different world size / rank")
        self.train_loader.restore(state.should_shuffle, state.shuffle_rng_state, state.current_shard_idx,
                                  state.current_sample_idx)
        self.sampler_rng.state = state.sampler_rng_state
        self.step = state.step

    # ------------------------------------------------------------------ the loop
    def print0(self, *a, **k) -> None:
        if self.rank == 0:
            print(*a, **k, flush=True)

    def train(self) -> None:
        a, m = self.args, self.model
        cfg = m.config
        dev_name = torch.cuda.get_device_name(self.device) if self.device.type == "cuda" else "cpu"
        self.print0(f"| model {a.load_filename} | params {m.num_parameters:,} | L {cfg.num_layer} NH {cfg.num_heads} "
                    f"C {cfg.channels} | B {a.batch_size} T {a.seq_len} | grad_accum {self.grad_accum} "
                    f"| world {self.world_size} | zero {a.zero_stage} | precision {self.precision.name} | {dev_name} |")
        N = self.train_num_batches
        while self.step <= N:
            step, last = self.step, self.step == N
            if a.val_loss_every > 0 and (step % a.val_loss_every == 0 or last) and self.val_loader is not None:
                self.print0(f"val loss {self.validate():.6f}")
                self.host_barrier()
            if a.sample_every > 0 and (step > 0 and step % a.sample_every == 0 or last):
                ids = self.sample(a.gen_tokens)
                self.print0("generating:\n---")
                self.print0(self.tokenizer.decode_sequence(ids) if self.tokenizer.has_initialized
                            else " ".join(str(i) for i in ids))
                self.print0("---")
                self.host_barrier()
            if a.checkpoint_every > 0 and a.output_log_dir and ((step > 0 and step % a.checkpoint_every == 0) or last):
                self.save(step)
                self.print0(f"Writing checkpoint at step {step}")
                self.host_barrier()                     # rank 0 writes the whole model; the others wait here, not on the device
            if last:
                break
            r = self.train_step()
            ms = r.get("device_ms", r["ms"])
            tok_s = self.total_batch_size / (r["ms"] / 1e3)
            ema = self.ema.update(tok_s) if step > 0 else tok_s
            mfu = estimate_mfu(m.num_parameters, cfg.num_layer, cfg.channels, a.seq_len,
                               self.total_batch_size // self.world_size, r["ms"] / 1e3, dev_name, self.precision.name)
            zl, zn = self.loss_outliers.update(r["loss"]), self.norm_outliers.update(r["norm"])
            self.print0(format_step_line(step + 1, N, r["loss"], zl, r["norm"], zn, r["lr"], r["ms"], mfu,
                                         self.precision.name, ema, r.get("device_ms")))
        self.tracer.flush()
