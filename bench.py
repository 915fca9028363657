#!/usr/bin/env python
"""Headline benchmark: GPT-2 124M bf16 training throughput (tokens/s) on N B200s of one node.

Config (the reference's headline setup): d12 (L=12, NH=12, C=768, padded vocab 50304), micro-batch
B=64, T=1024, 2**19 tokens per optimizer step through gradient accumulation, DDP (-z 0), AdamW
lr 6e-4 with warmup + cosine decay, grad clip 1.0, fp32 master weights, random-init weights and
synthetic uniform tokens.  The global batch is fixed, so per-GPU work shrinks with N ("strong").

Prints ONE JSON line on rank 0.  `value` is device-timed (CUDA events, max over ranks) with the
tokens already resident on the GPU; `e2e` runs the same steps through the public `Trainer` API
with the per-step pinned-host→device token copies and the device→host loss read inside the
timed region.  `--impl reference` is the reference arm: it runs the reference's own PyTorch trainer
(`train_gpt2.py`, NCCL DDP + cuBLAS + SDPA + fused AdamW; its Mojo trainer needs a compiler that is not
available) unmodified from `baseline/_ref` as a child process of every rank, on the same model,
batch and optimizer settings, and reads the step times that trainer prints.  `--impl torch` is a
plain PyTorch comparator built on this package's own model code, for on-box context only.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import shutil
import subprocess
import sys
import tempfile
import threading
import time

BASELINE_TOK_S_PER_GPU = 173010.0      # reference's best published per-GPU bf16 124M number (B=64, T=1024)
ROOT = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(ROOT, "baseline", "_ref")
REF_TOKENIZER_STANDIN = os.path.join(ROOT, "baseline", "tokenizer_standin")
METRIC = "GPT-2 124M train tokens/sec (device-timed, max over ranks)"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "torch"])
    ap.add_argument("--model", default="d12")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--total-batch", type=int, default=2 ** 19)
    ap.add_argument("--zero", type=int, default=0)
    ap.add_argument("--no-e2e", action="store_true")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows, self.proc, self.gpu = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm = sorted(float(r[1]) for r in self.rows if len(r) > 8 and r[1].replace(".", "").isdigit())
        mx = [float(r[2]) for r in self.rows if len(r) > 8 and r[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) > 8 for n, v in zip(names, r[5:9]) if v.lower() == "active"})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    from llm_mojo_b200 import ops
    from llm_mojo_b200.trainer import TrainArgs, Trainer

    targs = TrainArgs(load_filename=args.model, batch_size=args.batch, seq_len=args.seq,
                      total_batch_size=args.total_batch, learning_rate=6e-4, lr_scheduler_type="cosine",
                      warmup_iterations=10, final_learning_rate_frac=0.1, weight_decay=0.1, zero_stage=args.zero,
                      max_steps=10_000, precision="bf16", grad_clip=1.0, beta2=0.95, synthetic=True,
                      val_loss_every=0, sample_every=0, comm_backend=os.environ.get("LLMB_COMM", "auto"))
    tr = Trainer(targs, rank, world, local_rank)
    model, B, T = tr.model, args.batch, args.seq
    ga = tr.grad_accum

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---------------- kernel-only region: tokens already on the device
    gen = torch.Generator(device="cuda").manual_seed(1234 + rank)
    toks = torch.randint(0, model.config.vocab_size, (B * T + 1,), generator=gen, device="cuda", dtype=torch.int32)
    x_dev, y_dev = toks[:-1].view(B, T).contiguous(), toks[1:].view(B, T).contiguous()

    def device_step(step):
        for micro in range(ga):
            model.forward(x_dev, y_dev, ga, B=B, T=T)
            model.backward(ga, micro)
        norm = model.calculate_grad_norm()
        scale = model.clip_scale_from_norm(norm, 1.0)
        model.update(step + 1, tr.scheduler.get_learning_rate(step), 0.1, 1.0, 0.9, 0.95, 1e-8, dev_scale=scale)

    for s in range(args.warmup):
        device_step(s)
    barrier()
    model.read_loss()                      # reset the on-device loss accumulator
    sampler = ClockSampler(torch.cuda.current_device())
    if rank == 0:
        sampler.start()
    launches0 = ops.LAUNCHES
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    h0 = time.perf_counter()
    for s in range(args.steps):
        device_step(args.warmup + s)
    host_enqueue_ms = (time.perf_counter() - h0) * 1e3      # host time to enqueue the timed steps (no sync inside)
    e1.record()
    barrier()
    dev_ms = e0.elapsed_time(e1)
    launches = ops.LAUNCHES - launches0
    clocks = sampler.stop() if rank == 0 else None
    final_loss = model.read_loss() / args.steps      # mean over the timed steps
    status = ops._lib.read_status()

    # ---------------- end-to-end region through Trainer.train_step (H2D tokens + D2H loss per step)
    e2e_ms = None
    if not args.no_e2e:
        tr.step = args.warmup + args.steps
        for _ in range(min(2, args.warmup)):
            tr.train_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            r = tr.train_step()          # reads the loss (D2H) every step
        barrier()
        e2e_ms = (time.perf_counter() - t0) * 1e3
        final_loss = r["loss"]

    t = torch.tensor([dev_ms, e2e_ms or 0.0], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms_max = t.tolist()
    tokens = args.total_batch * args.steps
    value = tokens / (dev_ms / 1e3)
    out = {
        "metric": METRIC, "value": value, "unit": "tok/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": value / (BASELINE_TOK_S_PER_GPU * world),
        "dtype": "bf16", "data": "synthetic uniform tokens, random-init weights", "impl": "ours",
        "config": {"model": f"gpt2-124M ({args.model})", "global_batch": args.total_batch // args.seq, "seq_len": args.seq,
                   "micro_batch": B, "grad_accum": ga, "tokens_per_step": args.total_batch,
                   "parallelism": f"dp{world}" + (f"+zero{args.zero}" if args.zero else ""),
                   "optimizer": "AdamW lr 6e-4 warmup+cosine, clip 1.0, fp32 master",
                   "l2": "inputs larger than L2 (per-layer activations 100-400 MB, logits 6.6 GB)"},
        "clocks": clocks, "gpu_launches": launches, "final_loss": final_loss, "kernel_status": status,
        "gemm_impl": ops.GEMM_IMPL, "attn_impl": ops.ATTN_IMPL, "host_enqueue_ms_per_step": host_enqueue_ms / args.steps,
        "comm_backend": (tr.zero.backend_name if tr.zero is not None else "none (one GPU)"),
    }
    if e2e_ms_max:
        h2d = 2 * B * T * 4 * ga          # inputs + targets, int32, per step per rank
        out["e2e"] = {"value": tokens / (e2e_ms_max / 1e3), "unit": "tok/s", "h2d_bytes_per_step": h2d * world,
                      "d2h_bytes_per_step": 8 * world, "ms_per_step": e2e_ms_max / args.steps,
                      "api": "llm_mojo_b200.trainer.Trainer.train_step"}
    return out


_REF_STEP = re.compile(r"step\s+(\d+)/(\d+) \| train loss ([0-9.naif+-]+) \|.*\(([0-9.]+) ms \| ([0-9.]+) tok/s\)")


def run_reference(args, rank, world, local_rank):
    """Reference arm: the reference's own trainer, unmodified, as a child process of this rank.

    The child is `baseline/_ref/train_gpt2.py` (a plain copy of the reference tree; it has no
    setup.py, so a copy is its install) with the flags of the headline config: d12, B=64, T=1024,
    2**19 tokens per step, bf16 autocast, SDPA flash attention, DDP (`--zero_stage 0`), AdamW
    lr 6e-4 / wd 0.1 / betas (0.9, 0.95), warm-up + cosine, clip 1.0, sampling / validation /
    tensor dumps off.  Under torchrun every rank starts one child, which inherits RANK / LOCAL_RANK /
    WORLD_SIZE / MASTER_* and joins the NCCL group itself (`train_gpt2.py:1886`).  Tokens come from a
    synthetic uniform shard in the reference's own .bin format, long enough that the loader never
    reloads it inside the run.  The trainer builds the GPT-2 tiktoken encoding at start-up, which
    needs a download; the directory `baseline/tokenizer_standin` (first on the child's PYTHONPATH)
    supplies an encoding of the same size instead - it is never used to tokenize in this run.

    `value` is computed from the step times the trainer prints (host clock around the whole step,
    closed by `torch.cuda.synchronize()`, `train_gpt2.py:2316-2330`; rank 0 cannot finish a step
    before the gradient all-reduce has seen every rank, so its time is the max over ranks).  `e2e`
    is the wall clock this process sees between the arrival of two step lines, so it also contains
    the loader, the host-to-device token copies and the loss read of every step.
    """
    import numpy as np
    script = os.path.join(REF_DIR, "train_gpt2.py")
    if not os.path.exists(script):
        return {"impl": "reference", "unavailable": "baseline/_ref/train_gpt2.py is missing (copy the reference tree there)"}
    B, T, K, W = args.batch, args.seq, args.steps, args.warmup
    if args.total_batch % (B * T * world):
        return {"impl": "reference", "unavailable": f"total batch {args.total_batch} not divisible by {B}x{T}x{world}"}
    ga = args.total_batch // (B * T * world)
    work = tempfile.mkdtemp(prefix=f"refarm_r{rank}_")
    try:
        from llm_mojo_b200.utils.dataloader import write_datafile
        ntok = min((K + W) * args.total_batch + B * T * world + 1, 2 ** 28)
        shard = os.path.join(work, "synthetic_uniform.bin")
        write_datafile(shard, np.random.default_rng(1234).integers(0, 50257, size=ntok, dtype=np.uint16))
        cmd = [sys.executable, "-u", script, "--model", args.model, "--batch_size", str(B), "--sequence_length", str(T),
               "--total_batch_size", str(args.total_batch), "--dtype", "bfloat16", "--flash", "1", "--zero_stage", "0",
               "--learning_rate", "6e-4", "--warmup_iters", "10", "--learning_rate_decay_frac", "0.1",
               "--weight_decay", "0.1", "--grad_clip", "1.0", "--sample_every", "0", "--val_loss_every", "0",
               "--write_tensors", "0", "--compile", os.environ.get("BENCH_REF_COMPILE", "0"),
               "--num_iterations", str(K + W), "--input_bin", shard, "--input_val_bin", ""]
        env = dict(os.environ)
        env["PYTHONPATH"] = os.pathsep.join([REF_TOKENIZER_STANDIN] + ([env["PYTHONPATH"]] if env.get("PYTHONPATH") else []))
        env.setdefault("MASTER_ADDR", "127.0.0.1")
        sampler = ClockSampler(local_rank)
        child = subprocess.Popen(cmd, cwd=work, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        steps, arrival, tail = [], [], []
        for line in child.stdout:
            tail = (tail + [line.rstrip()])[-12:]
            m = _REF_STEP.search(line)
            if m:
                steps.append((int(m.group(1)), float(m.group(3)), float(m.group(4))))
                arrival.append(time.perf_counter())
                if len(steps) == W and rank == 0:
                    sampler.start()
        rc = child.wait()
        clocks = sampler.stop() if (rank == 0 and sampler.proc is not None) else None
        if rank != 0:
            return None
        if rc != 0 or len(steps) < K + W:
            why = next((l for l in reversed(tail) if "Error" in l or "error" in l), tail[-1] if tail else "no output")
            return {"impl": "reference", "unavailable": f"train_gpt2.py exited {rc} after {len(steps)} of {K + W} steps: {why[:300]}"}
        timed = steps[W:W + K]
        ms = sum(t[2] for t in timed)
        e2e_ms = (arrival[W + K - 1] - arrival[W - 1]) * 1e3 if W >= 1 else ms
        tokens = args.total_batch * K
        value = tokens / (ms / 1e3)
        return {
            "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": value / (BASELINE_TOK_S_PER_GPU * world), "dtype": "bf16",
            "data": "synthetic uniform tokens (reference .bin shard), random-init weights", "impl": "reference",
            "config": {"model": f"gpt2-124M ({args.model})", "global_batch": args.total_batch // T, "seq_len": T,
                       "micro_batch": B, "grad_accum": ga, "tokens_per_step": args.total_batch, "parallelism": f"dp{world}",
                       "optimizer": "AdamW (fused) lr 6e-4 warmup+cosine, clip 1.0, fp32 params under bf16 autocast",
                       "l2": "inputs larger than L2 (per-layer activations 100-400 MB, logits 6.6 GB)"},
            "same_config": True, "clocks": clocks, "gpu_launches": None, "final_loss": timed[-1][1],
            "code": "baseline/_ref/train_gpt2.py (unmodified), torch.compile " +
                    ("on" if os.environ.get("BENCH_REF_COMPILE", "0") == "1" else "off (its default)"),
            "timing": "the trainer's own per-step host clock closed by torch.cuda.synchronize(); rank 0's steps end after the "
                      "gradient all-reduce, i.e. at the max over ranks",
            "tokenizer": "stand-in tiktoken_ext.openai_public on PYTHONPATH (no network for vocab.bpe); unused in the run",
            "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": "tok/s", "ms_per_step": e2e_ms / K,
                    "h2d_bytes_per_step": 2 * B * T * 8 * ga * world, "d2h_bytes_per_step": 8 * world,
                    "api": "train_gpt2.py command line; wall clock between its step lines (loader + H2D + step + loss read)"},
        }
    finally:
        shutil.rmtree(work, ignore_errors=True)


def run_torch(args, rank, world, local_rank):
    """PyTorch comparator: autograd GPT-2 (cuBLAS GEMMs, SDPA flash attention, fused AdamW, NCCL DDP)."""
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F
    from llm_mojo_b200.config import parse_model_descriptor
    from llm_mojo_b200.models import random_init_params
    from llm_mojo_b200.models.reference import unflatten

    cfg = parse_model_descriptor(args.model)
    dev = torch.device("cuda", local_rank)
    flat = random_init_params(cfg).to(dev)
    names = unflatten(cfg, flat)
    params = {k: torch.nn.Parameter(v.clone()) for k, v in names.items()}
    B, T, C, NH, L, V = args.batch, args.seq, cfg.channels, cfg.num_heads, cfg.num_layer, cfg.vocab_size
    ga = args.total_batch // (B * T * world)
    opt = torch.optim.AdamW(params.values(), lr=6e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)

    def fwd(x, y):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            h = params["wte"][x] + params["wpe"][:T]
            for l in range(L):
                a = F.layer_norm(h, (C,), params["ln1w"][l], params["ln1b"][l])
                qkv = F.linear(a, params["qkvw"][l], params["qkvb"][l])
                q, k, v = (t.view(B, T, NH, C // NH).transpose(1, 2) for t in qkv.split(C, dim=2))
                o = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, T, C)
                h = h + F.linear(o, params["attprojw"][l], params["attprojb"][l])
                a = F.layer_norm(h, (C,), params["ln2w"][l], params["ln2b"][l])
                a = F.gelu(F.linear(a, params["fcw"][l], params["fcb"][l]), approximate="tanh")
                h = h + F.linear(a, params["fcprojw"][l], params["fcprojb"][l])
            h = F.layer_norm(h, (C,), params["lnfw"], params["lnfb"])
            logits = F.linear(h, params["wte"])
        return F.cross_entropy(logits[..., :V].reshape(-1, V).float(), y.reshape(-1))

    gen = torch.Generator(device="cuda").manual_seed(1234 + rank)
    toks = torch.randint(0, V, (B * T + 1,), generator=gen, device="cuda")
    x, y = toks[:-1].view(B, T), toks[1:].view(B, T)

    def step():
        opt.zero_grad(set_to_none=True)
        for _ in range(ga):
            (fwd(x, y) / ga).backward()
        if world > 1:
            for p in params.values():
                dist.all_reduce(p.grad)
                p.grad /= world
        torch.nn.utils.clip_grad_norm_(params.values(), 1.0)
        opt.step()

    for _ in range(args.warmup):
        step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = t.item()
    value = args.total_batch * args.steps / (ms / 1e3)
    return {"metric": METRIC, "value": value, "unit": "tok/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": value / (BASELINE_TOK_S_PER_GPU * world),
            "dtype": "bf16", "data": "synthetic uniform tokens, random-init weights", "impl": "torch",
            "config": {"model": f"gpt2-124M ({args.model})", "seq_len": T, "micro_batch": B, "grad_accum": ga,
                       "tokens_per_step": args.total_batch, "parallelism": f"dp{world}"}}


def main():
    args = parse()
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", rank))
    if args.impl == "reference":
        # no CUDA context and no process group here: the reference's trainer, started as a child, owns both
        try:
            import torch
            if torch.cuda.device_count() == 0 and args.total_batch > (1 << 16):   # counting devices creates no context
                # the reference's trainer does run on a CPU, and the tests use that with a tiny batch; the headline config would take hours
                out = {"impl": "reference", "unavailable": "no CUDA device"}
            else:
                out = run_reference(args, rank, world, local_rank)
        except Exception as e:                                        # the arm never fails the driver's run
            out = {"impl": "reference", "unavailable": f"{type(e).__name__}: {e}"[:300]}
        if rank == 0:
            print(json.dumps(out), flush=True)
        return 0
    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        if rank == 0:
            print(json.dumps({"impl": args.impl, "unavailable": "no CUDA device"}), flush=True)
        return 0
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        out = run_ours(args, rank, world, local_rank) if args.impl == "ours" else run_torch(args, rank, world, local_rank)
        if rank == 0:
            print(json.dumps(out), flush=True)
    finally:
        if world > 1:
            dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
