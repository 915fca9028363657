"""GPT-2 over flat buffers with explicit forward / backward / update.

Parity: ``train_gpt2.mojo:1189-1653`` (GPT2 struct and its three load paths), ``:3050-3848``
(forward), ``:3948-5056`` (backward), ``:5058-5259`` (update), ``:5261-5383`` (grad norm),
``:5615-5801`` (checkpoint glue), ``:5807-6011`` (memory report).

B200-first differences: one process per GPU; parameters are one flat tensor in the storage
dtype with an fp32 master copy, gradients are one flat **fp32** tensor (cast to bf16 only on
the wire); attention never materialises ``[T,T]``; the residual adds are fused into the
attn-proj / fc-proj GEMM epilogues; the clip factor stays on the device so an optimizer step
needs no host round trip.  Distributed behaviour (DDP / ZeRO-1/2/3) is delegated to a
``ZeroEngine`` (``parallel/zero.py``) through four hooks: ``before_layer``,
``grads_ready``, ``reduce_all`` and ``optimizer_step``.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Tuple

import torch

from .. import ops
from ..config import (GPT2Config, INIT_RNG_SEED, INIT_WEIGHT_STD, PARAM_NAMES, Precision,
                      is_model_descriptor, parse_model_descriptor)
from ..utils import checkpointing as ckpt
from ..utils.rand import MT19937, normal_

LAYER_TENSORS = ("ln1w", "ln1b", "qkvw", "qkvb", "attprojw", "attprojb", "ln2w", "ln2b",
                 "fcw", "fcb", "fcprojw", "fcprojb")


def random_init_params(config: GPT2Config, seed: int = INIT_RNG_SEED) -> torch.Tensor:
    """Flat fp32 parameter vector with the llm.c / PyTorch-compatible random init
    (``train_gpt2.mojo:2060-2160``): draws are layer-outer, tensor-inner from MT19937 +
    Box-Muller; N(0, 0.02), residual projections scaled by 1/sqrt(2L), LN gamma 1, rest 0."""
    L, C, V = config.num_layer, config.channels, config.vocab_size
    sizes = config.param_sizes()
    offsets = [0]
    for s in sizes:
        offsets.append(offsets[-1] + s)
    flat = torch.zeros(offsets[-1], dtype=torch.float32)
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)            # torch's CPU generator *is* MT19937; normal_ matches llmm/rand.mojo:162

    def draw(n: int, std: float) -> torch.Tensor:
        return torch.empty(n, dtype=torch.float32).normal_(0.0, std, generator=g)

    residual_scale = 1.0 / math.sqrt(2.0 * L)
    for l in range(L):
        for i, name in enumerate(PARAM_NAMES):
            off, n = offsets[i], sizes[i]
            if l == 0 and name in ("ln1w", "ln2w", "lnfw"):
                flat[off:off + n] = 1.0
            if l == 0 and name == "wte":
                flat[off:off + V * C] = draw(V * C, INIT_WEIGHT_STD)
            elif l == 0 and name == "wpe":
                flat[off:off + n] = draw(n, INIT_WEIGHT_STD)
            elif name in ("qkvw", "attprojw", "fcw", "fcprojw"):
                per = n // L
                std = INIT_WEIGHT_STD * (residual_scale if name in ("attprojw", "fcprojw") else 1.0)
                flat[off + l * per: off + (l + 1) * per] = draw(per, std)
    return flat


class GPT2:
    def __init__(self, source: str | GPT2Config, precision: Precision | str = "bf16",
                 device: str | torch.device = "cpu", zero=None, recompute: bool = False,
                 init_seed: int = INIT_RNG_SEED, params_flat: Optional[torch.Tensor] = None,
                 lm_head_chunks: Optional[int] = None, vocab_parallel: Optional[bool] = None,
                 fp8_static_scales=None):
        self.precision = precision if isinstance(precision, Precision) else Precision(precision)
        self.device = torch.device(device)
        self.recompute = recompute or os.environ.get("LLMM_RECOMPUTE", "") not in ("", "0")
        self.zero = zero
        # LM-head vocabulary tiling with chunked cross-entropy: K > 1 never materialises [B,T,Vp] logits
        # (train_gpt2.mojo:127-149 LM_HEAD_VOCAB_TILES / LM_HEAD_CHUNKED_CE; README.md:145-149)
        self.lm_head_chunks = int(os.environ.get("LLMM_LM_HEAD_CHUNKS", 1)) if lm_head_chunks is None else lm_head_chunks
        # Vocabulary-parallel LM head: every rank holds the logits of ALL ranks' rows for its 1/W slice of the
        # vocabulary (activation all-gather -> slice GEMM -> cross-entropy with the log-sum-exp merged across
        # ranks -> reduce-scatter of the hidden-state gradient).  The reference evaluated and rejected this on
        # PCIe (README.md:153); it needs a ZeRO engine with world_size > 1.  Under ZeRO-3 the slice is a view of the
        # gathered embedding window, which the token embedding needs in full anyway.
        vp = os.environ.get("LLMM_VOCAB_PARALLEL", "") not in ("", "0") if vocab_parallel is None else vocab_parallel
        self.vocab_parallel = bool(vp and zero is not None and zero.world_size > 1)
        self.checkpoint_path = source if isinstance(source, str) else ""
        # ---- three load paths: config/descriptor (random init), .bin, .safetensors
        if params_flat is not None:
            assert isinstance(source, GPT2Config)
            self.config = source
            flat = params_flat.float()
        elif isinstance(source, GPT2Config):
            self.config = source
            flat = random_init_params(self.config, init_seed)
        elif is_model_descriptor(source):
            self.config = parse_model_descriptor(source)
            flat = random_init_params(self.config, init_seed)
        elif source.endswith(".safetensors"):
            from ..utils.safetensors_io import load_hf_gpt2
            self.config, flat = load_hf_gpt2(source)
        else:
            self.config, _, flat = ckpt.read_model_checkpoint(source, dtype=torch.float32)
        cfg = self.config
        if self.device.type == "cpu" and self.precision.storage != torch.float32:
            raise ValueError("CPU training is fp32 by policy; use precision='fp32'")
        self.dtype = self.precision.storage
        self.param_sizes = cfg.param_sizes()
        self.param_shapes = cfg.param_shapes()
        self.num_parameters = sum(self.param_sizes)
        self.param_offsets = [0]
        for s in self.param_sizes:
            self.param_offsets.append(self.param_offsets[-1] + s)

        if self.zero is not None:
            self.params = self.grads = self.m = self.v = self.master = None
            self.p, self.g = {}, {}
            self.zero.attach(self, flat)           # allocates (possibly sharded) buffers and installs the views
        else:
            self.params = flat.to(self.device, self.dtype)
            self.grads = torch.zeros(self.num_parameters, dtype=torch.float32, device=self.device)
            self.m = torch.zeros(self.num_parameters, dtype=torch.float32, device=self.device)
            self.v = torch.zeros(self.num_parameters, dtype=torch.float32, device=self.device)
            self.master = flat.to(self.device, torch.float32).clone() if self.precision.use_master else None
            self.p = self._views(self.params)
            self.g = self._views(self.grads)
        del flat
        self.B = self.T = 0
        self.acts: Dict[str, torch.Tensor] = {}
        self.mean_loss = -1.0
        self.loss_acc = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.norm_sq = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.clip_scale = torch.ones(1, dtype=torch.float32, device=self.device)
        self.inputs_dev: Optional[torch.Tensor] = None
        self.targets_dev: Optional[torch.Tensor] = None
        self.rng_seed = 1337
        self.use_stochastic_rounding = False
        self.micro_steps_done = 0
        self.lowp = None
        if self.precision.name == "fp8":
            from ..ops.lowp import LowpState
            self.lowp = LowpState(cfg.num_layer, self.device)
            table = fp8_static_scales or os.environ.get("LLMM_FP8_STATIC_SCALES", "")
            if table:      # calibrated constants instead of delayed scaling: no amax / scale-update kernels in the step
                self.lowp.set_static_scales(LowpState.read_scale_table(table) if isinstance(table, str) else table)

    # ------------------------------------------------------------------ views / layout
    def _views(self, flat: torch.Tensor) -> Dict[str, torch.Tensor]:
        return {n: flat[self.param_offsets[i]:self.param_offsets[i + 1]].view(self.param_shapes[i])
                for i, n in enumerate(PARAM_NAMES)}

    def tensor_range(self, name: str, layer: Optional[int] = None) -> Tuple[int, int]:
        """[begin, end) of a tensor (or of one layer's slice of it) in the flat vector."""
        i = PARAM_NAMES.index(name)
        off, n = self.param_offsets[i], self.param_sizes[i]
        if layer is None:
            return off, off + n
        per = n // self.config.num_layer
        return off + layer * per, off + (layer + 1) * per

    def layer_ranges(self, layer: int) -> List[Tuple[int, int]]:
        """The 12 (offset, end) ranges of one transformer block (the per-layer gradient bucket
        and ZeRO-3 window of ``train_gpt2.mojo:1856-1940`` / ``:4921-4929``)."""
        return [self.tensor_range(n, layer) for n in LAYER_TENSORS]

    # ------------------------------------------------------------------ activations
    def allocate_activations(self, B: int, T: int) -> None:
        cfg, dev, dt = self.config, self.device, self.dtype
        L, C, NH, Vp = cfg.num_layer, cfg.channels, cfg.num_heads, cfg.padded_vocab_size
        if T > cfg.max_seq_len:
            raise ValueError(f"sequence length {T} exceeds max_seq_len {cfg.max_seq_len}")
        f32 = torch.float32

        def e(*shape, dtype=dt):
            return torch.empty(*shape, dtype=dtype, device=dev)

        a = {
            "encoded": e(B, T, C),
            "ln1": e(L, B, T, C), "ln1_mean": e(L, B, T, dtype=f32), "ln1_rstd": e(L, B, T, dtype=f32),
            "qkv": e(L, B, T, 3 * C), "atty": e(L, B, T, C), "lse": e(L, B, NH, T, dtype=f32),
            "residual2": e(L, B, T, C),
            "ln2": e(L, B, T, C), "ln2_mean": e(L, B, T, dtype=f32), "ln2_rstd": e(L, B, T, dtype=f32),
            "fch": e(L, B, T, 4 * C),
            "fch_gelu": e(1 if self.recompute else L, B, T, 4 * C),
            "residual3": e(L, B, T, C),
            "lnf": e(B, T, C), "lnf_mean": e(B, T, dtype=f32), "lnf_rstd": e(B, T, dtype=f32),
            "losses": e(B, T, dtype=f32),
            # backward scratch
            "dres": e(B, T, C), "dl_btc": e(B, T, C), "dl_bt4c": e(B, T, 4 * C),
        }
        self._fused_gather = None
        if self.vocab_parallel:
            W = self.zero.world_size
            self.vslice = ((Vp + W - 1) // W + 7) // 8 * 8
            a["logits_slice"] = e(W * B * T, self.vslice)
            a["ce_stats"] = e(W * B * T, 4, dtype=f32)
            # all-gather of the final LayerNorm rows fused into the slice GEMM (peer memory; bf16 tensor path, whole
            # 256-row tiles per rank); LLMM_FUSED_GATHER=0 keeps the collective + GEMM pair
            # (every rank must own at least 8 vocabulary columns: the peer-memory path is collective)
            if (self.device.type == "cuda" and self.dtype == torch.bfloat16 and (B * T) % 256 == 0 and
                    Vp - (W - 1) * self.vslice >= 8 and
                    getattr(self.zero, "backend_name", "") == "p2p" and os.environ.get("LLMM_FUSED_GATHER", "1") != "0"):
                from ..parallel.zero import FusedRowGather
                self._fused_gather = FusedRowGather(self.zero.rank, W, self.device, B * T, C)
                a["lnf"] = self._fused_gather.local.view(B, T, C)
        elif self.lm_head_chunks > 1:
            self.tile_width = ((Vp + self.lm_head_chunks - 1) // self.lm_head_chunks + 127) // 128 * 128
            a["logits_tile"] = e(B * T, self.tile_width)
            a["ce_stats"] = e(B * T, 4, dtype=f32)
        else:
            a["logits"] = e(B, T, Vp)
        self.acts = a
        self.B, self.T = B, T
        self.inputs_dev = torch.empty(B, T, dtype=torch.int32, device=dev)
        self.targets_dev = torch.empty(B, T, dtype=torch.int32, device=dev)

    def activation_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.acts.values())

    def _vocab_slice(self):
        z, Vp = self.zero, self.config.padded_vocab_size
        v0 = min(z.rank * self.vslice, Vp)
        return v0, min(self.vslice, Vp - v0)

    def _vocab_parallel_forward(self, p, dloss) -> None:
        a, z, V = self.acts, self.zero, self.config.vocab_size
        B, T, C = self.B, self.T, self.config.channels
        rows = B * T
        self._tgt_all = z.all_gather_rows(self.targets_dev.view(rows))
        v0, w = self._vocab_slice()
        tile = a["logits_slice"][:, :max(w, 8)]
        stats = a["ce_stats"]
        fg = self._fused_gather
        if fg is not None:
            # peer-memory path: this slice's statistics go into the symmetric buffer, ONE kernel merges all ranks' copies
            fg.stats_writable()
            fg.gemm(tile, p["wte"][v0:v0 + w])              # the other ranks' rows are pulled over NVLink inside the slice GEMM
            self._lnf_all = fg.buf
            ops.chunked_ce_pass1(fg.stats, tile, self._tgt_all, v0, w, V, True)
            fg.merge_stats(stats)
            losses_all = torch.empty(stats.shape[0], dtype=torch.float32, device=stats.device)
            ops.chunked_ce_loss(losses_all, stats)
            a["losses"].view(-1).copy_(losses_all[z.rank * rows:(z.rank + 1) * rows])
            self.loss_acc += a["losses"].sum() * dloss
            return
        self._lnf_all = z.all_gather_rows(a["lnf"].view(rows, C))
        if w > 0:
            ops.matmul_fwd(tile, self._lnf_all, p["wte"][v0:v0 + w])
        ops.chunked_ce_pass1(stats, tile, self._tgt_all, v0, w, V, True)
        # merge (max, sum-exp, target logit) over the vocabulary slices of all ranks
        allst = z.all_gather_rows(stats.unsqueeze(0))                      # [W, W·rows, 4]
        m = allst[:, :, 0].max(dim=0).values
        ssum = (allst[:, :, 1] * torch.exp(allst[:, :, 0] - m)).nan_to_num(0.0).sum(dim=0)
        stats[:, 0], stats[:, 1], stats[:, 2] = m, ssum, allst[:, :, 2].sum(dim=0)
        losses_all = torch.empty(stats.shape[0], dtype=torch.float32, device=stats.device)
        ops.chunked_ce_loss(losses_all, stats)
        a["losses"].view(-1).copy_(losses_all[z.rank * rows:(z.rank + 1) * rows])
        self.loss_acc += a["losses"].sum() * dloss

    def _vocab_parallel_backward(self, p, g, dl) -> None:
        a, z, V = self.acts, self.zero, self.config.vocab_size
        C = self.config.channels
        v0, w = self._vocab_slice()
        tile = a["logits_slice"][:, :max(w, 8)]
        n_all = tile.shape[0]
        partial = ops.scratch("vp_dlnf", n_all * C * a["lnf"].element_size(), tile.device).view(a["lnf"].dtype)[:n_all * C].view(n_all, C)
        fg = self._fused_gather
        if fg is not None:
            # peer-memory path: the hidden-state gradient of all rows in fp32, summed over ranks by the reduce kernel
            # (bf16 on the wire), each rank keeping its own rows
            p32 = ops.scratch("vp_dlnf32", n_all * C * 4, tile.device).view(torch.float32)[:n_all * C].view(n_all, C)
            own32 = ops.scratch("vp_dlnf_own", (n_all // z.world_size) * C * 4, tile.device).view(torch.float32)[:(n_all // z.world_size) * C]
            ops.chunked_ce_pass2(tile, a["ce_stats"], self._tgt_all, v0, w, V, self._dloss)
            ops.gemm(p32, tile, p["wte"][v0:v0 + w], b_mn=True, epi=ops.EPI_STORE_F32)
            ops.gemm(g["wte"][v0:v0 + w], tile, self._lnf_all, a_mn=True, b_mn=True, epi=ops.EPI_ACC_F32,
                     splits=ops._splits_for(w, C, n_all))
            z.reduce_scatter_rows_f32(p32.view(-1), own32)
            dl.view(-1).copy_(own32)
            return
        if w > 0:
            # dloss keeps the per-rank convention 1/(rows·accum): the slice's weight gradient then already
            # carries the factor W that the later mean over ranks removes
            ops.chunked_ce_pass2(tile, a["ce_stats"], self._tgt_all, v0, w, V, self._dloss)
            ops.lm_head_bwd_tile(partial, g["wte"][v0:v0 + w], tile, self._lnf_all, p["wte"][v0:v0 + w], accumulate=False)
        else:
            partial.zero_()
        dl.view(-1, C).copy_(z.reduce_scatter_rows(partial))

    def _vocab_tiles(self):
        """(first column, width) of each LM-head vocabulary tile (train_gpt2.mojo:2333-2350)."""
        Vp, w = self.config.padded_vocab_size, self.tile_width
        return [(c0, min(w, Vp - c0)) for c0 in range(0, Vp, w)]

    # ------------------------------------------------------------------ precision dispatch of the 4 linear sites
    def _site_mode(self, site: str, layer: int) -> str:
        """bf16 | fp8 | fp8b (per-128 block scales) | fp4 for one linear site (``train_gpt2.mojo:287-347``: FP8 covers the four
        linear layers of every block; NVFP4 covers only the MLP pair of layers [first, L-offset),
        the remaining sites of an fp4 run stay in bf16; LM head and attention are never low precision)."""
        pr = self.precision
        if pr.name == "fp8" and site in pr.fp8_sites:
            return "fp8b" if pr.fp8_block_scales else "fp8"
        if pr.name == "fp4" and site in ("fc", "fcproj") and pr.layer_in_fp4_range(layer, self.config.num_layer):
            return "fp4"
        return "bf16"

    def _linear_fwd(self, site, layer, out, inp, weight, bias, **kw) -> None:
        mode = self._site_mode(site, layer)
        if mode == "fp8":
            from ..ops import lowp
            lowp.matmul_fwd_fp8(out, inp, weight, bias, self.lowp.site(site, layer), **kw)
        elif mode == "fp8b":
            from ..ops import lowp
            lowp.matmul_fwd_fp8_block(out, inp, weight, bias, **kw)
        elif mode == "fp4":
            from ..ops import lowp
            lowp.matmul_fwd_fp4(out, inp, weight, bias, **kw)
        else:
            if self.zero is not None:
                self.zero.arm_linear(site, layer, backward=False)     # ZeRO-3: weight pulls ride on the layer GEMMs
            ops.matmul_fwd(out, inp, weight, bias, **kw)

    def _linear_bwd(self, site, layer, dinp, dweight, dbias, dout, inp, weight, **kw) -> None:
        mode = self._site_mode(site, layer)
        if mode == "fp8":
            from ..ops import lowp
            lowp.matmul_bwd_fp8(dinp, dweight, dbias, dout, inp, weight, self.lowp.site(site, layer), **kw)
        elif mode == "fp8b":
            from ..ops import lowp
            lowp.matmul_bwd_fp8_block(dinp, dweight, dbias, dout, inp, weight, **kw)
        elif mode == "fp4":
            from ..ops import lowp
            lowp.matmul_bwd_fp4(dinp, dweight, dbias, dout, inp, weight, rht=self.precision.fp4_rht,
                                sr=self.precision.fp4_sr, seed=self.rng_seed, step=self.micro_steps_done, **kw)
        else:
            if self.zero is not None:
                self.zero.arm_linear(site, layer, backward=True)      # armed for the input-gradient GEMM, the first one launched
            ops.matmul_bwd(dinp, dweight, dbias, dout, inp, weight, **kw)

    # ------------------------------------------------------------------ forward
    def forward(self, inputs: torch.Tensor, targets: Optional[torch.Tensor] = None,
                grad_accum_steps: int = 1, B: Optional[int] = None, T: Optional[int] = None,
                on_inputs_copied=None) -> None:
        """One micro-step forward.  ``inputs`` / ``targets`` are int32 host (ideally pinned) or
        device tensors of B·T tokens.  With targets the classifier also leaves dlogits in
        ``acts['logits']`` (llm.c design, ``train_gpt2.mojo:3751-3848``) and the micro-step's mean
        loss / grad_accum_steps is added to ``loss_acc`` on the device.  ``on_inputs_copied`` is called once
        the host-to-device token copies are enqueued (a loader records its buffer-reuse event there)."""
        if B is None:
            B, T = inputs.shape
        if (B, T) != (self.B, self.T):
            self.allocate_activations(B, T)
        cfg, a = self.config, self.acts
        L, C, NH, V = cfg.num_layer, cfg.channels, cfg.num_heads, cfg.vocab_size
        self.inputs_dev.copy_(inputs.view(B, T), non_blocking=True)
        if targets is not None:
            self.targets_dev.copy_(targets.view(B, T), non_blocking=True)
        if on_inputs_copied is not None:      # the host buffers may be reused once these two copies have run
            on_inputs_copied()
        z = self.zero
        if z is not None:
            z.before_embedding()
        p = self.p
        ops.encoder_fwd(a["encoded"], self.inputs_dev, p["wte"], p["wpe"])
        for l in range(L):
            if z is not None:
                z.before_layer(l, backward=False)
                p = self.p
            x_in = a["encoded"] if l == 0 else a["residual3"][l - 1]
            ops.layernorm_fwd(a["ln1"][l], a["ln1_mean"][l], a["ln1_rstd"][l], x_in, p["ln1w"][l], p["ln1b"][l])
            self._linear_fwd("qkv", l, a["qkv"][l], a["ln1"][l], p["qkvw"][l], p["qkvb"][l])
            ops.attention_fwd(a["atty"][l], a["lse"][l], a["qkv"][l], NH)
            self._linear_fwd("attproj", l, a["residual2"][l], a["atty"][l], p["attprojw"][l], p["attprojb"][l], residual=x_in)
            ops.layernorm_fwd(a["ln2"][l], a["ln2_mean"][l], a["ln2_rstd"][l], a["residual2"][l], p["ln2w"][l], p["ln2b"][l])
            gelu_out = a["fch_gelu"][0 if self.recompute else l]
            self._linear_fwd("fc", l, gelu_out, a["ln2"][l], p["fcw"][l], p["fcb"][l], pre_gelu=a["fch"][l])
            self._linear_fwd("fcproj", l, a["residual3"][l], gelu_out, p["fcprojw"][l], p["fcprojb"][l], residual=a["residual2"][l])
        if z is not None:
            z.before_head(backward=False)
            p = self.p
        if self._fused_gather is not None:
            self._fused_gather.wait_released()          # peers have finished reading the previous lnf rows
        ops.layernorm_fwd(a["lnf"], a["lnf_mean"], a["lnf_rstd"], a["residual3"][L - 1], p["lnfw"], p["lnfb"])
        dloss = 1.0 / (B * T * grad_accum_steps)
        self._dloss = dloss
        if self.vocab_parallel and targets is not None:
            self._vocab_parallel_forward(p, dloss)
            return
        if self.lm_head_chunks > 1 and targets is not None:
            # pass 1 over vocabulary tiles: running (max, sum-exp, target logit) per row
            for k, (c0, w) in enumerate(self._vocab_tiles()):
                tile = a["logits_tile"][:, :w]
                ops.matmul_fwd(tile, a["lnf"], p["wte"][c0:c0 + w])
                ops.chunked_ce_pass1(a["ce_stats"], tile, self.targets_dev, c0, w, V, k == 0)
            ops.chunked_ce_loss(a["losses"], a["ce_stats"])
            self.loss_acc += a["losses"].sum() * dloss
            return
        if "logits" not in a:
            a["logits"] = torch.empty(B, T, cfg.padded_vocab_size, dtype=self.dtype, device=self.device)
        ops.matmul_fwd(a["logits"], a["lnf"], p["wte"])
        if targets is not None:
            ops.fused_classifier(a["logits"], a["losses"], self.targets_dev, dloss, V)
            self.loss_acc += a["losses"].sum() * dloss

    def read_loss(self) -> float:
        """Synchronising read of the accumulated mean loss; resets the accumulator."""
        self.mean_loss = float(self.loss_acc.item())
        self.loss_acc.zero_()
        return self.mean_loss

    # ------------------------------------------------------------------ backward
    def zero_gradients(self) -> None:
        if self.zero is not None:
            self.zero.zero_gradients()
        else:
            self.grads.zero_()

    def backward(self, grad_accum_steps: int = 1, micro_step: int = 0, last_micro_step: Optional[bool] = None) -> None:
        """One micro-step backward; gradients accumulate (fp32).  ``micro_step == 0`` zeroes them
        (``train_gpt2.mojo:3948``); on the last micro-step the ZeRO engine reduces each bucket as
        soon as it is complete."""
        if last_micro_step is None:
            last_micro_step = micro_step == grad_accum_steps - 1
        if micro_step == 0:
            self.zero_gradients()
        cfg, a = self.config, self.acts
        L, NH = cfg.num_layer, cfg.num_heads
        z = self.zero
        B, T = self.B, self.T
        C = cfg.channels
        dres, dl, dl4 = a["dres"], a["dl_btc"], a["dl_bt4c"]
        dqkv = dl4.view(-1)[:B * T * 3 * C].view(B, T, 3 * C)
        if z is not None:
            z.before_head(backward=True)
        p, g = self.p, self.g
        # bucket 1: LM head
        if self.vocab_parallel:
            self._vocab_parallel_backward(p, g, dl)
        elif self.lm_head_chunks > 1:
            # pass 2: recompute each logits tile, turn it into dlogits, and consume it at once
            V = cfg.vocab_size
            for k, (c0, w) in enumerate(self._vocab_tiles()):
                tile = a["logits_tile"][:, :w]
                ops.matmul_fwd(tile, a["lnf"], p["wte"][c0:c0 + w])
                ops.chunked_ce_pass2(tile, a["ce_stats"], self.targets_dev, c0, w, V, self._dloss)
                ops.lm_head_bwd_tile(dl, g["wte"][c0:c0 + w], tile, a["lnf"], p["wte"][c0:c0 + w], accumulate=k > 0)
        else:                                  # dlogits are already in acts['logits']
            ops.matmul_bwd(dl, g["wte"], None, a["logits"], a["lnf"], p["wte"])
        # The bias gradients of attproj and fcproj are the column sums of the residual-stream gradient at the point where a
        # LayerNorm backward has just written it, so that kernel takes them in the same pass.  fcprojb of layer l is
        # produced one layer earlier (by ln1 of layer l + 1, or by the final LayerNorm): possible only where the
        # gradient tensors of all layers exist at once (no per-bucket pools, i.e. ZeRO stage < 2).
        ln_dbias = os.environ.get("LLMM_FUSED_LN_DBIAS", "0") != "0"     # measured: +0.043 ms in LayerNorm backward against a 0.032 ms pass of its own
        ln_dbias_prev = ln_dbias and (z is None or z.stage < 2)
        # bucket 2: final layernorm
        ops.layernorm_bwd(dres, g["lnfw"], g["lnfb"], dl, a["residual3"][L - 1], p["lnfw"], a["lnf_mean"], a["lnf_rstd"],
                          accumulate=False, dres_colsum=g["fcprojb"][L - 1] if ln_dbias_prev else None)
        if z is not None:
            z.grads_ready("head", last_micro_step)
        for l in range(L - 1, -1, -1):
            if z is not None:
                z.before_layer(l, backward=True)
                p, g = self.p, self.g
            x_in = a["encoded"] if l == 0 else a["residual3"][l - 1]
            if self.recompute:
                gelu_out = a["fch_gelu"][0]
                ops.gelu_fwd(gelu_out, a["fch"][l])       # train_gpt2.mojo:4490-4502
            else:
                gelu_out = a["fch_gelu"][l]
            # bf16 MLP: the fc bias gradient (column sums of dl4) is taken in the epilogue of the GEMM that writes dl4
            fc_dbias_upstream = self._site_mode("fcproj", l) == self._site_mode("fc", l) and self._site_mode("fc", l) in ("bf16", "fp8")
            kw = {"dinp_colsum": g["fcb"][l]} if fc_dbias_upstream else {}
            self._linear_bwd("fcproj", l, dl4, g["fcprojw"][l], None if ln_dbias_prev else g["fcprojb"][l], dres, gelu_out,
                             p["fcprojw"][l], gelu_pre=a["fch"][l], **kw)
            self._linear_bwd("fc", l, dl, g["fcw"][l], None if fc_dbias_upstream else g["fcb"][l], dl4, a["ln2"][l], p["fcw"][l])
            ops.layernorm_bwd(dres, g["ln2w"][l], g["ln2b"][l], dl, a["residual2"][l], p["ln2w"][l],
                              a["ln2_mean"][l], a["ln2_rstd"][l], accumulate=True,
                              dres_colsum=g["attprojb"][l] if ln_dbias else None)
            self._linear_bwd("attproj", l, dl, g["attprojw"][l], None if ln_dbias else g["attprojb"][l], dres, a["atty"][l],
                             p["attprojw"][l])
            # the qkv bias gradient (column sums of dqkv) comes out of the attention-backward epilogues
            attn_dbias = os.environ.get("LLMM_FUSED_QKV_DBIAS", "1") != "0"
            ops.attention_bwd(dqkv, dl, a["qkv"][l], a["atty"][l], a["lse"][l], NH, dbias=g["qkvb"][l] if attn_dbias else None)
            self._linear_bwd("qkv", l, dl, g["qkvw"][l], None if attn_dbias else g["qkvb"][l], dqkv, a["ln1"][l], p["qkvw"][l])
            ops.layernorm_bwd(dres, g["ln1w"][l], g["ln1b"][l], dl, x_in, p["ln1w"][l],
                              a["ln1_mean"][l], a["ln1_rstd"][l], accumulate=True,
                              dres_colsum=g["fcprojb"][l - 1] if (ln_dbias_prev and l > 0) else None)
            if z is not None:
                z.grads_ready(l, last_micro_step)
        if z is not None:
            z.before_embedding(backward=True)
            p, g = self.p, self.g
        ops.encoder_bwd(g["wte"], g["wpe"], dres, self.inputs_dev)
        self.micro_steps_done += 1
        if z is not None:
            z.grads_ready("embed", last_micro_step)
            if last_micro_step:
                z.reduce_all()

    # ------------------------------------------------------------------ optimizer
    def calculate_grad_norm(self) -> torch.Tensor:
        """Global L2 norm of the (reduced) gradients as a 1-element device tensor
        (``train_gpt2.mojo:5261-5383``)."""
        if self.zero is not None:
            return self.zero.grad_norm()
        ops.global_norm_squared(self.norm_sq, self.grads)
        return self.norm_sq.sqrt()

    def update(self, step: int, lr: float, weight_decay: float = 0.0, grad_scale: float = 1.0,
               beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8,
               dev_scale: Optional[torch.Tensor] = None) -> None:
        """AdamW step (``train_gpt2.mojo:5058-5259``; defaults β=(0.9, 0.999), eps 1e-8).
        ``grad_scale`` multiplies every gradient (clip factor); ``dev_scale`` is the same thing
        as a device scalar."""
        kw = dict(lr=lr, beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay, grad_scale=grad_scale,
                  step=step, seed=self.rng_seed + step, stochastic_rounding=self.use_stochastic_rounding,
                  dev_scale=dev_scale)
        if self.zero is not None:
            self.zero.optimizer_step(**kw)
        else:
            ops.adamw_update(self.params, self.master, self.grads, self.m, self.v, **kw)

    def clip_scale_from_norm(self, norm: torch.Tensor, max_norm: float = 1.0) -> torch.Tensor:
        """scale = max_norm / norm if norm > max_norm else 1, on the device
        (``train_gpt2.mojo:6532-6537``)."""
        torch.clamp(max_norm / (norm + 1e-6), max=1.0, out=self.clip_scale)
        return self.clip_scale

    # ------------------------------------------------------------------ checkpoints
    def full_params(self) -> torch.Tensor:
        return self.zero.gather_full_params() if self.zero is not None else self.params

    def write_checkpoint(self, model_path: str, state_path: str, state: ckpt.TrainingState, rank: int = 0) -> None:
        """Rank 0 writes the model file; every rank writes its m/v shard
        (``train_gpt2.mojo:5615-5696``)."""
        full = self.full_params()
        if rank == 0:
            ckpt.write_model_checkpoint(model_path, self.config, full, self.precision.checkpoint_version)
        state.use_master_weights = int(self.master is not None)
        ckpt.write_state_checkpoint(state_path, state, self.m, self.v)

    def load_checkpoint(self, model_path: str, state_path: str) -> ckpt.TrainingState:
        """Reload parameters and optimizer moments; the fp32 master copy is re-seeded from the
        parameters (``train_gpt2.mojo:5698-5801``)."""
        cfg, version = ckpt.read_model_header(model_path)
        if cfg != self.config:
            raise ValueError("Checkpoint error: model config does not match")
        if self.zero is not None:
            return self.zero.load_checkpoint(model_path, state_path)
        _, _, flat = ckpt.read_model_checkpoint(model_path, dtype=torch.float32)
        self.params.copy_(flat.to(self.device, self.dtype))
        if self.master is not None:
            self.master.copy_(self.params.float())
        state, m, v = ckpt.read_state_checkpoint(state_path, self.m.numel())
        self.m.copy_(m.to(self.device))
        self.v.copy_(v.to(self.device))
        return state

    def debug_nan_scan(self, which: str = "grads") -> dict:
        """Per-tensor census of non-finite values over the named parameter, gradient or activation views
        (``_debug_grad_nanscan``, ``train_gpt2.mojo:5385-5577``).  Returns {name: (nan, inf)} for tensors that have any."""
        views = {"grads": self.g, "params": self.p, "acts": self.acts}[which]
        bad = {}
        for name, t in views.items():
            if t is None or not torch.is_floating_point(t):
                continue
            nan, inf = ops.nan_census(t)
            if nan or inf:
                bad[name] = (nan, inf)
        return bad

    # ------------------------------------------------------------------ accounting
    def memory_report(self) -> dict:
        """Exact per-buffer accounting (``train_gpt2.mojo:5807-5999``; schema 3)."""
        def nbytes(t):
            return 0 if t is None else t.numel() * t.element_size()
        rep = {
            "schema": 3, "precision": self.precision.name, "num_parameters": self.num_parameters,
            "zero_stage": 0 if self.zero is None else self.zero.stage,
            "world_size": 1 if self.zero is None else self.zero.world_size,
            "params_bytes": nbytes(self.params), "grads_bytes": nbytes(self.grads), "m_bytes": nbytes(self.m),
            "v_bytes": nbytes(self.v), "master_bytes": nbytes(self.master),
            "activations_bytes": self.activation_bytes(), "B": self.B, "T": self.T,
        }
        if self.zero is not None:
            rep.update(self.zero.memory_report())
        rep["total_bytes"] = sum(v for k, v in rep.items() if k.endswith("_bytes"))
        return rep

    def print_memory_report(self) -> None:
        if os.environ.get("LLMM_MEM_REPORT", "") not in ("", "0"):
            print("[mem-report] " + json.dumps(self.memory_report()), flush=True)
