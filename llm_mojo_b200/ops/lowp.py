"""FP8 and NVFP4 linear layers: amax tracking, delayed scaling, quantisation, low-precision GEMMs.

Parity: ``llmm/lowp.mojo:51-99`` (precision specs: e4m3 forward operands, e5m2 output gradients,
per-tensor delayed scaling, history 16, margin 0), ``llmm/amax.mojo:230-682`` (amax + device-resident
scale state), ``llmm/matmul.mojo:1851-2138`` / ``:4146-4711`` (forward / backward wrappers for fp8 and
fp4), ``llmm/nvfp4_quant.mojo`` (NVFP4 format), ``llmm/hadamard.mojo`` (RHT-16),
``train_gpt2.mojo:861-994`` (``Fp8State``: per layer {qkv, attproj, fc, fcproj} x {input, weight,
d_output}).

GPU path: FP8 operands go straight into the tcgen05 ``kind::f8f6f4`` GEMM in the layout the
trainer already has (K-major or MN-major), so unlike the reference no transposed quantised copies
are made.  NVFP4 operands are quantised to e2m1 + e4m3 block scales (+ fp32 tensor scale) and the
GEMM runs on the dequantised value x block-scale in bf16 with the tensor scales folded into alpha:
every e2m1 x e4m3 product is exact in bf16, so the arithmetic equals the NVFP4 GEMM's while the
throughput is that of the bf16 tensor path.  CPU tensors run an emulation of the same numerics.
"""
from __future__ import annotations

import math
import os
from typing import Dict, Optional, Tuple

import torch

from . import (EPI_ACC_F32, EPI_BIAS, EPI_BIAS_GELU, EPI_BIAS_RESID, EPI_DGELU, EPI_NONE, _count, _gelu_grad_t, _gelu_t,
               _splits_for, dbias_reduce, gemm, gemm_mxfp8, gemm_nvfp4, scratch)
from ._lib import check, dtype_code, lib, ptr, stream
from . import matmul_fwd as ops_matmul_fwd, matmul_bwd as ops_matmul_bwd

E4M3, E5M2 = 0, 1
FMT_MAX = {E4M3: 448.0, E5M2: 57344.0}
AMAX_HISTORY = 16
E2M1_GRID = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
HADAMARD_SIGN = torch.tensor([-1., 1., 1., -1., -1., -1., -1., 1., -1., 1., 1., -1., 1., -1., -1., 1.])
NVFP4_SR_STREAM = 16


# ----------------------------------------------------------------------------- amax / scaling state
def compute_amax(out: torch.Tensor, x: torch.Tensor) -> None:
    """out[0] = max|x| (NaN if any element is NaN); ``llmm/amax.mojo:230-302``."""
    if x.is_cuda:
        check(lib().llmb_amax(ptr(out), ptr(x), x.numel(), dtype_code(x), stream()), "amax")
        _count()
    else:
        xf = x.float()
        out[0] = float("nan") if torch.isnan(xf).any() else xf.abs().max()


class AmaxState:
    """Device-resident delayed-scaling state of one GEMM operand site (``llmm/amax.mojo:425-565``)."""

    def __init__(self, device, fmt: int = E4M3, margin: int = 0):
        self.fmt, self.margin_mult = fmt, float(2 ** margin)
        self.state = torch.zeros(4 + AMAX_HISTORY, dtype=torch.float32, device=device)
        self.state[0] = 1.0
        self.state[1] = 1.0
        self.amax = torch.zeros(1, dtype=torch.float32, device=device)
        self.host_step = 0
        self.static = False

    def set_static(self, scale: float) -> None:
        """Freeze the scale at a calibrated constant: ``update_scale`` then does nothing, so neither the amax
        reduction nor the scale-update kernel runs for this operand (``llmm/lowp.mojo:880-935``, the reference's
        fastest FP8 mode).  Values beyond the calibrated range saturate in the encoder instead of overflowing."""
        if not (scale > 0 and math.isfinite(scale)):
            raise ValueError(f"static scale must be positive and finite, got {scale}")
        self.state[0], self.state[1] = float(scale), 1.0 / float(scale)
        self.static = True

    @property
    def scale(self) -> torch.Tensor:
        return self.state[0:1]

    @property
    def scale_inv(self) -> torch.Tensor:
        return self.state[1:2]

    def update_scale(self, x: torch.Tensor) -> None:
        """amax(x) → scale for this step (pre-push history; own amax during warm-up) → push."""
        if self.static:
            return
        compute_amax(self.amax, x)
        if x.is_cuda:
            check(lib().llmb_amax_update(ptr(self.state), ptr(self.amax), FMT_MAX[self.fmt], self.margin_mult, stream()),
                  "amax_update")
            _count()
        else:
            step, hist = self.host_step, self.state[4:]
            cur = float(self.amax)
            if step < AMAX_HISTORY:
                a = cur
            else:
                a = float("nan") if not torch.isfinite(hist).all() else float(hist.max())
            scale = 1.0 if (not math.isfinite(a) or a <= 0) else FMT_MAX[self.fmt] * self.margin_mult / a
            self.state[0], self.state[1] = scale, 1.0 / scale
            hist[step % AMAX_HISTORY] = cur
        self.host_step += 1


def _fp8_dtype(fmt: int):
    return torch.float8_e4m3fn if fmt == E4M3 else torch.float8_e5m2


def quantize_fp8(out_u8: torch.Tensor, x: torch.Tensor, scale: torch.Tensor, fmt: int) -> None:
    """out = fp8(x·scale) with saturation (``llmm/lowp.mojo:539-585``)."""
    if x.is_cuda:
        check(lib().llmb_quantize_fp8(ptr(out_u8), ptr(x), ptr(scale), x.numel(), fmt, dtype_code(x), stream()), "quantize_fp8")
        _count()
    else:
        y = (x.float() * scale).clamp(-FMT_MAX[fmt], FMT_MAX[fmt]).to(_fp8_dtype(fmt))
        out_u8.view(-1).copy_(y.view(torch.uint8).view(-1))


def dequantize_fp8(q_u8: torch.Tensor, scale_inv: torch.Tensor, fmt: int) -> torch.Tensor:
    return q_u8.view(_fp8_dtype(fmt)).float() * scale_inv.float().to(q_u8.device)


class LinearSite:
    """The three scaling states of one linear layer: input (e4m3), weight (e4m3), d_output (e5m2)."""

    def __init__(self, device):
        self.inp = AmaxState(device, E4M3)
        self.weight = AmaxState(device, E4M3)
        self.dout = AmaxState(device, E5M2)
        self.alpha = torch.ones(1, dtype=torch.float32, device=device)
        self.alpha2 = torch.ones(1, dtype=torch.float32, device=device)
        # fp8 copies of the forward operands, kept for the backward pass of the same micro-step (1 byte per element of the
        # layer input and of the weight) so that it does not quantise them a second time; `LLMM_FP8_KEEP_OPERANDS=0` drops
        # them and re-quantises, as the reference does
        self.qx: Optional[torch.Tensor] = None
        self.qw: Optional[torch.Tensor] = None
        self.kept = None          # (data_ptr, version) of the input and the weight the kept bytes were made from


class LowpState:
    """Per-layer sites {qkv, attproj, fc, fcproj} (``train_gpt2.mojo:861-994``)."""
    SITES = ("qkv", "attproj", "fc", "fcproj")

    def __init__(self, num_layer: int, device):
        self.sites: Dict[Tuple[str, int], LinearSite] = {(s, l): LinearSite(device) for l in range(num_layer) for s in self.SITES}

    def site(self, name: str, layer: int) -> LinearSite:
        return self.sites[(name, layer)]

    ROLES = ("inp", "weight", "dout")

    def set_static_scales(self, table: Dict[str, float], per_layer: bool = False) -> None:
        """Switch every site to static scaling from a table of ``site.layer.role`` (what ``calibrate_fp8_scales.py``
        writes) and / or ``site.role`` entries.  Default, as in the reference (``fp8_static_scale``,
        ``llmm/lowp.mojo:999``): ONE constant per (site, role) shared by all layers, the minimum over the layers in
        the table (the smallest scale is the safe one).  ``per_layer`` keeps each layer's own entry where present."""
        shared: Dict[Tuple[str, str], float] = {}
        for key, val in table.items():
            parts = key.split(".")
            if len(parts) == 3:
                sr = (parts[0], parts[2])
            elif len(parts) == 2:
                sr = (parts[0], parts[1])
            else:
                raise ValueError(f"bad static-scale key {key!r}")
            if sr[0] not in self.SITES or sr[1] not in self.ROLES:
                raise ValueError(f"unknown (site, role) pair in static-scale key {key!r}")
            shared[sr] = min(shared.get(sr, float("inf")), float(val))
        for (s, l), st in self.sites.items():
            for role in self.ROLES:
                if (s, role) not in shared:
                    raise ValueError(f"static-scale table has no entry for {s}.{role}")
                own = table.get(f"{s}.{l}.{role}") if per_layer else None
                getattr(st, role).set_static(float(own) if own is not None else shared[(s, role)])

    @staticmethod
    def read_scale_table(path: str) -> Dict[str, float]:
        import json
        with open(path) as f:
            blob = json.load(f)
        return {k: float(v) for k, v in (blob["scales"] if "scales" in blob else blob).items()}

    def min_scales(self) -> Dict[str, float]:
        """Current scale of every state (the fp8 calibration tool tracks their running minima)."""
        out = {}
        for (s, l), st in self.sites.items():
            for k in ("inp", "weight", "dout"):
                out[f"{s}.{l}.{k}"] = float(getattr(st, k).scale)
        return out


FUSED_DELAYED = os.environ.get("LLMM_FP8_FUSED_QUANT", "1") != "0"     # one pass (quantise + amax) once the amax history is full


KEEP_OPERANDS = os.environ.get("LLMM_FP8_KEEP_OPERANDS", "1") != "0"


def _q(name: str, x: torch.Tensor, state: AmaxState, buf: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Update the site's scale from ``x`` and return its fp8 quantisation (uint8 storage, same shape).

    While the amax history is filling up the scale of a step depends on the step's own amax: two passes (amax, then
    quantise).  Afterwards it depends on the history before this step only, and one kernel reads ``x`` once: it quantises
    with the scale just derived from the history and takes max|x| on the way, which is then pushed (same numbers as the
    two-pass order of ``llmm/amax.mojo:425-565``)."""
    if buf is None:
        buf = scratch("fp8_" + name, x.numel(), x.device)[:x.numel()].view(x.shape)
    vec = 8 if x.dtype == torch.bfloat16 else 4
    if (FUSED_DELAYED and x.is_cuda and not state.static and state.host_step >= AMAX_HISTORY and x.is_contiguous()
            and x.numel() % vec == 0 and x.dtype in (torch.bfloat16, torch.float32)):
        check(lib().llmb_quantize_fp8_delayed(ptr(buf), ptr(x), ptr(state.state), ptr(state.amax), x.numel(), state.fmt,
                                              FMT_MAX[state.fmt], state.margin_mult, dtype_code(x), stream()), "quantize_fp8_delayed")
        _count(3)
        state.host_step += 1
        return buf
    state.update_scale(x)
    quantize_fp8(buf, x, state.scale, state.fmt)
    return buf


def _delayed_ready(state: AmaxState, x: torch.Tensor) -> bool:
    """True when ``x`` can be quantised for ``state`` by the single-pass kernel: history full, scale not frozen."""
    vec = 8 if x.dtype == torch.bfloat16 else 4
    return (FUSED_DELAYED and x.is_cuda and not state.static and state.host_step >= AMAX_HISTORY and x.is_contiguous()
            and x.numel() % vec == 0 and x.dtype in (torch.bfloat16, torch.float32))


def _quant_amax(buf: torch.Tensor, x: torch.Tensor, state: AmaxState) -> None:
    check(lib().llmb_quantize_fp8_amax(ptr(buf), ptr(x), ptr(state.state), ptr(state.amax), x.numel(), state.fmt, dtype_code(x),
                                       stream()), "quantize_fp8_amax")
    _count()


def matmul_fwd_fp8(out, inp, weight, bias, site: LinearSite, *, pre_gelu=None, residual=None) -> None:
    """out = deq(q(inp)·q(W)ᵀ) (+bias)(+GELU / +residual); ``llmm/matmul.mojo:1851-2035``."""
    OC, C = weight.shape
    rows = inp.numel() // C
    x = inp.reshape(rows, C)
    site.kept = None
    if KEEP_OPERANDS and out.is_cuda:
        if site.qx is None or site.qx.shape != x.shape:
            site.qx = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
        if site.qw is None or site.qw.shape != weight.shape:
            site.qw = torch.empty(weight.shape, dtype=torch.uint8, device=x.device)
        if _delayed_ready(site.inp, x) and _delayed_ready(site.weight, weight):
            # both histories are full: one launch derives both scales and the GEMM's scale factor, one appends both amax values
            si, sw = site.inp, site.weight
            check(lib().llmb_fp8_prepare(ptr(si.state), ptr(si.amax), FMT_MAX[si.fmt], si.margin_mult, ptr(sw.state), ptr(sw.amax),
                                         FMT_MAX[sw.fmt], sw.margin_mult, ptr(site.alpha), ptr(si.state), ptr(sw.state), None, None, None,
                                         stream()), "fp8_prepare")
            qx, qw = site.qx, site.qw
            _quant_amax(qx, x, si)
            _quant_amax(qw, weight, sw)
            check(lib().llmb_fp8_push(ptr(si.state), ptr(si.amax), ptr(sw.state), ptr(sw.amax), stream()), "fp8_push")
            _count(2)
            si.host_step += 1
            sw.host_step += 1
        else:
            qx = _q("x", x, site.inp, site.qx)
            qw = _q("w", weight, site.weight, site.qw)
            torch.mul(site.inp.scale_inv, site.weight.scale_inv, out=site.alpha)
        site.kept = (x.data_ptr(), x._version, weight.data_ptr(), weight._version)
    else:
        qx = _q("x", x, site.inp)
        qw = _q("w", weight, site.weight)
        torch.mul(site.inp.scale_inv, site.weight.scale_inv, out=site.alpha)
    o = out.view(rows, OC)
    if out.is_cuda:
        if pre_gelu is not None:
            gemm(o, qx, qw, epi=EPI_BIAS_GELU, bias=bias, aux=pre_gelu.view(rows, OC), alpha=site.alpha, kind=2, a_fmt=E4M3, b_fmt=E4M3)
        elif residual is not None:
            gemm(o, qx, qw, epi=EPI_BIAS_RESID, bias=bias, aux=residual.view(rows, OC), alpha=site.alpha, kind=2, a_fmt=E4M3, b_fmt=E4M3)
        else:
            gemm(o, qx, qw, epi=EPI_BIAS if bias is not None else EPI_NONE, bias=bias, alpha=site.alpha, kind=2, a_fmt=E4M3, b_fmt=E4M3)
        return
    y = dequantize_fp8(qx, site.inp.scale_inv, E4M3) @ dequantize_fp8(qw, site.weight.scale_inv, E4M3).t()
    _finish_fwd(o, y, bias, pre_gelu, residual, rows, OC)


def _finish_fwd(o, y, bias, pre_gelu, residual, rows, OC):
    if bias is not None:
        y = y + bias.float()
    if pre_gelu is not None:
        pre_gelu.view(rows, OC).copy_(y)
        y = _gelu_t(pre_gelu.view(rows, OC).float())
    if residual is not None:
        y = y + residual.view(rows, OC).float()
    o.copy_(y)


def matmul_bwd_fp8(dinp, dweight, dbias, dout, inp, weight, site: LinearSite, *, gelu_pre=None, dinp_colsum=None) -> None:
    """dinp = deq(q5(dout)·q4(W)), dW += deq(q5(dout)ᵀ·q4(inp)); ``llmm/matmul.mojo:4146-4310``.  ``dinp_colsum`` (fp32 [C]) +=
    column sums of dinp, i.e. the bias gradient of the layer below, taken in the dGELU epilogue where that kernel runs."""
    OC, C = weight.shape
    rows = inp.numel() // C
    d, x = dout.reshape(rows, OC), inp.reshape(rows, C)
    site_fused = _delayed_ready(site.dout, d)
    if site_fused:
        # the d_output scale from its history and both GEMM scale factors (the input / weight scales of this step are final)
        sd = site.dout
        check(lib().llmb_fp8_prepare(ptr(sd.state), ptr(sd.amax), FMT_MAX[sd.fmt], sd.margin_mult, None, None, 0.0, 0.0, ptr(site.alpha),
                                     ptr(sd.state), ptr(site.weight.state), ptr(site.alpha2), ptr(sd.state), ptr(site.inp.state), stream()),
              "fp8_prepare")
        qd = scratch("fp8_d", d.numel(), d.device)[:d.numel()].view(d.shape)
        _quant_amax(qd, d, sd)
        check(lib().llmb_fp8_push(ptr(sd.state), ptr(sd.amax), None, None, stream()), "fp8_push")
        _count(2)
        sd.host_step += 1
    else:
        qd = _q("d", d, site.dout)
    if dinp is not None:
        if site.kept is not None and site.kept[2:] == (weight.data_ptr(), weight._version) and site.qw.shape == weight.shape:
            qw = site.qw                                                # the forward pass's bytes (same scale, same weight)
        else:
            qw = scratch("fp8_w", weight.numel(), weight.device)[:weight.numel()].view(weight.shape)
            quantize_fp8(qw, weight, site.weight.scale, E4M3)           # same scale as the forward pass of this step
        if not site_fused:
            torch.mul(site.dout.scale_inv, site.weight.scale_inv, out=site.alpha)
        di = dinp.view(rows, C)
        if dout.is_cuda:
            from . import colsum_usable, dbias_reduce as _dbias_reduce
            aux = gelu_pre.view(rows, C) if gelu_pre is not None else None
            fused = dinp_colsum is not None and aux is not None and colsum_usable(di, aux)
            gemm(di, qd, qw, b_mn=True, epi=EPI_DGELU if gelu_pre is not None else EPI_NONE, aux=aux, alpha=site.alpha, kind=2,
                 a_fmt=E5M2, b_fmt=E4M3, colsum=dinp_colsum if fused else None)
            if dinp_colsum is not None and not fused:
                _dbias_reduce(dinp_colsum, di)
        else:
            g = dequantize_fp8(qd, site.dout.scale_inv, E5M2) @ dequantize_fp8(qw, site.weight.scale_inv, E4M3)
            if gelu_pre is not None:
                g = g * _gelu_grad_t(gelu_pre.view(rows, C).float())
            di.copy_(g)
            if dinp_colsum is not None:
                dinp_colsum += di.float().sum(0)
    if site.kept is not None and site.kept[:2] == (x.data_ptr(), x._version) and site.qx.shape == x.shape:
        qx = site.qx
    else:
        qx = scratch("fp8_x", x.numel(), x.device)[:x.numel()].view(x.shape)
        quantize_fp8(qx, x, site.inp.scale, E4M3)
    if site_fused:
        alpha2 = site.alpha2
    else:
        alpha2 = site.dout.scale_inv * site.inp.scale_inv
    if dout.is_cuda:
        gemm(dweight.view(OC, C), qd, qx, a_mn=True, b_mn=True, epi=EPI_ACC_F32, splits=_splits_for(OC, C, rows), alpha=alpha2,
             kind=2, a_fmt=E5M2, b_fmt=E4M3)
        if dbias is not None:
            dbias_reduce(dbias, d)
    else:
        dweight.view(OC, C).add_(dequantize_fp8(qd, site.dout.scale_inv, E5M2).t() @ dequantize_fp8(qx, site.inp.scale_inv, E4M3))
        if dbias is not None:
            dbias += d.float().sum(0)


# ----------------------------------------------------------------------------- NVFP4
def hadamard16(x: torch.Tensor, inverse: bool = False) -> torch.Tensor:
    """16-point randomised Hadamard transform over consecutive blocks of the last dim
    (forward: H·(s⊙x), unnormalised; inverse: s⊙(H·y)/16); ``llmm/hadamard.mojo:229-264``."""
    out = torch.empty_like(x)
    if x.is_cuda:
        check(lib().llmb_hadamard16(ptr(out), ptr(x.contiguous()), x.numel(), int(inverse), dtype_code(x), stream()), "hadamard16")
        _count()
        return out
    H = torch.tensor([[(-1.0) ** bin(i & j).count("1") for j in range(16)] for i in range(16)])
    b = x.float().reshape(-1, 16)
    y = (b @ H.t()) * HADAMARD_SIGN / 16.0 if inverse else (b * HADAMARD_SIGN) @ H.t()
    return y.reshape(x.shape).to(x.dtype)


def _e2m1_round(v: torch.Tensor, rnd: Optional[torch.Tensor]) -> torch.Tensor:
    """Round |v| onto the e2m1 grid: nearest with ties to the even code (what the hardware convert
    ``cvt.rn.satfinite.e2m1x2.f32`` of the GPU kernels does), or stochastically."""
    a = v.abs().clamp(max=6.0)
    grid = E2M1_GRID.to(v.device)
    if rnd is None:
        mids = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], device=v.device)
        a = a.contiguous()
        idx = torch.bucketize(a, mids, right=True)                       # a tie goes up ...
        tie_down = torch.zeros_like(a, dtype=torch.bool)
        for j in (0, 2, 4, 6):                                           # ... unless the lower neighbour is the even code
            tie_down |= a == mids[j]
        idx = idx - tie_down.long()
    else:
        lo = (torch.bucketize(a.contiguous(), grid, right=True) - 1).clamp(0, 7)
        hi = (lo + 1).clamp(max=7)
        span = (grid[hi] - grid[lo]).clamp(min=1e-20)
        up = (rnd < (a - grid[lo]) / span) & (hi > lo)
        idx = torch.where(up, hi, lo)
    return torch.sign(v) * grid[idx]


def nvfp4_fake_quant(x: torch.Tensor, axis: int = 1, block_rows: int = 1, rht: bool = False, sr: bool = False,
                     seed: int = 0, stream_id: int = NVFP4_SR_STREAM, step: int = 0,
                     want_packed: bool = False, want_deq: bool = True):
    """Quantise a 2-D tensor to NVFP4 along ``axis`` and return ``(deq, tensor_scale[, q, scales])``
    where ``deq`` (bf16, same layout as ``x``) holds value × block-scale and ``tensor_scale`` is the
    fp32 second-level scale amax/(448·6) (``llmm/nvfp4_quant.mojo:528-724``).  ``q`` holds the packed e2m1 bytes
    [outer, K/2] with the quantised axis innermost and ``scales`` the ue4m3 block scales in 128×4 atoms: the operands
    of ``gemm_nvfp4``.  ``want_deq=False`` (GPU, with ``want_packed``) skips the bf16 image; ``deq`` is then None."""
    rows, cols = x.shape
    dev = x.device
    ts = torch.empty(1, dtype=torch.float32, device=dev)
    if x.is_cuda:
        amax = torch.empty(1, dtype=torch.float32, device=dev)
        src = x
        if rht:       # the tensor amax must be taken on what is quantised: amax of the transform, computed on the fly
            if (rows if axis == 0 else cols) % 16 == 0 and x.is_contiguous():
                check(lib().llmb_amax_rht(ptr(amax), ptr(x), rows, cols, axis, dtype_code(x), stream()), "amax_rht")
                _count()
            else:
                compute_amax(amax, _rht_along(x.float(), axis))
        else:
            compute_amax(amax, src)
        L = lib()
        check(L.llmb_nvfp4_tensor_scale(ptr(ts), ptr(amax), stream()), "nvfp4_tensor_scale")
        deq = torch.empty(rows, cols, dtype=torch.bfloat16, device=dev) if (want_deq or not want_packed) else None
        outer, K = (rows, cols) if axis == 1 else (cols, rows)
        q = torch.empty(outer * K // 2, dtype=torch.uint8, device=dev) if want_packed else None
        sc = torch.zeros(int(L.llmb_nvfp4_scale_bytes(outer, K, 1)), dtype=torch.uint8, device=dev) if want_packed else None
        check(L.llmb_nvfp4_quantize(ptr(q), ptr(sc), ptr(deq), ptr(x), ptr(ts), rows, cols, axis, block_rows, int(rht), int(sr),
                                    seed, stream_id, step, 1, dtype_code(x), stream()), "nvfp4_quantize")
        _count(3)
        return (deq, ts, q, sc) if want_packed else (deq, ts)
    # CPU emulation of the same numerics
    xf = x.float()
    if axis == 0:
        xf = xf.t()
    outer, K = xf.shape
    b = xf.reshape(outer, K // 16, 16)
    if rht:
        H = torch.tensor([[(-1.0) ** bin(i & j).count("1") for j in range(16)] for i in range(16)])
        b = (b * HADAMARD_SIGN) @ H.t()
    amax_t = b.abs().max()
    ts[0] = amax_t / (448.0 * 6.0) if amax_t > 0 else 1.0
    if block_rows == 16:
        pad = (-outer) % 16
        bb = torch.nn.functional.pad(b, (0, 0, 0, 0, 0, pad)).reshape(-1, 16, K // 16, 16)
        bamax = bb.abs().amax(dim=(1, 3)).repeat_interleave(16, dim=0)[:outer].unsqueeze(-1)
    else:
        bamax = b.abs().amax(dim=-1, keepdim=True)
    raw = torch.where(bamax > 0, bamax / 6.0 / ts, torch.ones_like(bamax))
    sc_dec = raw.clamp(max=448.0).to(torch.float8_e4m3fn).float()
    sc_val = sc_dec * ts
    sc_val = torch.where(sc_val > 0, sc_val, torch.ones_like(sc_val))
    rnd = torch.rand(b.shape, generator=torch.Generator().manual_seed(seed + step)) if sr else None
    qv = _e2m1_round(b / sc_val, rnd)
    deq = (qv * sc_dec).reshape(outer, K)
    if axis == 0:
        deq = deq.t()
    return deq.contiguous().to(torch.bfloat16 if x.dtype == torch.bfloat16 else torch.float32), ts


def _rht_along(x: torch.Tensor, axis: int) -> torch.Tensor:
    if axis == 1:
        return hadamard16(x)
    return hadamard16(x.t().contiguous()).t()


def nvfp4_native(*dims: int) -> bool:
    """True when the NVFP4 products run on the block-scaled tensor path (``gemm_nvfp4``) instead of the bf16 path
    on dequantised operands: on by default on a GPU, ``LLMM_FP4_NATIVE=0`` selects the latter; every contraction
    length in ``dims`` must be a multiple of 32 (16-byte rows of packed values)."""
    return os.environ.get("LLMM_FP4_NATIVE", "1") not in ("0", "") and all(d % 32 == 0 for d in dims)


def _qp(x, axis, block_rows, **kw):
    """Packed NVFP4 operand: (bytes [outer, K/2], swizzled scales, tensor scale)."""
    _, ts, q, sc = nvfp4_fake_quant(x, axis=axis, block_rows=block_rows, want_packed=True, want_deq=False, **kw)
    return q, sc, ts


def matmul_fwd_fp4(out, inp, weight, bias, *, pre_gelu=None, residual=None) -> None:
    """NVFP4 forward: activations 1x16 blocks, weights 16x16 blocks, RNE (``llmm/matmul.mojo:2038-2138``)."""
    OC, C = weight.shape
    rows = inp.numel() // C
    x = inp.reshape(rows, C)
    o = out.view(rows, OC)
    if out.is_cuda and nvfp4_native(C):
        qx, sx, tsx = _qp(x, 1, 1)
        qw, sw, tsw = _qp(weight, 1, 16)
        alpha = tsx * tsw
        if pre_gelu is not None:
            gemm_nvfp4(o, qx, sx, qw, sw, C, epi=EPI_BIAS_GELU, bias=bias, aux=pre_gelu.view(rows, OC), alpha=alpha)
        elif residual is not None:
            gemm_nvfp4(o, qx, sx, qw, sw, C, epi=EPI_BIAS_RESID, bias=bias, aux=residual.view(rows, OC), alpha=alpha)
        else:
            gemm_nvfp4(o, qx, sx, qw, sw, C, epi=EPI_BIAS if bias is not None else EPI_NONE, bias=bias, alpha=alpha)
        return
    dx, tsx = nvfp4_fake_quant(x, axis=1, block_rows=1)
    dw, tsw = nvfp4_fake_quant(weight, axis=1, block_rows=16)
    alpha = tsx * tsw
    if out.is_cuda:
        if pre_gelu is not None:
            gemm(o, dx, dw, epi=EPI_BIAS_GELU, bias=bias, aux=pre_gelu.view(rows, OC), alpha=alpha)
        elif residual is not None:
            gemm(o, dx, dw, epi=EPI_BIAS_RESID, bias=bias, aux=residual.view(rows, OC), alpha=alpha)
        else:
            gemm(o, dx, dw, epi=EPI_BIAS if bias is not None else EPI_NONE, bias=bias, alpha=alpha)
        return
    _finish_fwd(o, (dx.float() @ dw.float().t()) * alpha, bias, pre_gelu, residual, rows, OC)


def matmul_bwd_fp4(dinp, dweight, dbias, dout, inp, weight, *, gelu_pre=None, rht: bool = True, sr: bool = True,
                   seed: int = 0, step: int = 0) -> None:
    """NVFP4 backward (``llmm/matmul.mojo:4313-4711``): the gradient operand is rounded
    stochastically; the weight-gradient product applies the 16-point randomised Hadamard
    transform to both operands along the contraction (row) dimension and rescales by 1/16."""
    OC, C = weight.shape
    rows = inp.numel() // C
    d, x = dout.reshape(rows, OC), inp.reshape(rows, C)
    if dout.is_cuda and nvfp4_native(OC, rows):
        # the packed operand of a product contracted over axis 0 is written transposed ([cols, rows/2]), so all three
        # products are K-major x K-major on the block-scaled tensor path
        if dinp is not None:
            qd, sd, tsd = _qp(d, 1, 1, sr=sr, seed=seed, stream_id=NVFP4_SR_STREAM + 2, step=step)
            qw, sw, tsw = _qp(weight, 0, 16)
            gemm_nvfp4(dinp.view(rows, C), qd, sd, qw, sw, OC, epi=EPI_DGELU if gelu_pre is not None else EPI_NONE,
                       aux=gelu_pre.view(rows, C) if gelu_pre is not None else None, alpha=tsd * tsw)
        usable_rht = rht and rows % 16 == 0
        qd, sd, tsd = _qp(d, 0, 1, rht=usable_rht, sr=sr, seed=seed, stream_id=NVFP4_SR_STREAM + 3, step=step)
        qx, sx, tsx = _qp(x, 0, 1, rht=usable_rht)
        gemm_nvfp4(dweight.view(OC, C), qd, sd, qx, sx, rows, epi=EPI_ACC_F32,
                   splits=_splits_for(OC, C, rows, tile=128, tile_n=256, bk=256, units=148),
                   alpha=tsd * tsx * ((1.0 / 16.0) if usable_rht else 1.0))
        if dbias is not None:
            dbias_reduce(dbias, d)
        return
    if dinp is not None:
        dd, tsd = nvfp4_fake_quant(d, axis=1, block_rows=1, sr=sr, seed=seed, stream_id=NVFP4_SR_STREAM + 2, step=step)
        dw, tsw = nvfp4_fake_quant(weight, axis=0, block_rows=16)        # contraction runs over OC for dgrad
        alpha = tsd * tsw
        di = dinp.view(rows, C)
        if dout.is_cuda:
            gemm(di, dd, dw, b_mn=True, epi=EPI_DGELU if gelu_pre is not None else EPI_NONE,
                 aux=gelu_pre.view(rows, C) if gelu_pre is not None else None, alpha=alpha)
        else:
            g = (dd.float() @ dw.float()) * alpha
            if gelu_pre is not None:
                g = g * _gelu_grad_t(gelu_pre.view(rows, C).float())
            di.copy_(g)
    usable_rht = rht and rows % 16 == 0
    dd, tsd = nvfp4_fake_quant(d, axis=0, block_rows=1, rht=usable_rht, sr=sr, seed=seed, stream_id=NVFP4_SR_STREAM + 3, step=step)
    dx, tsx = nvfp4_fake_quant(x, axis=0, block_rows=1, rht=usable_rht)
    alpha = tsd * tsx * ((1.0 / 16.0) if usable_rht else 1.0)
    if dout.is_cuda:
        gemm(dweight.view(OC, C), dd, dx, a_mn=True, b_mn=True, epi=EPI_ACC_F32, splits=_splits_for(OC, C, rows), alpha=alpha)
        if dbias is not None:
            dbias_reduce(dbias, d)
    else:
        dweight.view(OC, C).add_((dd.float().t() @ dx.float()) * alpha)
        if dbias is not None:
            dbias += d.float().sum(0)


# ------------------------------------------------------------------------------ FP8 with per-128 block scales
def fp8_block_fake_quant(x: torch.Tensor, mode: int, fmt: int = E4M3) -> torch.Tensor:
    """x [rows, cols] → same shape holding fp8(x / s)·s with one power-of-two scale s = 2^ceil(log2(amax / fmt_max))
    per block.  ``mode`` 0: 1×128 blocks along the columns, 1: 128×1 blocks along the rows, 2: 128×128 blocks.
    Power-of-two scales keep value × scale exactly representable in bf16, so a GEMM on these tensors has the
    numerics of a block-scaled FP8 GEMM with fp32 accumulation (the per-128 scaling that the fp8 configuration of
    the benchmark asks for; the reference itself scales per tensor, ``llmm/lowp.mojo:89-99``)."""
    rows, cols = x.shape
    if x.is_cuda and x.dtype == torch.bfloat16:
        xc = x.contiguous()
        out = torch.empty_like(xc)
        check(lib().llmb_fp8_block_fake_quant(ptr(out), ptr(xc), rows, cols, mode, fmt, stream()), "fp8_block_fake_quant")
        _count()
        return out
    xf = x.float()
    if mode == 0:
        b = xf.reshape(rows, cols // 128, 128)
        amax = b.abs().amax(dim=-1, keepdim=True)
    elif mode == 1:
        b = xf.reshape(rows // 128, 128, cols)
        amax = b.abs().amax(dim=1, keepdim=True)
    else:
        b = xf.reshape(rows // 128, 128, cols // 128, 128)
        amax = b.abs().amax(dim=(1, 3), keepdim=True)
    ratio = amax / FMT_MAX[fmt]
    s = torch.where(amax > 0, torch.exp2(torch.ceil(torch.log2(ratio.clamp_min(1e-45)))), torch.ones_like(amax))
    dt = torch.float8_e4m3fn if fmt == E4M3 else torch.float8_e5m2
    q = (b / s).clamp(-FMT_MAX[fmt], FMT_MAX[fmt]).to(dt).float() * s
    return q.reshape(rows, cols).to(x.dtype)


def fp8_block_usable(rows: int, C: int, OC: int) -> bool:
    return rows % 128 == 0 and C % 128 == 0 and OC % 128 == 0


def fp8_block_quant(x: torch.Tensor, gran: int, fmt: int = E4M3, transpose: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """GPU only: x [rows, cols] bf16 → (fp8 bytes, ue8m0 scale atoms), the operands of ``gemm_mxfp8``.  ``gran`` 0 = 1×128
    blocks, 1 = 128×1 blocks (written transposed: bytes [cols, rows]), 2 = 128×128 blocks (either orientation).  Same
    scales and rounding as ``fp8_block_fake_quant`` modes 0 / 1 / 2."""
    rows, cols = x.shape
    q = torch.empty((cols, rows) if transpose else (rows, cols), dtype=torch.uint8, device=x.device)
    sf = torch.empty((rows // 128) * (cols // 128) * 512, dtype=torch.uint8, device=x.device)
    check(lib().llmb_fp8_block_quant(ptr(q), ptr(sf), ptr(x.contiguous()), rows, cols, gran, fmt, int(transpose), stream()),
          "fp8_block_quant")
    _count()
    return q, sf


def fp8_block_quant_dual(x: torch.Tensor, fmt: int = E4M3) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """GPU only: both orientations from one read of ``x`` [rows, cols]: ``(q0, s0)`` = ``fp8_block_quant(x, 0)`` (1×128 blocks,
    for a product contracted over the columns) and ``(q1, s1)`` = ``fp8_block_quant(x, 1, transpose=True)`` (128×1 blocks,
    bytes [cols, rows], for a product contracted over the rows)."""
    rows, cols = x.shape
    q0 = torch.empty((rows, cols), dtype=torch.uint8, device=x.device)
    q1 = torch.empty((cols, rows), dtype=torch.uint8, device=x.device)
    nsf = (rows // 128) * (cols // 128) * 512
    s0, s1 = (torch.empty(nsf, dtype=torch.uint8, device=x.device) for _ in range(2))
    check(lib().llmb_fp8_block_quant_dual(ptr(q0), ptr(s0), ptr(q1), ptr(s1), ptr(x.contiguous()), rows, cols, fmt, stream()),
          "fp8_block_quant_dual")
    _count()
    return q0, s0, q1, s1


FP8B_DUAL = os.environ.get("LLMM_FP8B_DUAL_QUANT", "1") != "0"
_FP8B_KEPT: Dict[Tuple[int, Tuple[int, ...]], Tuple[torch.Tensor, torch.Tensor]] = {}   # (input pointer, shape) -> its 128×1 bytes and scales


def fp8_block_native() -> bool:
    """Block-scaled FP8 products on the MXFP8 tensor path (default on a GPU); ``LLMM_FP8B_NATIVE=0`` runs them on the
    bf16 path over fake-quantised operands (same numerics, the path the tests compare against)."""
    return os.environ.get("LLMM_FP8B_NATIVE", "1") not in ("0", "")


def matmul_fwd_fp8_block(out, inp, weight, bias, *, pre_gelu=None, residual=None) -> None:
    """Block-scaled FP8 forward: e4m3 activations in 1×128 blocks along the contraction, e4m3 weights in 128×128
    blocks, power-of-two scales; on a GPU the product runs on the MXFP8 tensor path (the per-128 scale repeated for its
    four 32-value blocks), otherwise on fake-quantised operands (exact, see ``fp8_block_fake_quant``)."""
    OC, C = weight.shape
    rows = inp.numel() // C
    if not fp8_block_usable(rows, C, OC):
        return ops_matmul_fwd(out, inp, weight, bias, pre_gelu=pre_gelu, residual=residual)
    if out.is_cuda and inp.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and fp8_block_native():
        x2 = inp.reshape(rows, C)
        if FP8B_DUAL:
            # the 128×1 orientation the weight gradient will need comes out of the same read and is kept until the backward pass
            qx, sx, qxt, sxt = fp8_block_quant_dual(x2, E4M3)
            _FP8B_KEPT[(x2.data_ptr(), tuple(x2.shape))] = (qxt, sxt)
        else:
            qx, sx = fp8_block_quant(x2, 0, E4M3)
        qw, sw = fp8_block_quant(weight, 2, E4M3)
        o = out.view(rows, OC)
        if pre_gelu is not None:
            gemm_mxfp8(o, qx, sx, qw, sw, epi=EPI_BIAS_GELU, bias=bias, aux=pre_gelu.view(rows, OC))
        elif residual is not None:
            gemm_mxfp8(o, qx, sx, qw, sw, epi=EPI_BIAS_RESID, bias=bias, aux=residual.view(rows, OC))
        else:
            gemm_mxfp8(o, qx, sx, qw, sw, epi=EPI_BIAS if bias is not None else EPI_NONE, bias=bias)
        return
    dx = fp8_block_fake_quant(inp.reshape(rows, C), 0, E4M3)
    dw = fp8_block_fake_quant(weight, 2, E4M3)
    ops_matmul_fwd(out, dx, dw, bias, pre_gelu=pre_gelu, residual=residual)


def matmul_bwd_fp8_block(dinp, dweight, dbias, dout, inp, weight, *, gelu_pre=None) -> None:
    """Block-scaled FP8 backward: the output gradient is e5m2 (1×128 along OC for dinp, 128×1 along the rows for
    dW), the saved input e4m3 in 128×1 blocks along the rows, the weight e4m3 in 128×128 blocks."""
    OC, C = weight.shape
    rows = inp.numel() // C
    if not fp8_block_usable(rows, C, OC):
        return ops_matmul_bwd(dinp, dweight, dbias, dout, inp, weight, gelu_pre=gelu_pre)
    d, x = dout.reshape(rows, OC), inp.reshape(rows, C)
    if dout.is_cuda and dout.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and inp.dtype == torch.bfloat16 and fp8_block_native():
        # operands of a product contracted over the rows (or over OC for the weight) are written transposed: all K-major
        qdt = None
        if dinp is not None:
            if FP8B_DUAL:
                qd, sd, qdt, sdt = fp8_block_quant_dual(d, E5M2)      # both orientations of the output gradient from one read
            else:
                qd, sd = fp8_block_quant(d, 0, E5M2)
            qw, sw = fp8_block_quant(weight, 2, E4M3, transpose=True)
            gemm_mxfp8(dinp.view(rows, C), qd, sd, qw, sw, a_fmt=E5M2, b_fmt=E4M3, epi=EPI_DGELU if gelu_pre is not None else EPI_NONE,
                       aux=gelu_pre.view(rows, C) if gelu_pre is not None else None)
        if qdt is not None:
            qd, sd = qdt, sdt
        else:
            qd, sd = fp8_block_quant(d, 1, E5M2, transpose=True)
        kept = _FP8B_KEPT.pop((x.data_ptr(), tuple(x.shape)), None) if FP8B_DUAL else None
        if kept is not None:
            qx, sx = kept                                           # made in the forward pass of this micro-step from the same tensor
        else:
            qx, sx = fp8_block_quant(x, 1, E4M3, transpose=True)
        gemm_mxfp8(dweight.view(OC, C), qd, sd, qx, sx, a_fmt=E5M2, b_fmt=E4M3, epi=EPI_ACC_F32,
                   splits=_splits_for(OC, C, rows, tile=128, tile_n=256, bk=128, units=148))
        if dbias is not None:
            dbias_reduce(dbias, d)
        return
    if dinp is not None:
        ops_matmul_bwd(dinp, None, None, fp8_block_fake_quant(d, 0, E5M2), x, fp8_block_fake_quant(weight, 2, E4M3), gelu_pre=gelu_pre)
    ops_matmul_bwd(None, dweight, None, fp8_block_fake_quant(d, 1, E5M2), fp8_block_fake_quant(x, 1, E4M3), weight)
    if dbias is not None:
        dbias_reduce(dbias, d)
