"""Op library: every op of the GPT-2 trainer as explicit forward / backward functions.

CUDA tensors run the hand-written sm_100a kernels (``csrc/*.cu`` through ctypes); CPU tensors
run the fp32 PyTorch statement of the same math, which is both the CPU training target and the
oracle the GPU tests compare against.  All functions write into caller-provided outputs so the
training loop allocates nothing per step.

Parity map (reference ``llmm/`` module → function here):
encoder → ``encoder_fwd/bwd``; layernorm → ``layernorm_fwd``, ``residual_layernorm_fwd``,
``layernorm_bwd``; matmul → ``matmul_fwd``, ``matmul_bwd``; attention (+split/merge/softmax) →
``attention_fwd/bwd``; gelu → ``gelu_fwd/bwd``; fused_classifier → ``fused_classifier``;
adamw → ``adamw_update``; global_norm → ``global_norm_squared``.
"""
from __future__ import annotations

import math
import os
from typing import Optional

import torch
import torch.nn.functional as F

from . import _lib
from ._lib import check, dtype_code, lib, ptr, status_word, stream

LN_EPS = 1e-5
GELU_K = math.sqrt(2.0 / math.pi)

# Library GEMM/attention can be forced for A/B comparisons (never the default on CUDA).
GEMM_IMPL = os.environ.get("LLMB_GEMM", "tcgen05")        # tcgen05 | cublas
ATTN_IMPL = os.environ.get("LLMB_ATTN", "tcgen05")        # tcgen05 | sdpa
ATTN_BWD = os.environ.get("LLMB_ATTN_BWD", "fused")       # fused (one kernel, dQ partials reduced in fp32) | split (dK/dV and dQ kernels)

_SCRATCH = {}
LAUNCHES = 0     # number of kernel-library launches issued (bench.py reports it)


_CANARIES = {}


def _count(n: int = 1) -> None:
    global LAUNCHES
    LAUNCHES += n


CANARY_BYTES, CANARY_VALUE = 256, 0xA5


def scratch(name: str, nbytes: int, device: torch.device, zero: bool = False) -> torch.Tensor:
    """Persistent per-(name, device) scratch buffer, grown on demand (cf. llmm/memory.mojo:81-123).  ``zero``: the buffer
    is zero-filled when it is (re)allocated - for kernels that leave their accumulation scratch zeroed behind them.  Under
    ``LLMB_BOUNDS_CHECK=1`` every buffer is followed by a 256-byte canary that ``verify_scratch_canaries`` checks:
    a kernel that writes past the scratch it was given (the reference's ``_check_scratch``, llmm/zero.mojo:555) is
    caught at the end of the step instead of corrupting a neighbour."""
    key = (name, str(device))
    t = _SCRATCH.get(key)
    if t is None or t.numel() < nbytes:
        size = max(nbytes, 256)
        if _lib.BOUNDS_CHECK:
            full = torch.empty(size + CANARY_BYTES, dtype=torch.uint8, device=device)
            full[size:].fill_(CANARY_VALUE)
            _CANARIES[key] = full
            t = full[:size]
        else:
            t = torch.empty(size, dtype=torch.uint8, device=device)
        if zero:
            t.zero_()
        _SCRATCH[key] = t
    return t


def verify_scratch_canaries() -> None:
    """Raises if any scratch buffer's canary was overwritten (checked mode only; no-op otherwise)."""
    for (name, dev), full in _CANARIES.items():
        tail = full[full.numel() - CANARY_BYTES:]
        if not bool((tail == CANARY_VALUE).all()):
            raise _lib.KernelError(f"scratch buffer {name!r} on {dev}: a kernel wrote past its {full.numel() - CANARY_BYTES} bytes")


# ----------------------------------------------------------------------------- encoder
def encoder_fwd(out: torch.Tensor, tokens: torch.Tensor, wte: torch.Tensor, wpe: torch.Tensor) -> None:
    """out[b,t,:] = wte[tokens[b,t]] + wpe[t]   (llmm/encoder.mojo:214-281)."""
    B, T = tokens.shape
    C = wte.shape[1]
    if out.is_cuda:
        check(lib().llmb_encoder_fwd(ptr(out), ptr(tokens), ptr(wte), ptr(wpe), B, T, C, wte.shape[0], dtype_code(out), stream()),
              "encoder_fwd")
        _count()
    else:
        out.view(B, T, C).copy_(wte[tokens.long()] + wpe[:T].unsqueeze(0))


def encoder_bwd(dwte: torch.Tensor, dwpe: torch.Tensor, dout: torch.Tensor, tokens: torch.Tensor) -> None:
    """dwte[tok] += dout, dwpe[t] += Σ_b dout; deterministic (llmm/encoder.mojo:1032-1150)."""
    B, T = tokens.shape
    C = dwte.shape[1]
    if dout.is_cuda:
        L = lib()
        nb = L.llmb_encoder_bwd_scratch_bytes(B * T, C)
        s = scratch("encoder_bwd", nb, dout.device)
        vocab_bits = max(1, int(dwte.shape[0] - 1).bit_length())
        check(L.llmb_encoder_bwd(ptr(dwte), ptr(dwpe), ptr(dout), ptr(tokens), ptr(s), s.numel(), B, T, C, dwte.shape[0],
                                 vocab_bits, dtype_code(dout), stream()), "encoder_bwd")
        _count(4)
    else:
        d = dout.reshape(B * T, C).float()
        dwte.index_add_(0, tokens.reshape(-1).long(), d)
        dwpe[:T] += d.view(B, T, C).sum(0)


# ----------------------------------------------------------------------------- layernorm
def layernorm_fwd(out, mean, rstd, inp, weight, bias) -> None:
    """Row LayerNorm, saves mean / rstd in fp32 (llmm/layernorm.mojo:366-424)."""
    residual_layernorm_fwd(None, out, mean, rstd, inp, None, weight, bias)


def residual_layernorm_fwd(residual_out, out, mean, rstd, inp1, inp2, weight, bias) -> None:
    """residual_out = inp1 + inp2; out = LN(residual_out)   (llmm/layernorm.mojo:1002-1096)."""
    C = weight.numel()
    rows = inp1.numel() // C
    if out.is_cuda:
        check(lib().llmb_layernorm_fwd(ptr(out), ptr(mean), ptr(rstd), ptr(residual_out), ptr(inp1), ptr(inp2),
                                       ptr(weight), ptr(bias), rows, C, dtype_code(out), stream()), "layernorm_fwd")
        _count()
    else:
        x = inp1.reshape(rows, C)
        if inp2 is not None:
            x = x + inp2.reshape(rows, C)
            residual_out.view(rows, C).copy_(x)
        x = x.float()
        m = x.mean(1, keepdim=True)
        v = ((x - m) ** 2).mean(1, keepdim=True)
        r = torch.rsqrt(v + LN_EPS)
        out.view(rows, C).copy_((x - m) * r * weight.float() + bias.float())
        if mean is not None:
            mean.view(rows).copy_(m.view(rows))
        if rstd is not None:
            rstd.view(rows).copy_(r.view(rows))


def layernorm_bwd(dresidual, dweight, dbias, dout, inp, weight, mean, rstd, accumulate: bool = True,
                  dres_colsum=None) -> None:
    """dresidual (+)= LN'(dout); dweight += Σ dout·norm; dbias += Σ dout (fp32 grads).

    With ``accumulate`` the input gradient is added into ``dresidual`` — the fused
    residual-backward of llmm/layernorm.mojo:2426-2614.  ``dres_colsum`` (fp32 [C]) += Σ_rows of the values written
    to ``dresidual``: the bias gradient of the linear layer whose output gradient that is, taken in the same pass."""
    C = weight.numel()
    rows = inp.numel() // C
    if dout.is_cuda:
        L = lib()
        nb = L.llmb_layernorm_bwd_scratch_bytes(rows, C)
        s = scratch("layernorm_bwd", nb, dout.device)
        check(L.llmb_layernorm_bwd_colsum(ptr(dresidual), ptr(dweight), ptr(dbias), ptr(dres_colsum), ptr(s), s.numel(),
                                          ptr(dout), ptr(inp), ptr(weight), ptr(mean), ptr(rstd), rows, C, int(accumulate),
                                          dtype_code(dout), stream()), "layernorm_bwd")
        _count(2)
    else:
        d = dout.reshape(rows, C).float()
        x = inp.reshape(rows, C).float()
        norm = (x - mean.view(rows, 1)) * rstd.view(rows, 1)
        dweight += (d * norm).sum(0)
        dbias += d.sum(0)
        dn = d * weight.float()
        g = (dn - dn.mean(1, keepdim=True) - norm * (dn * norm).mean(1, keepdim=True)) * rstd.view(rows, 1)
        dr = dresidual.view(rows, C)
        if accumulate:
            dr += g.to(dr.dtype)
        else:
            dr.copy_(g)
        if dres_colsum is not None:
            dres_colsum += dr.float().sum(0)


# ----------------------------------------------------------------------------- GELU
def _gelu_t(x: torch.Tensor) -> torch.Tensor:
    return 0.5 * x * (1.0 + torch.tanh(GELU_K * (x + 0.044715 * x ** 3)))


def _gelu_grad_t(x: torch.Tensor) -> torch.Tensor:
    u = GELU_K * (x + 0.044715 * x ** 3)
    t = torch.tanh(u)
    return 0.5 * (1 + t) + 0.5 * x * (1 - t * t) * GELU_K * (1 + 3 * 0.044715 * x * x)


def gelu_fwd(out, inp) -> None:
    """tanh-GELU (llmm/gelu.mojo:35-82)."""
    if out.is_cuda:
        check(lib().llmb_gelu_fwd(ptr(out), ptr(inp), inp.numel(), dtype_code(inp), stream()), "gelu_fwd")
        _count()
    else:
        out.copy_(_gelu_t(inp.float()))


def gelu_bwd(dinp, inp, dout) -> None:
    """dinp = dout · gelu'(inp)   (llmm/gelu.mojo:337-430); dinp may alias dout."""
    if dout.is_cuda:
        check(lib().llmb_gelu_bwd(ptr(dinp), ptr(inp), ptr(dout), inp.numel(), dtype_code(inp), stream()), "gelu_bwd")
        _count()
    else:
        dinp.copy_(dout.float() * _gelu_grad_t(inp.float()))


# ----------------------------------------------------------------------------- matmul
EPI_NONE, EPI_BIAS, EPI_BIAS_GELU, EPI_DGELU, EPI_ACC_F32, EPI_BIAS_RESID, EPI_STORE_F32 = range(7)


def gemm(D, A, B, *, a_mn=False, b_mn=False, epi=EPI_NONE, bias=None, aux=None, alpha=None, splits=1,
         kind: int = 0, a_fmt: int = 0, b_fmt: int = 0, colsum=None) -> None:
    """Raw tcgen05 GEMM: D[M,N] = epi(A·Bᵀ).  A is [M,K] (or [K,M] when ``a_mn``), B is [N,K]
    (or [K,N] when ``b_mn``); all row-major with arbitrary row pitch.  ``colsum`` (fp32 [N], dGELU epilogue of
    the bf16 kernel only, see ``colsum_usable``) accumulates the column sums of D inside the epilogue."""
    M, N = D.shape
    K = A.shape[0] if a_mn else A.shape[1]
    if colsum is not None:
        lib().llmb_gemm_set_colsum(ptr(colsum))
    check(lib().llmb_gemm(ptr(D), ptr(A), ptr(B), ptr(bias), ptr(aux), ptr(alpha), M, N, K, A.stride(0), B.stride(0),
                          D.stride(0), aux.stride(0) if aux is not None else 0, int(a_mn), int(b_mn), kind, a_fmt,
                          b_fmt, epi, splits, ptr(status_word(D.device)), stream()), "gemm")
    _count()


def gemm_nvfp4(D, qa, sfa, qb, sfb, K: int, *, epi=EPI_NONE, bias=None, aux=None, alpha=None, splits=1) -> None:
    """Native NVFP4 GEMM (``tcgen05.mma.kind::mxf4nvf4``): D[M,N] = epi(alpha · (A·sfa)(B·sfb)ᵀ).  ``qa`` / ``qb`` are
    the packed e2m1 bytes of A [M,K] and B [N,K] and ``sfa`` / ``sfb`` their swizzled ue4m3 block scales, as
    ``nvfp4_fake_quant(..., want_packed=True)`` returns them (the cuBLASLt call of ``llmm/matmul.mojo:2038-2138``)."""
    M, N = D.shape
    check(lib().llmb_gemm_nvfp4(ptr(D), ptr(qa), ptr(qb), ptr(sfa), ptr(sfb), ptr(bias), ptr(aux), ptr(alpha), M, N, K,
                                D.stride(0), aux.stride(0) if aux is not None else 0, epi, splits,
                                ptr(status_word(D.device)), stream()), "gemm_nvfp4")
    _count()


def gemm_mxfp8(D, qa, sfa, qb, sfb, *, a_fmt=0, b_fmt=0, epi=EPI_NONE, bias=None, aux=None, alpha=None, splits=1) -> None:
    """Native MXFP8 GEMM (``tcgen05.mma.kind::mxf8f6f4.block_scale``): D[M,N] = epi(alpha · (A·sfa)(B·sfb)ᵀ) with fp8
    bytes ``qa`` [M,K] / ``qb`` [N,K] (format 0 = e4m3, 1 = e5m2) and one ue8m0 scale per row and 32 values of K in 128×4
    atoms, as ``lowp.fp8_block_quant`` writes them."""
    M, N = D.shape
    K = qa.shape[1]
    check(lib().llmb_gemm_mxfp8(ptr(D), ptr(qa), ptr(qb), ptr(sfa), ptr(sfb), ptr(bias), ptr(aux), ptr(alpha), M, N, K, a_fmt, b_fmt,
                                D.stride(0), aux.stride(0) if aux is not None else 0, epi, splits,
                                ptr(status_word(D.device)), stream()), "gemm_mxfp8")
    _count()


def colsum_usable(D: torch.Tensor, aux: torch.Tensor) -> bool:
    """The dGELU GEMM can add the column sums of its result (the bias gradient of the layer below) in its epilogue when
    it runs as the bf16 CTA-pair kernel with the TMA epilogue: 16-byte aligned bf16 rows of D and aux."""
    if not (D.is_cuda and D.dtype == torch.bfloat16 and aux.dtype == torch.bfloat16 and GEMM_IMPL == "tcgen05"):
        return False
    if os.environ.get("LLMB_GEMM_PAIR", "1") == "0" or os.environ.get("LLMB_GEMM_TMA_EPI", "1") == "0":
        return False
    if os.environ.get("LLMM_FUSED_FC_DBIAS", "1") == "0":
        return False
    return (D.data_ptr() | aux.data_ptr()) % 16 == 0 and (D.stride(0) * 2) % 16 == 0 and (aux.stride(0) * 2) % 16 == 0


def _tc_kind(t: torch.Tensor):
    """tcgen05 kind for a storage dtype: 0 (kind::f16, bf16 operands), 1 (kind::tf32, fp32 operands)."""
    if t.dtype == torch.bfloat16:
        return 0
    if t.dtype == torch.float32 and os.environ.get("LLMM_NO_TF32", "") in ("", "0"):
        return 1
    return None


def _splits_for(M: int, N: int, K: int, *, tile: int = 256, tile_n: int = 0, bk: int = 64, units: int = 74) -> int:
    """Split-K factor for the dW GEMMs (by default 256x256 tiles on 74 CTA pairs, 64 values of K per stage; the
    block-scaled kernels have 128x256 tiles on 148 CTAs): the number of splits that minimises waves x (k-blocks per
    unit + a fixed per-unit cost for the prologue and the fp32 red.add epilogue)."""
    tile_n = tile_n or tile
    tiles = max(1, ((M + tile - 1) // tile) * ((N + tile_n - 1) // tile_n))
    kb = (K + bk - 1) // bk
    best, best_cost = 1, None
    for s in range(1, max(1, min(16, kb // 8)) + 1):
        waves = -(-tiles * s // units)
        cost = waves * (kb / s + 24.0)
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


def matmul_fwd(out, inp, weight, bias=None, *, pre_gelu=None, residual=None) -> None:
    """out = inp·weightᵀ (+bias) — optionally out = GELU(pre), pre_gelu = inp·Wᵀ+b, or
    out = inp·Wᵀ + b + residual (llmm/matmul.mojo:1526-1722: BIAS / GELU_AUX_BIAS epilogues)."""
    OC, C = weight.shape
    rows = inp.numel() // C
    x = inp.reshape(rows, C)
    o = out if out.dim() == 2 else out.view(rows, OC)       # a 2-D output may be a column slice (row pitch > OC)
    if out.is_cuda and GEMM_IMPL == "tcgen05" and _tc_kind(out) is not None:
        kind = _tc_kind(out)          # bf16 -> kind::f16, fp32 storage -> kind::tf32 (fp32 accumulate either way)
        if pre_gelu is not None:
            gemm(o, x, weight, epi=EPI_BIAS_GELU, bias=bias, aux=pre_gelu.view(rows, OC), kind=kind)
        elif residual is not None:
            gemm(o, x, weight, epi=EPI_BIAS_RESID, bias=bias, aux=residual.view(rows, OC), kind=kind)
        else:
            gemm(o, x, weight, epi=EPI_BIAS if bias is not None else EPI_NONE, bias=bias, kind=kind)
        return
    y = x @ weight.t()
    if bias is not None:
        y = y + bias
    if pre_gelu is not None:
        pre_gelu.view(rows, OC).copy_(y)
        y = _gelu_t(pre_gelu.view(rows, OC).float())
    if residual is not None:
        y = y + residual.view(rows, OC)
    o.copy_(y)


def matmul_bwd(dinp, dweight, dbias, dout, inp, weight, *, gelu_pre=None, dinp_colsum=None) -> None:
    """dinp = dout·W (⊙ gelu'(gelu_pre)); dweight += doutᵀ·inp; dbias += Σ_rows dout (each output may be None).
    ``dinp_colsum`` (fp32 [C]) += Σ_rows dinp: the bias gradient of the layer whose output gradient dinp is, taken
    inside the dGELU epilogue when the kernel allows it, by a separate reduction otherwise.

    dweight / dbias are fp32 accumulators (llmm/matmul.mojo:3512-3563, DGELU epilogue :2789-2938)."""
    OC, C = weight.shape
    rows = inp.numel() // C
    d = dout.reshape(rows, OC)
    x = inp.reshape(rows, C)
    if dout.is_cuda and GEMM_IMPL == "tcgen05" and _tc_kind(dout) is not None:
        kind = _tc_kind(dout)
        if dinp is not None:
            di = dinp.view(rows, C)
            if gelu_pre is not None:
                aux = gelu_pre.view(rows, C)
                fused = dinp_colsum is not None and kind == 0 and colsum_usable(di, aux)
                gemm(di, d, weight, b_mn=True, epi=EPI_DGELU, aux=aux, kind=kind, colsum=dinp_colsum if fused else None)
                if dinp_colsum is not None and not fused:
                    dbias_reduce(dinp_colsum, di)
            else:
                gemm(di, d, weight, b_mn=True, epi=EPI_NONE, kind=kind)
                if dinp_colsum is not None:
                    dbias_reduce(dinp_colsum, di)
        if dweight is not None:
            gemm(dweight.view(OC, C), d, x, a_mn=True, b_mn=True, epi=EPI_ACC_F32, splits=_splits_for(OC, C, rows), kind=kind)
        if dbias is not None:
            dbias_reduce(dbias, d)
        return
    if dinp is not None:
        g = d @ weight
        if gelu_pre is not None:
            g = g.float() * _gelu_grad_t(gelu_pre.view(rows, C).float())
        dinp.view(rows, C).copy_(g)
        if dinp_colsum is not None:
            dinp_colsum += dinp.view(rows, C).float().sum(0)
    if dweight is not None:
        dweight.view(OC, C).add_((d.t() @ x).float())
    if dbias is not None:
        dbias += d.float().sum(0)


def lm_head_bwd_tile(dinp, dweight_tile, dlogits_tile, inp, weight_tile, accumulate: bool) -> None:
    """One vocabulary tile of the LM-head backward: dinp (+)= dlogits·W_tile, dW_tile += dlogitsᵀ·inp
    (llmm/matmul.mojo:3757-3908; beta=1 accumulation across tiles)."""
    w, C = weight_tile.shape
    rows = inp.numel() // C
    d, x, di = dlogits_tile, inp.reshape(rows, C), dinp.view(rows, C)
    if d.is_cuda and GEMM_IMPL == "tcgen05" and _tc_kind(d) is not None:
        kind = _tc_kind(d)
        if accumulate:      # D = acc + D: the residual epilogue reading the output tile itself
            gemm(di, d, weight_tile, b_mn=True, epi=EPI_BIAS_RESID, aux=di, kind=kind)
        else:
            gemm(di, d, weight_tile, b_mn=True, kind=kind)
        gemm(dweight_tile, d, x, a_mn=True, b_mn=True, epi=EPI_ACC_F32, splits=_splits_for(w, C, rows), kind=kind)
        return
    g = d.float() @ weight_tile.float()
    if accumulate:
        di += g.to(di.dtype)
    else:
        di.copy_(g)
    dweight_tile.add_((d.t().float() @ x.float()))


def dbias_reduce(dbias, dout2d) -> None:
    rows, OC = dout2d.shape
    if dout2d.is_cuda:
        L = lib()
        nb = L.llmb_dbias_scratch_bytes(rows, OC)
        s = scratch("dbias", nb, dout2d.device)
        check(L.llmb_dbias(ptr(dbias), ptr(dout2d), ptr(s), s.numel(), rows, OC, dtype_code(dout2d), stream()), "dbias")
        _count(2)
    else:
        dbias += dout2d.float().sum(0)


# ----------------------------------------------------------------------------- attention
def attention_fwd(out, lse, qkv, num_heads: int) -> None:
    """Causal multi-head attention on packed qkv [B,T,3C] → out [B,T,C], lse [B,NH,T].

    ``lse`` is log2-domain: log2 Σ_j 2^(s_ij·log2e/√d).  (llmm/attention.mojo:1748-1945.)"""
    B, T, C3 = qkv.shape
    C = C3 // 3
    hs = C // num_heads
    if qkv.is_cuda and ATTN_IMPL == "tcgen05" and hs == 64 and qkv.dtype == torch.bfloat16:
        check(lib().llmb_attention_fwd(ptr(out), ptr(lse), ptr(qkv), B, T, num_heads, ptr(status_word(qkv.device)),
                                       stream()), "attention_fwd")
        _count()
        return
    if qkv.is_cuda:      # library comparator (LLMB_ATTN=sdpa) and head sizes other than 64
        q, k, v = (t.view(B, T, num_heads, hs).transpose(1, 2) for t in qkv.split(C, dim=2))
        out.copy_(F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, T, C))
        return
    q, k, v = (t.view(B, T, num_heads, hs).transpose(1, 2) for t in qkv.split(C, dim=2))
    s = (q.float() @ k.float().transpose(-1, -2)) / math.sqrt(hs)
    mask = torch.ones(T, T, dtype=torch.bool, device=qkv.device).tril()
    s = s.masked_fill(~mask, float("-inf"))
    l = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - l.unsqueeze(-1))
    o = (p @ v.float()).transpose(1, 2).reshape(B, T, C)
    out.copy_(o)
    lse.copy_(l * math.log2(math.e))


def attention_bwd(dqkv, dout, qkv, out, lse, num_heads: int, dbias=None) -> None:
    """dqkv = ∂/∂qkv of causal attention (llmm/attention.mojo:5033-5276).  ``dbias`` (fp32 [3C]) += Σ_rows dqkv: the
    gradient of the qkv bias, taken in the kernels' epilogues on the tensor-core path, by a reduction otherwise."""
    B, T, C3 = qkv.shape
    C = C3 // 3
    hs = C // num_heads
    if qkv.is_cuda and ATTN_IMPL == "tcgen05" and hs == 64 and qkv.dtype == torch.bfloat16 and ATTN_BWD == "fused":
        L = lib()
        stats = scratch("attn_bwd_stats", L.llmb_attention_bwd_fused_stats_floats(B, T, num_heads) * 4, qkv.device)
        acc = scratch("attn_bwd_dq_acc", L.llmb_attention_bwd_fused_acc_floats(B, T, num_heads) * 4, qkv.device, zero=True)
        check(L.llmb_attention_bwd_fused(ptr(dqkv), ptr(dbias), ptr(stats), ptr(acc), ptr(dout), ptr(qkv), ptr(out), ptr(lse), B, T,
                                         num_heads, ptr(status_word(qkv.device)), stream()), "attention_bwd_fused")
        _count(3)
        return
    if qkv.is_cuda and ATTN_IMPL == "tcgen05" and hs == 64 and qkv.dtype == torch.bfloat16:
        dvec = scratch("attn_dvec", B * num_heads * (T + 128 * ((T + 63) // 64)) * 4 + 16, qkv.device)
        check(lib().llmb_attention_bwd_dbias(ptr(dqkv), ptr(dbias), ptr(dvec), ptr(dout), ptr(qkv), ptr(out), ptr(lse), B, T,
                                             num_heads, ptr(status_word(qkv.device)), stream()), "attention_bwd")
        _count(3)
        return
    if dbias is not None:
        attention_bwd(dqkv, dout, qkv, out, lse, num_heads)
        dbias_reduce(dbias, dqkv.view(B * T, C3))
        return
    if qkv.is_cuda:      # library comparator: recompute through SDPA under autograd
        with torch.enable_grad():
            leaf = qkv.detach().clone().requires_grad_(True)
            q, k, v = (t.view(B, T, num_heads, hs).transpose(1, 2) for t in leaf.split(C, dim=2))
            o = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, T, C)
            o.backward(dout.view(B, T, C))
        dqkv.copy_(leaf.grad)
        return
    q, k, v = (t.view(B, T, num_heads, hs).transpose(1, 2).float() for t in qkv.split(C, dim=2))
    do = dout.view(B, T, num_heads, hs).transpose(1, 2).float()
    o = out.view(B, T, num_heads, hs).transpose(1, 2).float()
    scale = 1.0 / math.sqrt(hs)
    s = (q @ k.transpose(-1, -2)) * scale
    mask = torch.ones(T, T, dtype=torch.bool, device=qkv.device).tril()
    p = torch.exp(s - (lse / math.log2(math.e)).unsqueeze(-1)).masked_fill(~mask, 0.0)
    dv = p.transpose(-1, -2) @ do
    dp = do @ v.transpose(-1, -2)
    dsum = (do * o).sum(-1, keepdim=True)
    ds = p * (dp - dsum) * scale
    dq = ds @ k
    dk = ds.transpose(-1, -2) @ q
    dqkv.copy_(torch.cat([t.transpose(1, 2).reshape(B, T, C) for t in (dq, dk, dv)], dim=2))


# ----------------------------------------------------------------------------- classifier
def fused_classifier(logits, losses, targets, dloss: float, vocab_size: int, write_dlogits: bool = True) -> None:
    """Per-row softmax cross-entropy; ``logits`` [rows,Vp] is overwritten with
    dlogits = (softmax − onehot)·dloss, padded tail zeroed (llmm/fused_classifier.mojo:311-370)."""
    Vp = logits.shape[-1]
    rows = logits.numel() // Vp
    if logits.is_cuda:
        check(lib().llmb_fused_classifier(ptr(logits), ptr(losses), ptr(targets), float(dloss), rows, vocab_size, Vp,
                                          int(write_dlogits), dtype_code(logits), ptr(status_word(logits.device)), stream()),
              "fused_classifier")
        _count()
    else:
        lg = logits.view(rows, Vp)
        x = lg[:, :vocab_size].float()
        lsm = torch.log_softmax(x, dim=-1)
        t = targets.reshape(rows).long()
        if losses is not None:
            losses.view(rows).copy_(-lsm.gather(1, t.unsqueeze(1)).squeeze(1))
        if write_dlogits:
            p = lsm.exp()
            p.scatter_add_(1, t.unsqueeze(1), torch.full((rows, 1), -1.0, dtype=p.dtype))
            lg[:, :vocab_size] = (p * dloss).to(lg.dtype)
            lg[:, vocab_size:] = 0


def chunked_ce_pass1(stats, tile, targets, col0: int, width: int, vocab_size: int, first: bool) -> None:
    """Merge one vocabulary tile [rows, width] into the per-row running (max, sum-exp, target logit)
    statistics ``stats`` [rows, 4] fp32 (llmm/fused_classifier.mojo:565-629)."""
    rows = stats.shape[0]
    if tile.is_cuda:
        check(lib().llmb_ce_pass1(ptr(stats), ptr(tile), ptr(targets), rows, tile.stride(0), col0, width, vocab_size,
                                  int(first), dtype_code(tile), stream()), "ce_pass1")
        _count()
        return
    valid = max(0, min(width, vocab_size - col0))
    if first:
        stats[:, 0], stats[:, 1], stats[:, 2] = float("-inf"), 0.0, 0.0
    if valid > 0:
        x = tile[:, :valid].float()
        mx = x.max(1).values
        m_new = torch.maximum(stats[:, 0], mx)
        stats[:, 1] = stats[:, 1] * torch.exp(stats[:, 0] - m_new) + torch.exp(x - mx[:, None]).sum(1) * torch.exp(mx - m_new)
        stats[:, 0] = m_new
        t = targets.reshape(rows).long() - col0
        hit = (t >= 0) & (t < valid)
        stats[hit, 2] = x[hit, t[hit]]


def chunked_ce_loss(losses, stats) -> None:
    """losses[row] = logsumexp − target logit from the merged statistics (llmm/fused_classifier.mojo:656)."""
    if stats.is_cuda:
        check(lib().llmb_ce_loss(ptr(losses), ptr(stats), stats.shape[0], stream()), "ce_loss")
        _count()
    else:
        losses.view(-1).copy_(-(stats[:, 2] - stats[:, 0] - torch.log(stats[:, 1])))


def chunked_ce_pass2(tile, stats, targets, col0: int, width: int, vocab_size: int, dloss: float) -> None:
    """Overwrite a recomputed logits tile with dlogits = (softmax − onehot)·dloss; padded columns → 0
    (llmm/fused_classifier.mojo:782-841)."""
    rows = stats.shape[0]
    if tile.is_cuda:
        check(lib().llmb_ce_pass2(ptr(tile), ptr(stats), ptr(targets), rows, tile.stride(0), col0, width, vocab_size,
                                  float(dloss), dtype_code(tile), stream()), "ce_pass2")
        _count()
        return
    lse = stats[:, 0] + torch.log(stats[:, 1])
    x = tile[:, :width].float()
    p = torch.exp(x - lse[:, None])
    t = targets.reshape(rows).long() - col0
    hit = (t >= 0) & (t < width)
    p[hit, t[hit]] -= 1.0
    cols = torch.arange(width, device=tile.device) + col0
    p[:, cols >= vocab_size] = 0.0
    tile[:, :width] = (p * dloss).to(tile.dtype)


def softmax_rows(logits2d: torch.Tensor, vocab_size: int, temperature: float = 1.0) -> torch.Tensor:
    """Row softmax over the first ``vocab_size`` columns → fp32 (llmm/softmax.mojo:306)."""
    rows = logits2d.shape[0]
    if logits2d.is_cuda:
        out = torch.empty(rows, vocab_size, dtype=torch.float32, device=logits2d.device)
        check(lib().llmb_softmax_rows(ptr(out), ptr(logits2d), rows, vocab_size, logits2d.stride(0),
                                      1.0 / temperature, dtype_code(logits2d), stream()), "softmax_rows")
        _count()
        return out
    return torch.softmax(logits2d[:, :vocab_size].float() / temperature, dim=-1)


def softmax_bwd(dprobs: torch.Tensor, probs: torch.Tensor, vocab_size: int) -> torch.Tensor:
    """Gradient of a row softmax with respect to its logits: ``p ∘ (dp − Σ_k dp_k p_k)`` over the first
    ``vocab_size`` columns, zero in the padded tail; fp32 ``[rows, ld]`` in and out (llmm/softmax.mojo:632)."""
    rows, ld = probs.shape
    if probs.is_cuda:
        out = torch.empty_like(probs, dtype=torch.float32)
        check(lib().llmb_softmax_bwd(ptr(out), ptr(dprobs), ptr(probs), rows, vocab_size, ld, stream()), "softmax_bwd")
        _count()
        return out
    p, dp = probs[:, :vocab_size].float(), dprobs[:, :vocab_size].float()
    out = torch.zeros(rows, ld, dtype=torch.float32)
    out[:, :vocab_size] = p * (dp - (dp * p).sum(-1, keepdim=True))
    return out


def crossentropy_fwd(probs: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Unfused cross-entropy over stored probabilities ``[rows, ld]`` fp32: ``−log p[target]``
    (llmm/crossentropy.mojo:110).  The training path uses ``fused_classifier`` instead."""
    rows, ld = probs.shape
    if probs.is_cuda:
        out = torch.empty(rows, dtype=torch.float32, device=probs.device)
        check(lib().llmb_crossentropy_fwd(ptr(out), ptr(probs), ptr(targets), rows, ld, stream()), "crossentropy_fwd")
        _count()
        return out
    return -torch.log(probs.float().gather(1, targets.long().view(-1, 1)).squeeze(1))


def crossentropy_bwd(dprobs: torch.Tensor, dlosses: torch.Tensor, probs: torch.Tensor, targets: torch.Tensor) -> None:
    """Writes ``dprobs[row, target] = −dloss / p[row, target]``; every other entry of ``dprobs`` is left as it is
    (llmm/crossentropy.mojo:284)."""
    rows, ld = probs.shape
    if probs.is_cuda:
        check(lib().llmb_crossentropy_bwd(ptr(dprobs), ptr(dlosses), ptr(probs), ptr(targets), rows, ld, stream()),
              "crossentropy_bwd")
        _count()
        return
    idx = targets.long().view(-1, 1)
    dprobs.scatter_(1, idx, (-dlosses.float().view(-1, 1) / probs.float().gather(1, idx)).to(dprobs.dtype))


# ----------------------------------------------------------------------------- optimizer
def adamw_update(params, master, grads, m, v, *, lr, beta1, beta2, eps, weight_decay, grad_scale, step,
                 seed: int = 0, stochastic_rounding: bool = False, dev_scale=None) -> None:
    """AdamW on a flat (shard of the) parameter vector; wd applies to every element
    (llmm/adamw.mojo:93-211).  ``master`` (fp32) may be None when params are fp32.
    ``dev_scale`` is an optional 1-element device tensor multiplied into ``grad_scale`` so the
    clip factor never has to visit the host."""
    n = grads.numel()
    if grads.is_cuda:
        check(lib().llmb_adamw(ptr(params), ptr(master), ptr(grads), ptr(m), ptr(v), n, lr, beta1, beta2, eps,
                               weight_decay, grad_scale, ptr(dev_scale), step, seed, int(stochastic_rounding), dtype_code(params),
                               stream()), "adamw")
        _count()
    else:
        g = grads.float() * grad_scale
        if dev_scale is not None:
            g = g * dev_scale.float()
        m.mul_(beta1).add_(g, alpha=1 - beta1)
        v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
        mh = m / (1 - beta1 ** step)
        vh = v / (1 - beta2 ** step)
        p = master if master is not None else params.float()
        p = p - lr * (mh / (vh.sqrt() + eps) + weight_decay * p)
        if master is not None:
            master.copy_(p)
        params.copy_(p)


def nan_census(x: torch.Tensor) -> tuple:
    """(number of NaN, number of ±Inf) in ``x`` — the per-tensor debug scan of ``train_gpt2.mojo:5385-5577``."""
    if x.is_cuda and x.dtype in (torch.float32, torch.bfloat16):
        counts = torch.zeros(2, dtype=torch.int32, device=x.device)
        flat = x.reshape(-1)
        check(lib().llmb_nan_census(ptr(counts), ptr(flat), flat.numel(), dtype_code(flat), stream()), "nan_census")
        _count()
        c = counts.tolist()
        return int(c[0]), int(c[1])
    xf = x.float()
    return int(torch.isnan(xf).sum().item()), int(torch.isinf(xf).sum().item())


def global_norm_squared(out, x, accumulate: bool = False) -> None:
    """out[0] (=|+=) Σ x² (fp32; llmm/global_norm.mojo:194-282)."""
    if x.is_cuda:
        L = lib()
        s = scratch("norm_sq", L.llmb_norm_sq_blocks() * 4, x.device)
        check(L.llmb_global_norm_sq(ptr(out), ptr(x), x.numel(), ptr(s), int(accumulate), stream()), "global_norm_sq")
        _count(2)
    else:
        val = (x.double() ** 2).sum().float()
        if accumulate:
            out[0] += val
        else:
            out[0] = val
