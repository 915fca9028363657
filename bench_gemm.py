#!/usr/bin/env python
"""bench_gemm — the tcgen05 GEMM on the GPT-2 training shapes against cuBLAS (torch.matmul).

Parity: ``bench_gemm.mojo:1-60`` (candidate kernels vs the library GEMM on the real model shapes).
Prints one row per (shape, variant): forward (K-major x K-major), dinp (B stored [K,N]) and dW (both
operands stored [K,·], split-K with fp32 red.add), in CTA-pair and single-CTA tile modes, as TF/s and as
a fraction of the measured cuBLAS bf16 peak in MEASURED_PEAKS.json when that file is present.

``--layer`` times the calls a transformer block actually makes (``ops.matmul_fwd`` / ``ops.matmul_bwd`` with their
fused bias, GELU, dGELU and residual epilogues, dinp + dW + dbias for the backward) with a 256 MB L2 flush between
timed launches; ``LLMB_GEMM_TMA_EPI=0`` selects the register/shared-memory epilogue for comparison."""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

from llm_mojo_b200 import ops
from llm_mojo_b200.config import parse_model_descriptor
from llm_mojo_b200.ops import _lib


def timed(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def timed_flushed(fn, iters=10, warmup=3):
    """Per-launch CUDA-event time with an L2 flush (a 256 MB memset) between launches."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    total = 0.0
    for _ in range(iters):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return total / iters


def layer_calls(C: int, rows: int, Vp: int) -> None:
    bf = torch.bfloat16

    def rnd(*shape):
        return (torch.randn(*shape, device="cuda") * 0.05).to(bf)

    for name, OC, K, mode in [("qkv", 3 * C, C, "bias"), ("attproj", C, C, "resid"), ("fc", 4 * C, C, "gelu"),
                              ("fcproj", C, 4 * C, "resid"), ("lm_head", Vp, C, "none")]:
        x, w, b = rnd(rows, K), rnd(OC, K), rnd(OC)
        out = torch.empty(rows, OC, device="cuda", dtype=bf)
        aux = torch.empty(rows, OC, device="cuda", dtype=bf)
        if mode == "bias":
            fn = lambda: ops.matmul_fwd(out, x, w, b)
        elif mode == "resid":
            fn = lambda: ops.matmul_fwd(out, x, w, b, residual=aux)
        elif mode == "gelu":
            fn = lambda: ops.matmul_fwd(out, x, w, b, pre_gelu=aux)
        else:
            fn = lambda: ops.matmul_fwd(out, x, w, None)
        ms = timed_flushed(fn)
        print(f"fwd {name:8s} ({mode:5s}) {ms:.3f} ms {2.0 * rows * OC * K / ms / 1e9:6.0f} TF/s")
        if name == "lm_head":
            continue
        dinp = torch.empty(rows, K, device="cuda", dtype=bf)
        dw = torch.zeros(OC, K, device="cuda")
        db = torch.zeros(OC, device="cuda")
        gelu_pre = rnd(rows, K) if name == "fcproj" else None      # fcproj's input gradient passes through dGELU
        ms = timed_flushed(lambda: ops.matmul_bwd(dinp, dw, db, out, x, w, gelu_pre=gelu_pre))
        print(f"bwd {name:8s} (dinp{'+dGELU' if gelu_pre is not None else ''}, dW, dbias) {ms:.3f} ms {4.0 * rows * OC * K / ms / 1e9:6.0f} TF/s")


def lowp_rows(shapes, rows: int) -> None:
    """bf16, fp8 and NVFP4 forward products of the same shapes (operands quantised outside the timed region)."""
    from llm_mojo_b200.ops import lowp
    one = torch.ones(1, device="cuda")
    for name, N, K in shapes:
        A = torch.randn(rows, K, device="cuda").bfloat16()
        W = (torch.randn(N, K, device="cuda") * 0.02).bfloat16()
        D = torch.empty(rows, N, device="cuda", dtype=torch.bfloat16)
        fl = 2.0 * rows * N * K
        ms = timed_flushed(lambda: ops.gemm(D, A, W))
        print(f"{name:8s} {rows}x{N}x{K}  bf16  {ms:.3f} ms {fl / ms / 1e9:7.0f} TF/s")
        qa = torch.empty(rows, K, dtype=torch.uint8, device="cuda")
        qw = torch.empty(N, K, dtype=torch.uint8, device="cuda")
        lowp.quantize_fp8(qa, A, one, lowp.E4M3)
        lowp.quantize_fp8(qw, W, one * 16, lowp.E4M3)
        ms = timed_flushed(lambda: ops.gemm(D, qa, qw, alpha=one, kind=2, a_fmt=lowp.E4M3, b_fmt=lowp.E4M3))
        print(f"   fp8 (per-tensor scale, CTA-pair 256x256 tiles)        {ms:.3f} ms {fl / ms / 1e9:7.0f} TF/s")
        if rows % 128 == 0 and N % 128 == 0 and K % 128 == 0:
            ba, sfa = lowp.fp8_block_quant(A, 0, lowp.E4M3)
            bw, sfw = lowp.fp8_block_quant(W, 2, lowp.E4M3)
            ms = timed_flushed(lambda: ops.gemm_mxfp8(D, ba, sfa, bw, sfw))
            print(f"   fp8, per-128 block scales (MXFP8 tensor path, 128x256 tiles) {ms:.3f} ms {fl / ms / 1e9:7.0f} TF/s")
        if K % 32 == 0:
            _, tsa, pa, sa = lowp.nvfp4_fake_quant(A, axis=1, block_rows=1, want_packed=True, want_deq=False)
            _, tsw, pw, sw = lowp.nvfp4_fake_quant(W, axis=1, block_rows=16, want_packed=True, want_deq=False)
            al = tsa * tsw
            ms = timed_flushed(lambda: ops.gemm_nvfp4(D, pa, sa, pw, sw, K, alpha=al))
            print(f"   nvfp4 (block-scaled tensor path, 128x256 tiles)       {ms:.3f} ms {fl / ms / 1e9:7.0f} TF/s")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="d12")
    ap.add_argument("-b", type=int, default=64)
    ap.add_argument("-t", type=int, default=1024)
    ap.add_argument("--modes", default="1,0", help="1 = CTA-pair tiles, 0 = single-CTA tiles")
    ap.add_argument("--layer", action="store_true", help="time the fused per-layer calls with an L2 flush between launches")
    ap.add_argument("--lowp", action="store_true", help="forward GEMMs on the fp8 (kind::f8f6f4) and NVFP4 (kind::mxf4nvf4) tensor paths")
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("bench_gemm needs a GPU")
        return 0
    cfg = parse_model_descriptor(a.model)
    C, rows = cfg.channels, a.b * a.t
    if a.layer:
        layer_calls(C, rows, cfg.padded_vocab_size)
        print("kernel status", _lib.read_status())
        return 0
    peak = None
    pk = os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peak = json.load(open(pk)).get("bf16_tflops")
    shapes = [("qkv", 3 * C, C), ("attproj", C, C), ("fc", 4 * C, C), ("fcproj", C, 4 * C), ("lm_head", cfg.padded_vocab_size, C)]
    if a.lowp:
        lowp_rows(shapes[:4], rows)
        print("kernel status", _lib.read_status())
        return 0
    for name, N, K in shapes:
        A = torch.randn(rows, K, device="cuda").bfloat16()
        W = (torch.randn(N, K, device="cuda") * 0.02).bfloat16()
        D = torch.empty(rows, N, device="cuda", dtype=torch.bfloat16)
        fl = 2.0 * rows * N * K
        lib_ms = timed(lambda: torch.matmul(A, W.t(), out=D))
        print(f"{name:8s} {rows}x{N}x{K}  cuBLAS fwd {lib_ms:.3f} ms {fl / lib_ms / 1e9:7.0f} TF/s")
        for mode in [int(m) for m in a.modes.split(",")]:
            _lib.lib().llmb_gemm_set_pair_mode(mode)
            tag = "pair  " if mode else "single"
            ms = timed(lambda: ops.gemm(D, A, W))
            frac = f" ({fl / ms / 1e9 / peak:.2f} of measured)" if peak else ""
            print(f"   {tag} fwd  {ms:.3f} ms {fl / ms / 1e9:7.0f} TF/s{frac}")
            dA = torch.empty(rows, K, device="cuda", dtype=torch.bfloat16)
            ms = timed(lambda: ops.gemm(dA, D, W, b_mn=True))
            print(f"   {tag} dinp {ms:.3f} ms {fl / ms / 1e9:7.0f} TF/s")
            dW = torch.zeros(N, K, device="cuda")
            sp = ops._splits_for(N, K, rows)
            ms = timed(lambda: ops.gemm(dW, D, A, a_mn=True, b_mn=True, epi=ops.EPI_ACC_F32, splits=sp))
            print(f"   {tag} dW   {ms:.3f} ms {fl / ms / 1e9:7.0f} TF/s (split-K {sp})")
        _lib.lib().llmb_gemm_set_pair_mode(1)
    print("kernel status", _lib.read_status())
    return 0


if __name__ == "__main__":
    sys.exit(main())
