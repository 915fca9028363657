#!/usr/bin/env python
"""Run ONE hot kernel family on a small, L2-exceeding case so that a profiler capture ends in seconds.

    python profile_kernels.py attn        # flash attention forward + backward, B=32 T=1024 NH=12
    python profile_kernels.py gemm        # fc GEMM with the fused bias+GELU epilogue, its dinp (dGELU) and dW GEMMs
    python profile_kernels.py lmhead      # LM-head GEMM on 8192 rows + fused softmax/cross-entropy
    python profile_kernels.py layernorm   # LayerNorm forward + backward on 65536 x 768
    python profile_kernels.py fusedpull   # a layer GEMM that pulls its own weight (four emulated owners) with its copier warps
    python profile_kernels.py fusedgather # the all-gather-fused GEMM with four "ranks" emulated on ONE GPU: the peers'
                                          # chunks are other local buffers and their flags are preset, so the single
                                          # kernel (copier warps + tile loop) runs exactly as on a rank of a 4-GPU job

Each case launches its kernels `--reps` times (default 2) and prints the device status word.  Meant to be run
plain first and then under `ncu -k regex:<kernel> -c <n>` with the same command line; the per-step counterpart
that times the whole model is profile_gpt2.py (reference: profile_gpt2.mojo / profile_gpt2cu.py).
"""
import argparse

import torch

from llm_mojo_b200 import ops


def case_attn(reps):
    B, T, NH, C = 32, 1024, 12, 768
    qkv = torch.randn(B, T, 3 * C, device="cuda").bfloat16()
    out = torch.empty(B, T, C, device="cuda", dtype=torch.bfloat16)
    lse = torch.empty(B, NH, T, device="cuda")
    dqkv = torch.empty_like(qkv)
    dout = torch.randn(B, T, C, device="cuda").bfloat16()
    for _ in range(reps):
        ops.attention_fwd(out, lse, qkv, NH)
        ops.attention_bwd(dqkv, dout, qkv, out, lse, NH)


def case_gemm(reps):
    rows, C = 32768, 768
    x = torch.randn(rows, C, device="cuda").bfloat16()
    w = (torch.randn(4 * C, C, device="cuda") * 0.02).bfloat16()
    b = torch.zeros(4 * C, device="cuda", dtype=torch.bfloat16)
    pre = torch.empty(rows, 4 * C, device="cuda", dtype=torch.bfloat16)
    act = torch.empty_like(pre)
    dx = torch.empty_like(x)
    dw = torch.zeros(4 * C, C, device="cuda")
    db = torch.zeros(4 * C, device="cuda")
    w2 = (torch.randn(C, 4 * C, device="cuda") * 0.02).bfloat16()
    dw2 = torch.zeros(C, 4 * C, device="cuda")
    dact = torch.empty_like(pre)
    dy = torch.randn(rows, C, device="cuda").bfloat16()
    for _ in range(reps):
        ops.matmul_fwd(act, x, w, b, pre_gelu=pre)                       # bias + GELU epilogue, two outputs
        ops.matmul_bwd(dact, dw2, None, dy, act, w2, gelu_pre=pre)       # fcproj backward: dGELU epilogue on dinp
        ops.matmul_bwd(dx, dw, db, dact, x, w)                           # fc backward: dinp (B MN-major), split-K dW


def case_lmhead(reps):
    rows, C, V, Vp = 8192, 768, 50257, 50304
    x = torch.randn(rows, C, device="cuda").bfloat16()
    w = (torch.randn(Vp, C, device="cuda") * 0.02).bfloat16()
    logits = torch.empty(rows, Vp, device="cuda", dtype=torch.bfloat16)
    losses = torch.empty(rows, device="cuda")
    tgt = torch.randint(0, V, (rows,), device="cuda", dtype=torch.int32)
    for _ in range(reps):
        ops.matmul_fwd(logits, x, w)
        ops.fused_classifier(logits, losses, tgt, 1.0 / rows, V)


def case_layernorm(reps):
    rows, C = 65536, 768
    x = torch.randn(rows, C, device="cuda").bfloat16()
    w = torch.ones(C, device="cuda", dtype=torch.bfloat16)
    b = torch.zeros(C, device="cuda", dtype=torch.bfloat16)
    o = torch.empty_like(x)
    mean = torch.empty(rows, device="cuda")
    rstd = torch.empty(rows, device="cuda")
    dx = torch.zeros_like(x)
    dw = torch.zeros(C, device="cuda")
    db = torch.zeros(C, device="cuda")
    dout = torch.randn(rows, C, device="cuda").bfloat16()
    for _ in range(reps):
        ops.layernorm_fwd(o, mean, rstd, x, w, b)
        ops.layernorm_bwd(dx, dw, db, dout, x, w, mean, rstd)


def case_fusedgather(reps):
    import ctypes
    from llm_mojo_b200.ops import _lib
    W, me, n, K, N = 4, 1, 8192, 768, 6288
    L = _lib.lib()
    P, I, U, LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint, ctypes.c_longlong
    L.llmb_gemm_set_gather.argtypes = [P, P, P, P, LL, U, I, I, I]
    L.llmb_gemm_set_gather.restype = None
    peers = [(torch.randn(n, K, device="cuda") * 0.05).bfloat16() for _ in range(W)]     # chunk r as rank r holds it
    local = torch.zeros(W * n, K, device="cuda", dtype=torch.bfloat16)
    local[me * n:(me + 1) * n] = peers[me]
    wt = (torch.randn(N, K, device="cuda") * 0.02).bfloat16()
    out = torch.empty(W * n, N, device="cuda", dtype=torch.bfloat16)
    flags = torch.full((64,), 1 << 20, dtype=torch.int32, device="cuda")                 # every rank has announced every sequence
    counts = torch.zeros(16, dtype=torch.int32, device="cuda")
    src = (ctypes.c_void_p * 8)(*[t.data_ptr() for t in peers])
    for rep in range(reps):
        counts.zero_()
        L.llmb_gemm_set_gather(src, local.data_ptr(), flags.data_ptr(), counts.data_ptr(), n * K * 2, rep + 1, W, me, n)
        ops.gemm(out, local, wt)
    torch.cuda.synchronize()
    want = torch.cat(peers).float() @ wt.float().t()
    print("max abs diff vs fp32 reference", (out.float() - want).abs().max().item())


def case_fusedpull(reps):
    """The ZeRO-3 weight pull inside a layer GEMM, with four "owners" emulated on ONE GPU: the segments of the weight
    live in four other local buffers, the copier warps of the kernel copy them into the window the GEMM reads as its B
    operand while the tile loop waits for them only at its start - exactly what a rank of a 4-GPU job runs, minus NVLink."""
    import ctypes
    from llm_mojo_b200.ops import _lib
    rows, C, OC = 32768, 768, 3072
    L = _lib.lib()
    P, I, U, LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint, ctypes.c_longlong
    L.llmb_gemm_set_pull.argtypes = [ctypes.POINTER(P), ctypes.POINTER(P), ctypes.POINTER(LL), ctypes.POINTER(I), I, P, U, P,
                                     ctypes.POINTER(P), ctypes.POINTER(LL), I, I]
    L.llmb_gemm_set_pull.restype = I
    x = torch.randn(rows, C, device="cuda").bfloat16()
    w_true = (torch.randn(OC, C, device="cuda") * 0.02).bfloat16()
    nseg = 4
    pieces = [w_true.view(-1)[i * (OC * C // nseg):(i + 1) * (OC * C // nseg)].clone() for i in range(nseg)]    # the "owners' shards"
    window = torch.zeros(OC, C, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(rows, OC, device="cuda", dtype=torch.bfloat16)
    bias = torch.zeros(OC, device="cuda", dtype=torch.bfloat16)
    flags = torch.zeros(256, dtype=torch.int32, device="cuda")
    counts = torch.zeros(16, dtype=torch.int32, device="cuda")
    seg_bytes = OC * C // nseg * 2
    for rep in range(reps):
        window.zero_()
        counts.zero_()
        src = (P * 8)(*[t.data_ptr() for t in pieces])
        dst = (P * 8)(*[window.data_ptr() + i * seg_bytes for i in range(nseg)])
        nb = (LL * 8)(*([seg_bytes] * nseg))
        own = (I * 8)(*range(nseg))
        wc = (P * 8)(*[counts.data_ptr() + 4 * i for i in range(nseg)])
        assert L.llmb_gemm_set_pull(src, dst, nb, own, nseg, flags.data_ptr(), 0, counts.data_ptr(), wc, nb, nseg, nseg) == 0
        ops.gemm(out, x, window, epi=ops.EPI_BIAS, bias=bias)
    torch.cuda.synchronize()
    want = x.float() @ w_true.float().t()
    print("max abs diff vs fp32 reference", (out.float() - want).abs().max().item(), "| window == weight:", bool(torch.equal(window, w_true)))


def case_nvfp4(reps):
    """NVFP4 linear layer pieces: stochastic-rounding quantise (both orientations), native block-scaled GEMM."""
    from llm_mojo_b200.ops import lowp
    rows, C, OC = 8192, 1600, 6400
    x = torch.randn(rows, C, device="cuda").bfloat16()
    w = (torch.randn(OC, C, device="cuda") * 0.02).bfloat16()
    d = torch.randn(rows, OC, device="cuda").bfloat16()
    out = torch.empty(rows, OC, device="cuda", dtype=torch.bfloat16)
    dinp = torch.empty(rows, C, device="cuda", dtype=torch.bfloat16)
    dw = torch.zeros(OC, C, device="cuda")
    for i in range(reps):
        lowp.matmul_fwd_fp4(out, x, w, None)
        lowp.matmul_bwd_fp4(dinp, dw, None, d, x, w, seed=1, step=i)


CASES = {"nvfp4": case_nvfp4, "fusedgather": case_fusedgather, "fusedpull": case_fusedpull, "attn": case_attn, "gemm": case_gemm, "lmhead": case_lmhead, "layernorm": case_layernorm}

if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("case", choices=sorted(CASES))
    ap.add_argument("--reps", type=int, default=2)
    a = ap.parse_args()
    torch.manual_seed(0)
    CASES[a.case](a.reps)
    torch.cuda.synchronize()
    print("ok, kernel status", ops._lib.read_status())
