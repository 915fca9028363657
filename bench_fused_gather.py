#!/usr/bin/env python
"""bench_fused_gather — the vocabulary-parallel LM-head forward as ONE kernel (all-gather fused into the GEMM, copier
warps pulling the peers' activation rows over NVLink inside the tcgen05 tile loop) against all-gather followed by
the same GEMM.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 bench_fused_gather.py [--rows 65536]

Per rank: A chunk [rows, 768] bf16, weight slice [ceil(50304 / W / 8) * 8, 768], output [W * rows, slice].  Times are
CUDA events on the launching stream (3 warm-up + 10 timed), max over ranks.  Roofline of the fused kernel = the slower
of FLOPs / measured cuBLAS bf16 peak and bytes received over NVLink / 770 GB/s (measured peer-copy rate per direction)."""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from llm_mojo_b200 import ops
from llm_mojo_b200.parallel.runtime import init_distributed
from llm_mojo_b200.parallel.zero import FusedRowGather

WARMUP, ITERS = 3, 10


def timed(fn):
    for _ in range(WARMUP):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(ITERS):
        fn()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / ITERS], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=65536, help="activation rows per rank (multiple of 256)")
    ap.add_argument("--channels", type=int, default=768)
    ap.add_argument("--vocab", type=int, default=50304)
    a = ap.parse_args()
    ctx = init_distributed()
    rank, W, dev = ctx.rank, ctx.world_size, ctx.device
    n, K = a.rows, a.channels
    N = ((a.vocab + W - 1) // W + 7) // 8 * 8
    fg = FusedRowGather(rank, W, dev, n, K)
    fg.local.copy_((torch.randn(n, K, device=dev) * 0.05).bfloat16())
    wt = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
    out = torch.empty(W * n, N, device=dev, dtype=torch.bfloat16)
    ref = torch.empty_like(out)
    gathered = torch.empty(W * n, K, device=dev, dtype=torch.bfloat16)

    def unfused():
        dist.all_gather_into_tensor(gathered, fg.local)
        ops.gemm(ref, gathered, wt)

    def fused():
        fg.wait_released()
        fg.gemm(out, wt)

    def gemm_only():
        ops.gemm(ref, gathered, wt)

    t_unf, t_fus, t_gemm = timed(unfused), timed(fused), timed(gemm_only)
    torch.cuda.synchronize()
    err = (out.float() - ref.float()).abs().max().item()
    if rank == 0:
        flops = 2.0 * W * n * N * K
        nvl = (W - 1) * n * K * 2
        peak = 1620.4e12
        pk = os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")
        if os.path.exists(pk):
            peak = json.load(open(pk)).get("bf16_tflops", 1620.4) * 1e12
        roof_ms = max(flops / peak, nvl / 770e9) * 1e3
        print(json.dumps({"world": W, "rows_per_rank": n, "K": K, "N_slice": N, "fused_ms": round(t_fus, 4),
                          "allgather_then_gemm_ms": round(t_unf, 4), "gemm_alone_ms": round(t_gemm, 4),
                          "roofline_ms": round(roof_ms, 4), "fused_fraction_of_roofline": round(roof_ms / t_fus, 3),
                          "nvlink_bytes_per_rank": nvl, "max_abs_diff_vs_unfused": err, "kernel_status": ops._lib.read_status()}))
    dist.barrier()
    fg.arena.close()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
