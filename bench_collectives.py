#!/usr/bin/env python
"""bench_collectives — all-reduce / reduce-scatter / all-gather sweep of the peer-memory kernels,
with NCCL (torch.distributed) as the comparison column.

Parity: ``bench_collectives.mojo:46-200``: 3 warm-up + 10 timed iterations per size, one ``BENCH_ROW``
line per (collective, size) and a final ``BENCH_JSON`` line.  Launch with torchrun:

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 bench_collectives.py

Times are CUDA events on the launching stream, max over ranks.  Bus bandwidth uses the usual
conventions: all-reduce 2·(W-1)/W·bytes, reduce-scatter / all-gather (W-1)/W·bytes; "bytes" is the fp32
payload on the caller's side (our kernels move bf16 on the wire, which is part of the design)."""
from __future__ import annotations

import json
import os
import sys

import torch
import torch.distributed as dist

WARMUP, ITERS = 3, 10
SIZES_MIB = (0.75, 12, 96, 240, 474.8)


def timed(fn, sync):
    for _ in range(WARMUP):
        fn()
    sync()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(ITERS):
        fn()
    sync_stream()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / ITERS], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


_backend = None


def sync_stream():
    if _backend is not None:
        _backend.sync()


def main() -> int:
    global _backend
    rank, W = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    if not torch.cuda.is_available() or W < 2:
        print("bench_collectives needs >= 2 GPUs (run under torchrun)")
        return 0
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from llm_mojo_b200.parallel.zero import P2PBackend, shard_size
    max_n = int(max(SIZES_MIB) * (1 << 20) / 4)
    max_n = (max_n + 8 * W - 1) // (8 * W) * (8 * W)
    be = P2PBackend(rank, W, torch.device("cuda", local), max_n, shard_size(max_n, W))
    _backend = be
    rows = []

    def barrier():
        be.sync()
        torch.cuda.synchronize()
        dist.barrier()

    for mib in SIZES_MIB:
        n = int(mib * (1 << 20) / 4)
        n = (n + 8 * W - 1) // (8 * W) * (8 * W)
        S = n // W
        buf = torch.randn(n, device="cuda")
        shard = torch.zeros(S, device="cuda")
        window = torch.empty(n, dtype=torch.bfloat16, device="cuda")
        nbytes = n * 4
        res = {}
        res["allreduce"] = timed(lambda: be.reduce_ranges(buf, [(0, n, 0)], (rank * S, (rank + 1) * S), None, False, True), barrier)
        res["reducescatter"] = timed(lambda: be.reduce_ranges(buf, [(0, n, 0)], (rank * S, (rank + 1) * S), shard, False, False), barrier)
        res["allgather"] = timed(lambda: be.gather_ranges(None, S, [(0, n, 0)], window), barrier)
        # NCCL on equal terms: our kernels put bf16 on the wire (the fp32 -> bf16 cast and the 1/W scale are fused
        # into the pack), so the library moves a bf16 tensor of the same element count; the fp32 run is kept beside
        # it because that is what the torch.distributed backend of the engine actually sends.
        nc, nc32 = {}, {}
        buf16 = buf.bfloat16()
        out16 = torch.empty(S, dtype=torch.bfloat16, device="cuda")
        full16 = torch.empty(n, dtype=torch.bfloat16, device="cuda")
        nc["allreduce"] = timed(lambda: dist.all_reduce(buf16), barrier)
        nc["reducescatter"] = timed(lambda: dist.reduce_scatter_tensor(out16, buf16), barrier)
        nc["allgather"] = timed(lambda: dist.all_gather_into_tensor(full16, out16), barrier)
        out = torch.empty(S, device="cuda")
        nc32["allreduce"] = timed(lambda: dist.all_reduce(buf), barrier)
        nc32["reducescatter"] = timed(lambda: dist.reduce_scatter_tensor(out, buf), barrier)
        nc32["allgather"] = nc["allgather"]                  # parameters are bf16 in both backends
        for coll, factor in (("allreduce", 2 * (W - 1) / W), ("reducescatter", (W - 1) / W), ("allgather", (W - 1) / W)):
            wire = n * 2                                      # bytes per rank on the wire: bf16 in our kernels
            row = {"collective": coll, "mib": mib, "world": W, "elements": n, "wire_dtype": "bf16",
                   "ms": res[coll], "busbw_gbs": factor * wire / res[coll] / 1e6,
                   "nccl_bf16_ms": nc[coll], "nccl_bf16_busbw_gbs": factor * wire / nc[coll] / 1e6,
                   "nccl_fp32_ms": nc32[coll]}
            rows.append(row)
            if rank == 0:
                print(f"BENCH_ROW {coll:14s} {mib:7.2f} MiB fp32 src ({n} elements, bf16 wire)  ours {row['ms']:.3f} ms "
                      f"{row['busbw_gbs']:.1f} GB/s | nccl bf16 {row['nccl_bf16_ms']:.3f} ms {row['nccl_bf16_busbw_gbs']:.1f} GB/s"
                      f" | nccl fp32 {row['nccl_fp32_ms']:.3f} ms", flush=True)
    from llm_mojo_b200.ops import _lib
    status = _lib.read_status()
    if rank == 0:
        print("BENCH_JSON " + json.dumps({"world": W, "status": status, "rows": rows}), flush=True)
    barrier()
    be.close()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
