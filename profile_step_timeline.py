#!/usr/bin/env python
"""profile_step_timeline — where one data-parallel optimizer step spends its time, on both streams.

Run under torchrun (one process per GPU) or alone.  It performs the headline step (d12, B=64, T=1024, 2**19 tokens per
step split over the ranks, AdamW with clipping) and records CUDA events

* on the main stream: start, end of every forward, end of every backward's kernels, after the join with the
  communication stream, after the gradient norm, after the update;
* per gradient bucket: the moment its gradients are complete (main stream) and the end of its pack -> reduce ->
  unpack chain on the communication stream (the peer-memory kernels of ``csrc/comm.cu``), by wrapping
  ``P2PBackend.reduce_ranges``; the difference is the bucket's latency from "ready" to "reduced on every rank".

From these it prints, per rank and as the maximum over ranks: the span of each phase, how much of the collective
work lies after the last backward kernel (the exposed part), the busy time of the communication stream and the
size of every bucket.  Nothing here runs under a profiler; the events cost a few microseconds per step.

    torchrun --nproc-per-node 8 profile_step_timeline.py --steps 6 [--zero 0] [--json out.json]
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch
import torch.distributed as dist

from llm_mojo_b200.trainer import TrainArgs, Trainer


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--model", default="d12")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--total-batch", type=int, default=2 ** 19)
    ap.add_argument("--zero", type=int, default=0)
    ap.add_argument("--json", default="")
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    targs = TrainArgs(load_filename=a.model, batch_size=a.batch, seq_len=a.seq, total_batch_size=a.total_batch,
                      learning_rate=6e-4, warmup_iterations=10, final_learning_rate_frac=0.1, weight_decay=0.1,
                      zero_stage=a.zero, max_steps=10_000, precision="bf16", grad_clip=1.0, beta2=0.95, synthetic=True,
                      val_loss_every=0, sample_every=0)
    tr = Trainer(targs, rank, world, local)
    m, ga, B, T = tr.model, tr.grad_accum, a.batch, a.seq
    gen = torch.Generator(device="cuda").manual_seed(1234 + rank)
    toks = torch.randint(0, m.config.vocab_size, (B * T + 1,), generator=gen, device="cuda", dtype=torch.int32)
    x, y = toks[:-1].view(B, T).contiguous(), toks[1:].view(B, T).contiguous()

    def ev():
        e = torch.cuda.Event(enable_timing=True)
        return e

    comm_spans = []                                     # (bucket elements, begin event, end event) of the current step
    be = tr.zero.backend if tr.zero is not None else None
    if be is not None and hasattr(be, "stream"):
        orig = be.reduce_ranges

        def wrapped(src, segs, *args, **kw):
            e0, e1 = ev(), ev()
            e0.record()                                 # main stream: the bucket's gradients are complete here
            orig(src, segs, *args, **kw)
            e1.record(be.stream)
            comm_spans.append((sum(n for _, n, _ in segs), e0, e1))
        be.reduce_ranges = wrapped

    rows = []
    for step in range(a.warmup + a.steps):
        comm_spans.clear()
        marks = {"start": ev()}
        marks["start"].record()
        for micro in range(ga):
            m.forward(x, y, ga, B=B, T=T)
            f = ev(); f.record(); marks[f"fwd{micro}"] = f
            last = micro == ga - 1
            if last and tr.zero is not None:
                # split the last backward: its own kernels end before reduce_all joins the streams
                orig_ra = tr.zero.reduce_all
                holder = {}

                def ra():
                    e = ev(); e.record(); holder["bwd_kernels"] = e
                    orig_ra()
                tr.zero.reduce_all = ra
                m.backward(ga, micro)
                tr.zero.reduce_all = orig_ra
                marks["bwd_kernels"] = holder.get("bwd_kernels")
            else:
                m.backward(ga, micro)
            b = ev(); b.record(); marks[f"bwd{micro}"] = b
        norm = m.calculate_grad_norm()
        n_ = ev(); n_.record(); marks["norm"] = n_
        scale = m.clip_scale_from_norm(norm, 1.0)
        m.update(step + 1, tr.scheduler.get_learning_rate(step), 0.1, 1.0, 0.9, 0.95, 1e-8, dev_scale=scale)
        u = ev(); u.record(); marks["update"] = u
        torch.cuda.synchronize()
        m.read_loss()
        if step < a.warmup:
            continue
        t0 = marks["start"]
        last = ga - 1
        r = {"total": t0.elapsed_time(marks["update"]),
             "forward_sum": sum((marks[f"bwd{i - 1}"] if i else t0).elapsed_time(marks[f"fwd{i}"]) for i in range(ga)),
             "backward_sum": sum(marks[f"fwd{i}"].elapsed_time(marks[f"bwd{i}"]) for i in range(ga)),
             "norm": marks[f"bwd{last}"].elapsed_time(marks["norm"]),
             "update": marks["norm"].elapsed_time(marks["update"])}
        if marks.get("bwd_kernels") is not None:
            r["last_backward_kernels"] = marks[f"fwd{last}"].elapsed_time(marks["bwd_kernels"])
            r["exposed_collectives"] = marks["bwd_kernels"].elapsed_time(marks[f"bwd{last}"])
        if comm_spans:
            r["bucket_latency_sum"] = sum(e0.elapsed_time(e1) for _, e0, e1 in comm_spans)
            r["buckets"] = [{"elements": n, "begin_after_step_start": t0.elapsed_time(e0), "ms": e0.elapsed_time(e1),
                             "end_after_last_backward_kernel": (marks["bwd_kernels"].elapsed_time(e1)
                                                               if marks.get("bwd_kernels") is not None else None)}
                            for n, e0, e1 in comm_spans]
        rows.append(r)

    keys = [k for k in rows[0] if k != "buckets"]
    med = {k: statistics.median(r[k] for r in rows) for k in keys}
    t = torch.tensor([med[k] for k in keys], device="cuda", dtype=torch.float64)
    tmax = t.clone()
    if world > 1:
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(f"step timeline, {a.model} B={B} T={T} world={world} zero={a.zero} grad_accum={ga} "
              f"backend={(tr.zero.backend_name if tr.zero else 'none')}; median of {a.steps} steps, ms")
        print(f"{'phase':28s} {'rank 0':>10s} {'max over ranks':>16s}")
        for k, v0, vm in zip(keys, t.tolist(), tmax.tolist()):
            print(f"{k:28s} {v0:10.3f} {vm:16.3f}")
        if "buckets" in rows[-1]:
            print("collective chains of the last step on the communication stream (rank 0):")
            print(f"{'#':>3s} {'elements':>12s} {'ready (ms after step start)':>28s} {'ready->reduced':>14s} {'end after last backward kernel':>32s}")
            for i, b in enumerate(rows[-1]["buckets"]):
                tail = "" if b["end_after_last_backward_kernel"] is None else f"{b['end_after_last_backward_kernel']:32.3f}"
                print(f"{i:3d} {b['elements']:12d} {b['begin_after_step_start']:28.3f} {b['ms']:14.3f} {tail}")
        if a.json:
            with open(a.json, "w") as f:
                json.dump({"world": world, "zero": a.zero, "median_rank0": dict(zip(keys, t.tolist())),
                           "median_max": dict(zip(keys, tmax.tolist())), "last_step_buckets": rows[-1].get("buckets")}, f, indent=1)
    if world > 1:
        dist.barrier()
        if tr.zero is not None:
            tr.zero.close()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
