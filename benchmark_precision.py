#!/usr/bin/env python
"""benchmark_precision — step time of every training precision on one model, same recipe, one GPU.

Parity: the per-precision arms of ``scripts/benchmark_train.py`` / ``scripts/benchmark_precision.py`` and the
low-precision scaling sweep the reference publishes (bf16 / fp8 / nvfp4 ms per step on d12 ... d36): all arms share
model, batch, schedule and data (synthetic uniform tokens) and differ only in GEMM precision, so the ratio to bf16
is the cost or gain of the precision path itself.  Prints one table row per arm and a JSON blob.

    python benchmark_precision.py --model d36 -b 16 --steps 8 --arms bf16,fp8,fp8b,fp4 [--fp8-static-scales t.json]
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys

import torch

from llm_mojo_b200.trainer import TrainArgs, Trainer


def run_arm(model: str, precision: str, B: int, T: int, steps: int, warmup: int, static_scales: str) -> dict:
    args = TrainArgs(load_filename=model, batch_size=B, seq_len=T, total_batch_size=B * T, learning_rate=3e-4,
                     max_steps=steps + warmup + 1, precision=precision, synthetic=True, val_loss_every=0, sample_every=0,
                     fp8_static_scales=static_scales if precision == "fp8" else "")
    tr = Trainer(args)
    ms, losses = [], []
    for i in range(warmup + steps):
        r = tr.train_step()
        if i >= warmup:
            ms.append(r.get("device_ms", r["ms"]))
        losses.append(r["loss"])
    del tr
    torch.cuda.empty_cache() if torch.cuda.is_available() else None
    med = statistics.median(ms)
    return {"precision": precision + ("+static" if args.fp8_static_scales else ""), "ms_per_step": med,
            "tok_per_s": B * T / (med / 1e3), "first_loss": losses[0], "last_loss": losses[-1]}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="d12")
    ap.add_argument("-b", type=int, default=16)
    ap.add_argument("-t", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--arms", default="bf16,fp8,fp8b,fp4")
    ap.add_argument("--fp8-static-scales", default="", help="adds an fp8 arm with static scales from this table")
    a = ap.parse_args(argv)
    arms = [(p, "") for p in a.arms.split(",") if p]
    if a.fp8_static_scales:
        arms.append(("fp8", a.fp8_static_scales))
    rows = [run_arm(a.model, p, a.b, a.t, a.steps, a.warmup, s) for p, s in arms]
    base = next((r["ms_per_step"] for r in rows if r["precision"] == "bf16"), rows[0]["ms_per_step"])
    print(f"| precision | ms/step | tok/s | x bf16 step time | loss first -> last |  ({a.model}, B={a.b}, T={a.t})")
    print("|---|---|---|---|---|")
    for r in rows:
        r["vs_bf16"] = r["ms_per_step"] / base
        print(f"| {r['precision']} | {r['ms_per_step']:.2f} | {r['tok_per_s']:.0f} | {r['vs_bf16']:.3f} | "
              f"{r['first_loss']:.3f} -> {r['last_loss']:.3f} |")
    print("BENCH_JSON " + json.dumps({"model": a.model, "B": a.b, "T": a.t, "rows": rows}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
