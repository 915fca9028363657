#!/usr/bin/env python
"""record_run_result — turn one finished training run's own artefacts into a JSON fragment and a results table.

Parity: ``scripts/record_arm_result.py`` + ``scripts/update_readme_results.py`` + the HellaSwag part of
``scripts/benchmark_eval.py``: everything is parsed from what the run wrote (the trainer's log lines, the output of
``infer_gpt2.py --eval``), nothing is typed in by hand, so a published table cannot drift from the run.

    python record_run_result.py record --name 124M-bf16 --log train.log [--eval eval.log] [--out-dir results]
    python record_run_result.py table  [--out-dir results]        # Markdown table of every fragment present

A fragment holds: steps, tokens per step (from the first line's tok/s and ms), median ms/step and tok/s over the last
half of the run, final and best validation loss, HellaSwag accuracy with its Wilson 95 % interval.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import re
import statistics
import sys

STEP_RE = re.compile(r"^step\s+(\d+)/(\d+) \| loss ([0-9.]+).*?\| ([0-9.]+) ms .*?\| (\d+) tok/s", re.M)
VAL_RE = re.compile(r"^val loss ([0-9.]+)", re.M)
HELLA_RE = re.compile(r"HellaSwag: (\d+)/(\d+)")


def wilson(k: int, n: int, z: float = 1.96):
    """Wilson score interval of a proportion: better than ±1.96·SE near the edges and for moderate n."""
    if n == 0:
        return (float("nan"), float("nan"))
    p = k / n
    den = 1 + z * z / n
    mid = (p + z * z / (2 * n)) / den
    half = z * math.sqrt(p * (1 - p) / n + z * z / (4 * n * n)) / den
    return (mid - half, mid + half)


def parse_log(text: str) -> dict:
    steps = [(int(a), int(b), float(l), float(ms), int(t)) for a, b, l, ms, t in STEP_RE.findall(text)]
    if not steps:
        raise ValueError("no step lines found in the log")
    tail = steps[len(steps) // 2:]
    vals = [float(v) for v in VAL_RE.findall(text)]
    ms, tok = statistics.median(s[3] for s in tail), statistics.median(s[4] for s in tail)
    return {"steps_run": steps[-1][0], "steps_planned": steps[-1][1], "final_train_loss": steps[-1][2],
            "ms_per_step_median": ms, "tok_per_s_median": tok, "tokens_per_step": round(tok * ms / 1e3),
            "val_loss_final": vals[-1] if vals else None, "val_loss_best": min(vals) if vals else None}


def record(name: str, log: str, eval_log: str, out_dir: str) -> dict:
    res = {"name": name, **parse_log(open(log).read())}
    if eval_log:
        m = HELLA_RE.search(open(eval_log).read())
        if m:
            k, n = int(m.group(1)), int(m.group(2))
            lo, hi = wilson(k, n)
            res["hellaswag"] = {"correct": k, "total": n, "acc_norm": k / n, "wilson95": [lo, hi]}
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, name + ".json"), "w") as f:
        json.dump(res, f, indent=1)
    return res


def table(out_dir: str) -> str:
    rows = []
    for fn in sorted(os.listdir(out_dir)) if os.path.isdir(out_dir) else []:
        if fn.endswith(".json"):
            rows.append(json.load(open(os.path.join(out_dir, fn))))
    lines = ["| run | steps | tok/step | ms/step | tok/s | val loss | HellaSwag acc_norm (95 % CI) |", "|---|---|---|---|---|---|---|"]
    for r in rows:
        h = r.get("hellaswag")
        hs = f"{100 * h['acc_norm']:.2f} % ({100 * h['wilson95'][0]:.2f}-{100 * h['wilson95'][1]:.2f})" if h else "-"
        vl = f"{r['val_loss_final']:.4f}" if r.get("val_loss_final") is not None else "-"
        lines.append(f"| {r['name']} | {r['steps_run']}/{r['steps_planned']} | {r['tokens_per_step']} | "
                     f"{r['ms_per_step_median']:.2f} | {r['tok_per_s_median']:.0f} | {vl} | {hs} |")
    return "\n".join(lines)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    r = sub.add_parser("record")
    r.add_argument("--name", required=True)
    r.add_argument("--log", required=True)
    r.add_argument("--eval", default="")
    r.add_argument("--out-dir", default="results")
    t = sub.add_parser("table")
    t.add_argument("--out-dir", default="results")
    a = ap.parse_args(argv)
    if a.cmd == "record":
        print(json.dumps(record(a.name, a.log, a.eval, a.out_dir), indent=1))
    else:
        print(table(a.out_dir))
    return 0


if __name__ == "__main__":
    sys.exit(main())
