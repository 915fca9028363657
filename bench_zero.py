#!/usr/bin/env python
"""bench_zero — step time, tok/s and memory of every ZeRO stage on N GPUs.

Parity: ``scripts/benchmark_zero.py:44-67``, ``:175-229``: for each stage run the trainer for a few steps,
parse the per-step log lines (``step i/N | loss … | … ms | … tok/s``) and the ``[mem-report]`` JSON, drop the
warm-up steps, and print one JSON document per (precision, stage) plus the loss agreement across stages.

    python bench_zero.py --gpus 2 --model d12 -b 8 -t 1024 --steps 10
"""
from __future__ import annotations

import argparse
import json
import os
import re
import subprocess
import sys

STEP_RE = re.compile(r"step\s+(\d+)/(\d+) \| loss ([\d.]+) .*?\| ([\d.]+) ms \|.*?\| (\d+) tok/s(?: \| device ([\d.]+) ms)?")


def parse_log(text: str, warmup: int):
    steps, mem = [], None
    for line in text.splitlines():
        m = STEP_RE.search(line)
        if m:
            steps.append({"step": int(m.group(1)), "loss": float(m.group(3)), "ms": float(m.group(4)),
                          "tok_s": float(m.group(5)), "device_ms": float(m.group(6)) if m.group(6) else None})
        if line.startswith("[mem-report] "):          # ranks may interleave their lines: take the first JSON document
            try:
                mem, _ = json.JSONDecoder().raw_decode(line[len("[mem-report] "):])
            except json.JSONDecodeError:
                pass
    timed = steps[warmup:] if len(steps) > warmup else steps
    if not timed:
        return None
    ms = sorted(s["device_ms"] or s["ms"] for s in timed)
    return {"ms_median": ms[len(ms) // 2], "last_loss": steps[-1]["loss"], "steps": len(steps), "mem": mem}


def run_stage(stage, a):
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1", "--nnodes=1",
           f"--nproc-per-node={a.gpus}", os.path.join(here, "train_gpt2.py"), "-e", a.model, "-b", str(a.b), "-t", str(a.t),
           "-x", str(a.steps), "-z", str(stage), "-v", "0", "-s", "0", "--synthetic", "1", "--precision", a.precision]
    if a.gpus == 1:
        cmd = [sys.executable, os.path.join(here, "train_gpt2.py")] + cmd[cmd.index("-e"):]
    env = dict(os.environ, LLMM_MEM_REPORT="1")
    r = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=a.timeout)
    if r.returncode != 0:
        return {"stage": stage, "error": (r.stdout + r.stderr)[-1500:]}
    res = parse_log(r.stdout, a.warmup)
    if res is None:
        return {"stage": stage, "error": "no step lines in the log"}
    tokens = a.b * a.t * a.gpus
    res.update({"stage": stage, "world": a.gpus, "precision": a.precision, "tok_s": tokens / (res["ms_median"] / 1e3)})
    return res


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=2)
    ap.add_argument("--model", default="d12")
    ap.add_argument("--precision", default="bf16")
    ap.add_argument("-b", type=int, default=8)
    ap.add_argument("-t", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--stages", default="0,1,2,3")
    ap.add_argument("--timeout", type=int, default=900)
    a = ap.parse_args(argv)
    results = [run_stage(int(s), a) for s in a.stages.split(",")]
    for r in results:
        print("BENCH_ZERO " + json.dumps(r), flush=True)
    losses = [r["last_loss"] for r in results if "last_loss" in r]
    if len(losses) > 1:
        print(f"loss agreement across stages: max spread {max(losses) - min(losses):.6f}")
    return 0 if all("error" not in r for r in results) else 1


if __name__ == "__main__":
    sys.exit(main())
