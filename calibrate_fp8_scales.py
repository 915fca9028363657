#!/usr/bin/env python
"""calibrate_fp8_scales — derive a static FP8 scale table.

Parity: ``calibrate_fp8_scales.mojo:1-57``: run N fp8 training steps, track the running minimum of every
``AmaxState.scale`` (the smallest scale seen = the largest amax), divide by a safety factor (2) and print
the table, one ``site.layer.operand scale`` line each, and with ``--out`` a JSON file that a later run loads
with ``train_gpt2.py --precision fp8 --fp8-static-scales <file>`` (or ``LLMM_FP8_STATIC_SCALES=<file>``): that run
uses one constant per (site, operand) - the minimum over the layers - and launches no amax or scale-update kernel.
On a machine without a GPU the calibration runs the fp8 emulation of the CPU path (slow; small models only)."""
from __future__ import annotations

import argparse
import json
import sys

import torch

from llm_mojo_b200.config import Precision
from llm_mojo_b200.models import GPT2


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="d12")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("-b", type=int, default=4)
    ap.add_argument("-t", type=int, default=1024)
    ap.add_argument("--safety", type=float, default=2.0)
    ap.add_argument("--out", default="")
    a = ap.parse_args(argv)
    on_gpu = torch.cuda.is_available()
    model = GPT2(a.model, Precision("fp8", fp32_storage=not on_gpu), "cuda" if on_gpu else "cpu")
    T = min(a.t, model.config.max_seq_len)
    g = torch.Generator().manual_seed(3)
    mins = {}
    for step in range(a.steps):
        toks = torch.randint(0, model.config.vocab_size, (a.b, T + 1), generator=g, dtype=torch.int32)
        model.forward(toks[:, :-1].contiguous(), toks[:, 1:].contiguous())
        model.backward()
        model.update(step + 1, 3e-4)
        loss = model.read_loss()
        for k, v in model.lowp.min_scales().items():
            mins[k] = min(mins.get(k, float("inf")), v)
        print(f"step {step + 1}/{a.steps} loss {loss:.4f}")
    table = {k: v / a.safety for k, v in sorted(mins.items())}
    for k, v in table.items():
        print(f"{k:24s} {v:.6g}")
    if a.out:
        with open(a.out, "w") as f:
            json.dump({"safety": a.safety, "scales": table}, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
