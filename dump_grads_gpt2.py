#!/usr/bin/env python
"""dump_grads_gpt2 — write every per-layer gradient tensor (fp32) after one forward + backward.

Parity: ``dump_grads_gpt2.mojo:1-24``: 4 global tensors (wte, wpe, lnfw, lnfb) plus 12 tensors for each
of the L layers (148 files for a 12-layer model), so that a low-precision build can be compared
tensor by tensor with the bf16 build (``compare_grad_dumps.py``).

    python dump_grads_gpt2.py --precision bf16 --out grads_bf16
    python dump_grads_gpt2.py --precision fp8  --out grads_fp8
    python compare_grad_dumps.py grads_bf16 grads_fp8
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

from llm_mojo_b200.models import GPT2
from llm_mojo_b200.models.gpt2 import LAYER_TENSORS


def dump(model: GPT2, out_dir: str) -> int:
    os.makedirs(out_dir, exist_ok=True)
    n = 0
    for name in ("wte", "wpe", "lnfw", "lnfb"):
        model.g[name].detach().float().cpu().numpy().tofile(os.path.join(out_dir, f"{name}.bin"))
        n += 1
    for l in range(model.config.num_layer):
        for name in LAYER_TENSORS:
            model.g[name][l].detach().float().cpu().numpy().tofile(os.path.join(out_dir, f"layer{l:02d}_{name}.bin"))
            n += 1
    return n


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="d12")
    ap.add_argument("--precision", default="bf16")
    ap.add_argument("--out", required=True)
    ap.add_argument("-b", type=int, default=4)
    ap.add_argument("-t", type=int, default=1024)
    ap.add_argument("--device", default="")
    ap.add_argument("--warm-steps", type=int, default=0, help="optimizer steps before the dump (fills fp8 amax history)")
    a = ap.parse_args(argv)
    dev = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
    model = GPT2(a.model, a.precision if dev != "cpu" else "fp32", dev)
    T = min(a.t, model.config.max_seq_len)
    g = torch.Generator().manual_seed(11)
    toks = torch.randint(0, model.config.vocab_size, (a.b, T + 1), generator=g, dtype=torch.int32)
    x, y = toks[:, :-1].contiguous(), toks[:, 1:].contiguous()
    for s in range(a.warm_steps):
        model.forward(x, y); model.backward(); model.update(s + 1, 1e-4)
        model.read_loss()
    model.forward(x, y)
    model.backward()
    print(f"loss {model.read_loss():.6f}; wrote {dump(model, a.out)} gradient files to {a.out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
