#!/usr/bin/env python
"""bench_gemm_vocab_tiles — cost of tiling the LM head over the vocabulary.

Parity: ``bench_gemm_vocab_tiles.mojo:1-48``: times the LM-head forward for several tile counts against
the single-GEMM baseline and reports the logits memory each choice needs; with ``--train`` it times the
whole forward+backward step of the model with chunked cross-entropy instead (README "chunked CE" row)."""
from __future__ import annotations

import argparse
import sys

import torch

from llm_mojo_b200 import ops
from llm_mojo_b200.config import parse_model_descriptor
from llm_mojo_b200.models import GPT2


def timed(fn, iters=5, warmup=2):
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


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="d12")
    ap.add_argument("-b", type=int, default=32)
    ap.add_argument("-t", type=int, default=1024)
    ap.add_argument("--tiles", default="1,2,4,8,16")
    ap.add_argument("--train", action="store_true")
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("needs a GPU")
        return 0
    cfg = parse_model_descriptor(a.model)
    rows, C, Vp = a.b * a.t, cfg.channels, cfg.padded_vocab_size
    tiles = [int(k) for k in a.tiles.split(",")]
    if a.train:
        g = torch.Generator().manual_seed(0)
        toks = torch.randint(0, cfg.vocab_size, (a.b, a.t + 1), generator=g, dtype=torch.int32)
        x, y = toks[:, :-1].contiguous(), toks[:, 1:].contiguous()
        base = None
        for k in tiles:
            m = GPT2(cfg, "bf16", "cuda", lm_head_chunks=k)
            ms = timed(lambda: (m.forward(x, y), m.backward()))
            base = base or ms
            key = "logits_tile" if k > 1 else "logits"
            print(f"tiles {k:3d}: fwd+bwd {ms:8.2f} ms ({100 * (ms / base - 1):+.2f}%)  logits buffer {m.acts[key].numel() * 2 / 2**20:8.1f} MiB")
            del m
            torch.cuda.empty_cache()
        return 0
    lnf = torch.randn(rows, C, device="cuda").bfloat16()
    wte = (torch.randn(Vp, C, device="cuda") * 0.02).bfloat16()
    base = None
    for k in tiles:
        w = ((Vp + k - 1) // k + 127) // 128 * 128
        buf = torch.empty(rows, w if k > 1 else Vp, device="cuda", dtype=torch.bfloat16)

        def run():
            for c0 in range(0, Vp, w if k > 1 else Vp):
                ww = min(w if k > 1 else Vp, Vp - c0)
                ops.gemm(buf[:, :ww], lnf, wte[c0:c0 + ww])
        ms = timed(run)
        base = base or ms
        print(f"tiles {k:3d}: LM-head fwd {ms:7.3f} ms ({100 * (ms / base - 1):+.2f}%)  tile width {buf.shape[1]:6d}  logits {buf.numel() * 2 / 2**20:8.1f} MiB")
    return 0


if __name__ == "__main__":
    sys.exit(main())
