#!/usr/bin/env python
"""FineWeb (10B / 100B sample) → shards of 10^8 tokens; shard 0 is the validation split
(``data/fineweb.py:1-15`` of the reference).  Needs the `datasets` package and network access.

    python -m data.fineweb --version 10B
"""
import argparse
import multiprocessing as mp
import os

import numpy as np

from data.common import tokenize_document, write_datafile


def _tok(doc):
    return np.asarray(tokenize_document(doc["text"]), dtype=np.uint16)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--version", default="10B", choices=["10B", "100B"])
    ap.add_argument("--shard-size", type=int, default=10 ** 8)
    a = ap.parse_args()
    from datasets import load_dataset
    name = {"10B": "sample-10BT", "100B": "sample-100BT"}[a.version]
    out = os.path.join(os.path.dirname(__file__), f".fineweb{a.version}")
    os.makedirs(out, exist_ok=True)
    ds = load_dataset("HuggingFaceFW/fineweb", name=name, split="train")
    shard, buf, fill = 0, np.empty(a.shard_size, dtype=np.uint16), 0
    with mp.Pool(max(1, os.cpu_count() - 2)) as pool:
        for toks in pool.imap(_tok, ds, chunksize=16):
            while len(toks):
                take = min(len(toks), a.shard_size - fill)
                buf[fill:fill + take] = toks[:take]
                fill += take
                toks = toks[take:]
                if fill == a.shard_size:
                    split = "val" if shard == 0 else "train"
                    write_datafile(os.path.join(out, f"fineweb_{split}_{shard:06d}.bin"), buf)
                    shard, fill = shard + 1, 0
    if fill:
        split = "val" if shard == 0 else "train"
        write_datafile(os.path.join(out, f"fineweb_{split}_{shard:06d}.bin"), buf[:fill])


if __name__ == "__main__":
    main()
