#!/usr/bin/env python
"""compare_grad_dumps — cross-precision gradient gate over two ``dump_grads_gpt2.py`` directories.

Parity: ``tests/compare_grad_dumps.py:49-55``, ``:161-214``: per tensor cosine similarity (floor 0.93) and
relative L2 (median < 0.20, max < 0.50), a depth-spike check (no layer's relative L2 more than twice
the median of its tensor kind), NaN/Inf and non-triviality (a tensor that is all zero fails)."""
from __future__ import annotations

import os
import sys
from collections import defaultdict

import numpy as np

COSINE_FLOOR = 0.93
REL_L2_MEDIAN_MAX = 0.20
REL_L2_MAX = 0.50
DEPTH_SPIKE = 2.0


def compare(ref_dir: str, test_dir: str, verbose: bool = True) -> bool:
    names = sorted(f for f in os.listdir(ref_dir) if f.endswith(".bin"))
    if not names:
        print("no gradient files found")
        return False
    ok, rels, by_kind = True, [], defaultdict(list)
    for n in names:
        a = np.fromfile(os.path.join(ref_dir, n), dtype=np.float32).astype(np.float64)
        p = os.path.join(test_dir, n)
        if not os.path.exists(p):
            print(f"MISSING {n}")
            ok = False
            continue
        b = np.fromfile(p, dtype=np.float32).astype(np.float64)
        if a.shape != b.shape or not np.isfinite(b).all():
            print(f"FAIL {n}: shape mismatch or non-finite values")
            ok = False
            continue
        na, nb = np.linalg.norm(a), np.linalg.norm(b)
        if nb == 0 and na > 0:
            print(f"FAIL {n}: all-zero gradient")
            ok = False
            continue
        if na == 0:
            continue
        cos = float(a @ b / (na * nb))
        rel = float(np.linalg.norm(a - b) / na)
        rels.append(rel)
        kind = n.split("_", 1)[1] if n.startswith("layer") else n
        by_kind[kind].append((n, rel))
        good = cos >= COSINE_FLOOR and rel <= REL_L2_MAX
        ok &= good
        if verbose or not good:
            print(f"{'ok  ' if good else 'FAIL'} {n:28s} cosine {cos:.4f} relL2 {rel:.4f}")
    med = float(np.median(rels)) if rels else 0.0
    if med > REL_L2_MEDIAN_MAX:
        print(f"FAIL median relative L2 {med:.4f} > {REL_L2_MEDIAN_MAX}")
        ok = False
    for kind, items in by_kind.items():
        if len(items) < 3:
            continue
        km = float(np.median([r for _, r in items]))
        for n, r in items:
            if km > 0 and r > DEPTH_SPIKE * km and r > 0.05:
                print(f"FAIL depth spike: {n} relL2 {r:.4f} vs median {km:.4f} of {kind}")
                ok = False
    print(f"{len(rels)} tensors, median relL2 {med:.4f}, max {max(rels) if rels else 0:.4f}: {'PASS' if ok else 'FAIL'}")
    return ok


if __name__ == "__main__":
    if len(sys.argv) < 3:
        print("usage: compare_grad_dumps.py <reference dir> <test dir> [-q]")
        sys.exit(2)
    sys.exit(0 if compare(sys.argv[1], sys.argv[2], "-q" not in sys.argv) else 1)
