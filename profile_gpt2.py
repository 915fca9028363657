#!/usr/bin/env python
"""profile_gpt2 — per-phase timing harness (forward / backward / grad-norm / update).

Parity: ``profile_gpt2.mojo:61-181`` (synthetic tokens ``i % V``, phase wall times, optional
Chrome/Perfetto trace) and ``profile_gpt2.py:42-70`` (kernel-family buckets for an ``ncu`` run).
Environment: LLMM_PROFILE_B, LLMM_PROFILE_T, LLMM_PROFILE_LAYERS, LLMM_PROFILE_STEPS,
LLMM_PROFILE_TRACE (file), LLMM_PROFILE_MODEL (descriptor, default d12), LLMM_PROFILE_PRECISION (bf16 | fp8 | fp8b | fp4).

Phases are timed with CUDA events on the launching stream (wall clock on CPU).  The printed
`forward / backward / update` seconds line is the one benchmark scripts parse.
"""
from __future__ import annotations

import os
import sys
import time

import torch

from llm_mojo_b200.config import parse_model_descriptor
from llm_mojo_b200.models import GPT2
from llm_mojo_b200.utils.profiler import TraceProfiler

# kernel-name substring → family, for classifying an ncu launch list (csv with "Kernel Name", "gpu__time_duration.sum")
FAMILIES = (("gemm", "matmul"), ("attn", "attention"), ("ln_", "layernorm"), ("classifier", "classifier"),
            ("adamw", "adamw"), ("encoder", "encoder"), ("wte_bwd", "encoder"), ("wpe_bwd", "encoder"),
            ("dbias", "matmul"), ("gelu", "gelu"), ("norm_sq", "global_norm"), ("pack_kernel", "comm"),
            ("reduce_kernel", "comm"), ("unpack_kernel", "comm"), ("gather_kernel", "comm"), ("quantize", "quant"),
            ("amax", "quant"))


def classify(kernel_name: str) -> str:
    for key, fam in FAMILIES:
        if key in kernel_name:
            return fam
    return "other"


def summarize_launch_csv(path: str) -> dict:
    """Bucket an ``ncu --csv`` launch list into kernel families.

    With ``--metrics gpu__time_duration.sum`` alone (one pass per launch) the result is {family: microseconds}.  When the
    capture also holds ``dram__bytes_read.sum``, ``dram__bytes_write.sum`` and / or
    ``sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_elapsed`` (more passes: capture a small case), every
    family additionally gets its DRAM megabytes and its time-weighted tensor-pipe activity under ``detail``."""
    import csv
    with open(path) as f:
        rows = [r for r in csv.reader(f) if r and not r[0].startswith("==")]
    hdr = rows[0]
    ni, vi, ui = hdr.index("Kernel Name"), hdr.index("Metric Value"), hdr.index("Metric Unit")
    mi = hdr.index("Metric Name") if "Metric Name" in hdr else None
    idi = hdr.index("ID") if "ID" in hdr else None
    launches = {}                                    # launch id -> {"name", metric: value}
    for n, r in enumerate(rows[1:]):
        if len(r) <= vi:
            continue
        key = r[idi] if idi is not None else str(n)
        metric = r[mi] if mi is not None else "gpu__time_duration.sum"
        try:
            v = float(r[vi].replace(",", ""))
        except ValueError:
            continue
        unit = r[ui]
        if metric.startswith("gpu__time_duration"):
            v = v / 1e3 if unit in ("ns", "nsecond") else v * 1e3 if unit in ("ms", "msecond") else v      # microseconds
        elif metric.startswith("dram__bytes"):
            v = v * {"byte": 1e-6, "Kbyte": 1e-3, "Mbyte": 1.0, "Gbyte": 1e3}.get(unit, 1e-6)              # megabytes
        launches.setdefault(key, {"name": r[ni]})[metric] = v
    out, detail = {}, {}
    for rec in launches.values():
        fam = classify(rec["name"])
        us = rec.get("gpu__time_duration.sum", 0.0)
        out[fam] = out.get(fam, 0.0) + us
        d = detail.setdefault(fam, {"dram_mb": 0.0, "tensor_x_us": 0.0, "launches": 0})
        d["launches"] += 1
        d["dram_mb"] += rec.get("dram__bytes_read.sum", 0.0) + rec.get("dram__bytes_write.sum", 0.0)
        d["tensor_x_us"] += rec.get("sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_elapsed", 0.0) * us
    if any(d["dram_mb"] or d["tensor_x_us"] for d in detail.values()):
        out["detail"] = {fam: {"launches": d["launches"], "dram_mb": d["dram_mb"],
                               "tensor_pipe_pct": d["tensor_x_us"] / out[fam] if out.get(fam) else 0.0}
                         for fam, d in detail.items()}
    return out


def run_profile() -> dict:
    B = int(os.environ.get("LLMM_PROFILE_B", 4))
    T = int(os.environ.get("LLMM_PROFILE_T", 1024))
    steps = int(os.environ.get("LLMM_PROFILE_STEPS", 5))
    cfg = parse_model_descriptor(os.environ.get("LLMM_PROFILE_MODEL", "d12"))
    if os.environ.get("LLMM_PROFILE_LAYERS"):
        cfg.num_layer = int(os.environ["LLMM_PROFILE_LAYERS"])
    dev = torch.device("cuda" if torch.cuda.is_available() and not os.environ.get("LLMM_USE_CPU") else "cpu")
    T = min(T, cfg.max_seq_len)
    model = GPT2(cfg, os.environ.get("LLMM_PROFILE_PRECISION", "bf16") if dev.type == "cuda" else "fp32", dev)
    toks = (torch.arange(B * T + 1) % cfg.vocab_size).to(torch.int32)
    x, y = toks[:-1].view(B, T).contiguous(), toks[1:].view(B, T).contiguous()
    tracer = TraceProfiler(os.environ.get("LLMM_PROFILE_TRACE", ""))
    totals = {"forward": 0.0, "backward": 0.0, "grad_norm": 0.0, "update": 0.0}

    def timed(name, fn):
        if dev.type == "cuda":
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            with tracer.span(name):
                fn()
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) / 1e3
        t0 = time.perf_counter()
        with tracer.span(name):
            fn()
        return time.perf_counter() - t0

    for step in range(steps + 1):                    # step 0 is warm-up and is not counted
        t = {"forward": timed("forward", lambda: model.forward(x, y)),
             "backward": timed("backward", lambda: model.backward())}
        norm_box = {}
        t["grad_norm"] = timed("grad_norm", lambda: norm_box.setdefault("n", model.calculate_grad_norm()))
        t["update"] = timed("update", lambda: model.update(step + 1, 1e-4, 0.0,
                                                          dev_scale=model.clip_scale_from_norm(norm_box["n"])))
        loss = model.read_loss()
        print(f"step {step}: loss {loss:.6f} | forward {t['forward'] * 1e3:.2f} ms | backward {t['backward'] * 1e3:.2f} ms"
              f" | grad_norm {t['grad_norm'] * 1e3:.2f} ms | update {t['update'] * 1e3:.2f} ms")
        if step > 0:
            for k in totals:
                totals[k] += t[k]
    n = max(steps, 1)
    print(f"forward / backward / update: {totals['forward'] / n:.6f} {totals['backward'] / n:.6f} "
          f"{(totals['update'] + totals['grad_norm']) / n:.6f}")
    tracer.flush()
    return {k: v / n for k, v in totals.items()}


if __name__ == "__main__":
    if len(sys.argv) > 2 and sys.argv[1] == "--families":
        res = summarize_launch_csv(sys.argv[2])
        detail = res.pop("detail", {})
        for fam, us in sorted(res.items(), key=lambda kv: -kv[1]):
            extra = ""
            if fam in detail:
                d = detail[fam]
                extra = f"   {d['launches']:4d} launches   DRAM {d['dram_mb']:10.1f} MB   tensor pipe {d['tensor_pipe_pct']:5.1f} %"
            print(f"{fam:12s} {us / 1e3:10.3f} ms{extra}")
    else:
        run_profile()
