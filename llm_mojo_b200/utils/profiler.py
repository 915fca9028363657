"""Span tracer that writes Chrome-trace / Perfetto JSON (``llmm/profiler.mojo:160-273``).

Host spans use ``perf_counter_ns``; ``cuda_span`` additionally brackets the span with CUDA
events so that the device time of a phase is reported.  Enabled by ``LLMM_TRACE=<file>``.
"""
from __future__ import annotations

import contextlib
import json
import os
import threading
import time
from typing import List, Optional

import torch


class TraceProfiler:
    def __init__(self, path: Optional[str] = None, pid: int = 0):
        self.path = path if path is not None else os.environ.get("LLMM_TRACE", "")
        self.enabled = bool(self.path)
        self.pid = pid
        self.events: List[dict] = []
        self._cuda: List[tuple] = []
        self._t0 = time.perf_counter_ns()

    def _now_us(self) -> float:
        return (time.perf_counter_ns() - self._t0) / 1e3

    @contextlib.contextmanager
    def span(self, name: str, cat: str = "host"):
        if not self.enabled:
            yield
            return
        ts = self._now_us()
        try:
            yield
        finally:
            self.events.append({"name": name, "cat": cat, "ph": "X", "ts": ts,
                                "dur": self._now_us() - ts, "pid": self.pid,
                                "tid": threading.get_ident() % 100000})

    @contextlib.contextmanager
    def cuda_span(self, name: str):
        if not self.enabled or not torch.cuda.is_available():
            with self.span(name):
                yield
            return
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ts = self._now_us()
        a.record()
        try:
            yield
        finally:
            b.record()
            self._cuda.append((name, ts, a, b))

    def flush(self) -> None:
        if not self.enabled:
            return
        if self._cuda:
            torch.cuda.synchronize()
            for name, ts, a, b in self._cuda:
                self.events.append({"name": name, "cat": "cuda", "ph": "X", "ts": ts,
                                    "dur": a.elapsed_time(b) * 1e3, "pid": self.pid, "tid": 1})
            self._cuda.clear()
        with open(self.path, "w") as f:
            json.dump({"traceEvents": self.events, "displayTimeUnit": "ms"}, f)
