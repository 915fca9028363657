"""Per-step log line, outlier z-scores and the token-rate EMA.

Parity: ``train_gpt2.mojo:362-410`` (OutlierDetector, 128-sample window),
``:6553-6561`` (bias-corrected 0.95 EMA of tok/s), ``:6578-6603`` (line grammar).
"""
from __future__ import annotations

import math
from typing import Optional

OUTLIER_WINDOW = 128


class OutlierDetector:
    """Rolling z-score; returns NaN until the window is full."""

    def __init__(self, window: int = OUTLIER_WINDOW):
        self.window = window
        self.buf = [0.0] * window
        self.count = 0
        self.index = 0
        self.sum = 0.0
        self.sum_sq = 0.0

    def update(self, x: float) -> float:
        if self.count < self.window:
            self.buf[self.count] = x
            self.sum += x
            self.sum_sq += x * x
            self.count += 1
            return float("nan")
        old = self.buf[self.index]
        self.sum += x - old
        self.sum_sq += x * x - old * old
        self.buf[self.index] = x
        self.index = (self.index + 1) % self.window
        mean = self.sum / self.window
        var = self.sum_sq / self.window - mean * mean
        std = math.sqrt(var) if var > 0 else 0.0
        return 0.0 if std == 0.0 else (x - mean) / std


class TokenRateEMA:
    def __init__(self, beta: float = 0.95):
        self.beta, self.ema, self.n = beta, 0.0, 0

    def update(self, tok_per_s: float) -> float:
        self.n += 1
        self.ema = self.beta * self.ema + (1 - self.beta) * tok_per_s
        return self.ema / (1 - self.beta ** self.n)


def format_step_line(step: int, total: int, loss: float, z_loss: float, norm: float, z_norm: float,
                     lr: float, ms: float, mfu: float, precision: str, tok_s: float,
                     device_ms: Optional[float] = None) -> str:
    line = (f"step {step:4d}/{total} | loss {loss:.6f} ({z_loss:+.2f}z)| norm {norm:.4f} ({z_norm:+.2f}z)"
            f"| lr {lr:.2e} | {ms:.2f} ms | {100.0 * mfu:.1f}% {precision} MFU | {tok_s:.0f} tok/s")
    if device_ms is not None:
        line += f" | device {device_ms:.2f} ms"
    return line
