"""Model-FLOPs-utilisation estimate (``llmm/mfu.mojo:73-88``, ``:187-289``, ``:333``).

``flops/token = 6·N + 6·L·C·T`` (N excludes nothing, as in the reference); peak comes from a
per-GPU table by precision, extended with the B200 entry the reference lacks.
"""
from __future__ import annotations

from typing import Optional

# dense tensor peaks in TFLOP/s: name substring → {precision: peak}
PEAK_TFLOPS = {
    "B200": {"bf16": 2250.0, "fp16": 2250.0, "tf32": 1125.0, "fp32": 1125.0, "fp8": 4500.0, "fp4": 9000.0},
    "H100": {"bf16": 989.4, "fp16": 989.4, "tf32": 494.7, "fp32": 494.7, "fp8": 1978.9, "fp4": 1978.9},
    "A100": {"bf16": 312.0, "fp16": 312.0, "tf32": 156.0, "fp32": 156.0, "fp8": 312.0, "fp4": 312.0},
    "GB10": {"bf16": 125.0, "fp16": 125.0, "tf32": 62.5, "fp32": 62.5, "fp8": 250.0, "fp4": 500.0},
    "RTX PRO 6000": {"bf16": 438.9, "fp16": 438.9, "tf32": 219.4, "fp32": 219.4, "fp8": 877.8, "fp4": 1755.6},
}


def peak_flops(device_name: str, precision: str) -> Optional[float]:
    for key, row in PEAK_TFLOPS.items():
        if key.lower() in device_name.lower():
            return row.get(precision, row["bf16"]) * 1e12
    return None


def flops_per_token(num_parameters: int, num_layer: int, channels: int, seq_len: int) -> float:
    return 6.0 * num_parameters + 6.0 * num_layer * channels * seq_len


def estimate_mfu(num_parameters: int, num_layer: int, channels: int, seq_len: int,
                 num_tokens: int, dt_seconds: float, device_name: str, precision: str) -> float:
    """Fraction of peak (−1 when the device is unknown, as the reference prints)."""
    peak = peak_flops(device_name, precision)
    if peak is None or dt_seconds <= 0:
        return -1.0
    return flops_per_token(num_parameters, num_layer, channels, seq_len) * num_tokens / dt_seconds / peak
