"""xorshift* RNG and CDF sampling from logits (``llmm/sampler.mojo:19-66``)."""
from __future__ import annotations

import numpy as np

_MASK64 = (1 << 64) - 1


class SamplerRNG:
    def __init__(self, state: int = 1337):
        self.state = state & _MASK64

    def random_u32(self) -> int:
        s = self.state
        s ^= s >> 12
        s ^= (s << 25) & _MASK64
        s ^= s >> 27
        self.state = s
        return ((s * 0x2545F4914F6CDD1D) & _MASK64) >> 32

    def random_f32(self) -> float:
        return float(np.float32(self.random_u32() >> 8) / np.float32(16777216.0))


def sample_softmax(logits: np.ndarray, coin: float) -> int:
    """Sample an index from softmax(logits) given a uniform ``coin`` in [0,1).

    The logits are used unnormalised (exp without max subtraction), as in the reference.
    """
    e = np.exp(logits.astype(np.float32))
    norm = float(e.astype(np.float64).sum())
    c = np.float32(coin * norm)
    cdf = np.cumsum(e, dtype=np.float32)
    idx = int(np.searchsorted(cdf, c, side="right"))
    return min(idx, len(logits) - 1)
