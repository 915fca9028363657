"""MT19937 generator that is draw-for-draw compatible with torch's CPU generator.

Parity: ``llmm/rand.mojo:40-202`` (``randint32``, ``random_permutation``, ``normal_``).
The 624-word state refill is vectorised with numpy; single draws are plain Python.
"""
from __future__ import annotations

import math
from typing import List

import numpy as np

_N, _M = 624, 397
_UMASK, _LMASK, _MATRIX_A = 0x80000000, 0x7FFFFFFF, 0x9908B0DF
BOX_MULLER_EPSILON = 0.0  # torch's normal_fill uses log(1 - u) with u in [0, 1)


class MT19937:
    def __init__(self, seed: int = 5489):
        self.seed(seed)

    def seed(self, seed: int) -> None:
        st = np.empty(_N, dtype=np.uint64)
        st[0] = seed & 0xFFFFFFFF
        for j in range(1, _N):
            prev = int(st[j - 1])
            st[j] = (1812433253 * (prev ^ (prev >> 30)) + j) & 0xFFFFFFFF
        self.state = st.astype(np.uint32)
        self.left = 1
        self.next = 0
        self.draws = 0

    def _next_state(self) -> None:
        st = self.state.astype(np.uint64)
        # The reference recurrence is sequential (state[j+M] may already be refreshed for
        # j >= N-M); do it in the three classic segments so each uses the right operands.
        def twist(u, v):
            y = (u & _UMASK) | (v & _LMASK)
            return (y >> 1) ^ np.where(y & 1, _MATRIX_A, 0).astype(np.uint64)
        k = _N - _M
        st[:k] = st[_M:_M + k] ^ twist(st[:k], st[1:k + 1])
        # second segment depends on values written in the first: process in chunks of k
        j = k
        while j < _N - 1:
            e = min(j + k, _N - 1)
            st[j:e] = st[j - k:e - k] ^ twist(st[j:e], st[j + 1:e + 1])
            j = e
        st[_N - 1] = st[_M - 1] ^ twist(st[_N - 1:_N], st[0:1])[0]
        self.state = (st & 0xFFFFFFFF).astype(np.uint32)
        self.left = _N
        self.next = 0

    def randint32(self) -> int:
        self.left -= 1
        if self.left <= 0:
            self._next_state()
        y = int(self.state[self.next])
        self.next += 1
        self.draws += 1
        y ^= y >> 11
        y ^= (y << 7) & 0x9D2C5680
        y ^= (y << 15) & 0xEFC60000
        y ^= y >> 18
        return y & 0xFFFFFFFF

    def randint64(self) -> int:
        hi = self.randint32()
        lo = self.randint32()
        return (hi << 32) | lo

    def randfloat32(self) -> float:
        return float(np.float32(self.randint32() & 0xFFFFFF) * np.float32(1.0 / (1 << 24)))

    def randfloat64(self) -> float:
        return (self.randint64() & ((1 << 53) - 1)) * (1.0 / (1 << 53))

    def randint32_array(self, n: int) -> np.ndarray:
        return np.fromiter((self.randint32() for _ in range(n)), dtype=np.uint32, count=n)


def random_permutation(arr: List[int], rng: MT19937) -> None:
    """Fisher-Yates over the mt19937 stream (llm.c order; ``llmm/rand.mojo:132``)."""
    for i in range(len(arr) - 1, 0, -1):
        j = rng.randint32() % (i + 1)
        arr[i], arr[j] = arr[j], arr[i]


def _normal_fill_16(data: np.ndarray, mean: float, std: float) -> None:
    u1 = np.float32(1.0) - data[:8]
    u2 = data[8:16].copy()
    radius = np.sqrt(np.float32(-2.0) * np.log(u1)).astype(np.float32)
    theta = (2.0 * math.pi * u2.astype(np.float64)).astype(np.float32)
    data[:8] = radius * np.cos(theta) * np.float32(std) + np.float32(mean)
    data[8:16] = radius * np.sin(theta) * np.float32(std) + np.float32(mean)


def normal_(rng: MT19937, numel: int, mean: float = 0.0, std: float = 1.0) -> np.ndarray:
    """N(mean, std²) samples matching ``torch.Tensor.normal_`` on CPU (``llmm/rand.mojo:162``)."""
    data = np.empty(numel, dtype=np.float32)
    if numel >= 16:
        raw = rng.randint32_array(numel)
        data[:] = (raw & 0xFFFFFF).astype(np.float32) * np.float32(1.0 / (1 << 24))
        for i in range(0, numel - 15, 16):
            _normal_fill_16(data[i:i + 16], mean, std)
        if numel % 16:
            tail = data[numel - 16:]
            raw = rng.randint32_array(16)
            tail[:] = (raw & 0xFFFFFF).astype(np.float32) * np.float32(1.0 / (1 << 24))
            _normal_fill_16(tail, mean, std)
    else:
        has_next, nxt = False, 0.0
        for t in range(numel):
            if has_next:
                data[t] = np.float32(nxt * std + mean)
                has_next = False
                continue
            u1 = np.float32(rng.randfloat64())
            u2 = np.float32(rng.randfloat64())
            radius = np.sqrt(np.float32(-2.0) * np.log(np.float32(1.0) - u2))
            theta = np.float32(2.0 * math.pi * float(u1))
            nxt = float(radius * np.sin(theta))
            has_next = True
            data[t] = radius * np.cos(theta) * np.float32(std) + np.float32(mean)
    return data
