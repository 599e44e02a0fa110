"""The trainer's seeded generator, restated: SplitMix64 with a 24-bit uniform and Box-Muller
normals (reference src/tensor.rs:155-199).  Vectorised with NumPy: the i-th output of the
stream depends only on seed and i, so whole vectors are produced at once and still equal the
reference's sequential draws value for value.
"""
from __future__ import annotations

import numpy as np

_GOLDEN = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


class Rng:
    def __init__(self, seed: int):
        self.state = np.uint64(seed & 0xFFFFFFFFFFFFFFFF) ^ _GOLDEN

    def _next_block(self, n: int) -> np.ndarray:
        with np.errstate(over="ignore"):
            idx = np.arange(1, n + 1, dtype=np.uint64)
            z = self.state + idx * _GOLDEN
            self.state = z[-1] if n else self.state
            z = (z ^ (z >> np.uint64(30))) * _M1
            z = (z ^ (z >> np.uint64(27))) * _M2
            return z ^ (z >> np.uint64(31))

    def next_u64(self) -> int:
        return int(self._next_block(1)[0])

    def uniform(self, n: int) -> np.ndarray:
        """n draws of `(next_u64 >> 40) / 2^24` as float32."""
        return (self._next_block(n) >> np.uint64(40)).astype(np.float32) / np.float32(1 << 24)

    def uniform_sym(self, n: int, bound: float) -> np.ndarray:
        return (self.uniform(n) * np.float32(2.0) - np.float32(1.0)) * np.float32(bound)

    def normal(self, n: int, std: float = 1.0) -> np.ndarray:
        """Box-Muller, two uniforms per value, cosine branch only (tensor.rs:178-182)."""
        u = self.uniform(2 * n)
        u1 = np.maximum(u[0::2], np.float32(1e-12))
        u2 = u[1::2]
        r = np.sqrt(np.float32(-2.0) * np.log(u1)).astype(np.float32)
        v = r * np.cos(np.float32(2.0 * np.pi) * u2).astype(np.float32)
        return (v * np.float32(std)).astype(np.float32)

    def below(self, n: int) -> int:
        return self.next_u64() % n

    def shuffle(self, v: list) -> None:
        """Fisher-Yates from the top (tensor.rs:186-191)."""
        for i in range(len(v) - 1, 0, -1):
            j = self.below(i + 1)
            v[i], v[j] = v[j], v[i]
