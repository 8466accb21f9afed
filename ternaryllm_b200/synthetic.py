"""Seeded synthetic ternary weights with the shapes and sparsities of the benchmark configurations."""
from __future__ import annotations

import numpy as np


def make_weight(seed: int, K: int, N: int, sparsity: float) -> np.ndarray:
    """Seeded ternary matrix [K, N]: i.i.d. zeros with probability `sparsity` (rounded to a multiple of 1/256),
    +1 and -1 equiprobable among the rest -- the reference's non-uniform generator (TernaryLinear.py:79-83) with a
    byte-wide random source, which is what makes generating 10^8 entries take seconds."""
    rng = np.random.default_rng(seed)
    z = int(round(sparsity * 256))
    half = (256 - z) // 2
    r = rng.integers(0, 256, size=(K, N), dtype=np.uint8)
    w = np.zeros((K, N), np.int8)
    w[(r >= z) & (r < z + half)] = -1
    w[r >= z + half] = 1
    return w
