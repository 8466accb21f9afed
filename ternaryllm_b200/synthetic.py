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


def block_weight(seed: int, K: int, N: int, sparsity: float, axis: int, nblocks: int, first: int = 0, count: int | None = None) -> np.ndarray:
    """Blocks [first, first + count) of a seeded ternary matrix [K, N] that is defined as the concatenation of `nblocks`
    independently seeded blocks along `axis` (0: row blocks, 1: column blocks).  A tensor-parallel rank generates
    only the blocks it holds, and every partitioning of the blocks sees the same matrix."""
    if count is None:
        count = nblocks - first
    if (N if axis else K) % nblocks:
        raise ValueError("the blocked axis does not divide into the blocks")
    shape = (K, N // nblocks) if axis else (K // nblocks, N)
    parts = [make_weight(seed * 1009 + b, shape[0], shape[1], sparsity) for b in range(first, first + count)]
    return np.ascontiguousarray(np.concatenate(parts, axis=axis))
