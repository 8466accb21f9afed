"""Shared-segment rows: the library's sparse-segment image of a ternary matrix (host memory, `tllm_ssr_encode` /
`tllm_ssr_decode` of include/tllm.h).

The reference names a sparse-segment encoding without defining one (its SSR/README.md is a citation and the consumer in
ternaryLLM_GPU/csrc/ter_spmm_kernel.cuh:159-160 is commented out); this is the library's own.  The 8 columns of a
group share, per segment of 256 rows, one ascending list of the rows that any of them uses and a word of two-bit codes
per listed row, 2 + 3n bytes per (group, segment).  A storage form for matrices of 90 % zeros and more: no kernel reads
it; `decode` gives back the dense matrix that `PackedWeight.from_dense` packs for the GPU.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib

GROUP_COLUMNS = 8
SEGMENT_ROWS = 256


def encode(w: np.ndarray) -> np.ndarray:
    """int8 [K, N] with entries in {-1, 0, +1} (other values count by their sign) -> the image as a uint8 array."""
    w = np.ascontiguousarray(w, dtype=np.int8)
    if w.ndim != 2:
        raise ValueError("encode takes a matrix [K, N]")
    K, N = w.shape
    n = C.c_size_t(0)
    _lib.check(_lib.lib().tllm_ssr_encode(_lib.np_ptr(w), K, N, None, 0, C.byref(n)), "tllm_ssr_encode")
    image = np.empty(n.value, dtype=np.uint8)
    _lib.check(_lib.lib().tllm_ssr_encode(_lib.np_ptr(w), K, N, _lib.np_ptr(image), image.size, C.byref(n)), "tllm_ssr_encode")
    return image


def decode(image: np.ndarray, inners: int, columns: int) -> np.ndarray:
    """The int8 matrix [inners, columns] an image holds; a damaged or foreign image raises RuntimeError."""
    image = np.ascontiguousarray(image, dtype=np.uint8)
    out = np.empty((inners, columns), dtype=np.int8)
    _lib.check(_lib.lib().tllm_ssr_decode(_lib.np_ptr(image), image.size, inners, columns, _lib.np_ptr(out)), "tllm_ssr_decode")
    return out


def expected_bytes_per_entry(zeros: float) -> float:
    """Bytes per entry of W for independent entries with that share of zeros (header and group table left out)."""
    listed = SEGMENT_ROWS * (1.0 - zeros ** GROUP_COLUMNS)
    return (2.0 + 3.0 * listed) / (SEGMENT_ROWS * GROUP_COLUMNS)
