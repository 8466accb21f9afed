"""Drop-in for the reference's `ter_spmm` extension module.

The reference builds a pybind11 module named `ter_spmm` with four callables
(ternaryLLM_GPU/csrc/ter_spmm_wrapper.cu:350-355); this module offers the same four names, positional
signatures and return shapes on top of the C ABI (include/tllm.h).  `install()` registers it under the
name `ter_spmm`, so that `import ter_spmm` in unmodified reference code resolves here.

Differences, all additive:
  * `ter_spmm` accepts fp16 / bf16 / int8 activations besides fp32 (the result has the activation's
    dtype, int32 for int8), an optional per-tensor `scale`, an `out=` tensor, and launches on torch's
    current stream instead of the legacy stream plus two ad-hoc streams
    (ternaryLLM_GPU/csrc/ter_spmm_kernel.cuh:345-374);
  * the activation layout is taken from the tensor's shape: [..., rows, inners] is read row-major and
    [..., inners, rows] column-major (the reference kernel always indexes [inners][rows], :173, whatever it
    is handed);
  * `convert_to_ter_tiled_mcsc` is lossless unless `compat=True` asks for the reference's truncating
    behaviour (ter_spmm_wrapper.cu:277-291).
"""
from __future__ import annotations

import sys

import numpy as np

from . import _lib
from ._lib import check, lib, np_ptr


def tile_size_for(inners: int) -> int:
    """TILE_K as the reference picks it: MapKSizeToTileSize (TernaryLinear.py:9-16) for the sizes it knows,
    DISPATCH_K (ternaryLLM_GPU/csrc/utils.cuh:59-80) for the rest -- which the map agrees with."""
    if inners <= 512:
        return 64
    if inners <= 2048:
        return 256
    return 512


def _as_w(w):
    """int32 [inners, columns] C-contiguous numpy view of a torch / numpy weight."""
    if hasattr(w, "detach"):
        if w.device.type != "cpu":
            raise RuntimeError("ter_spmm packers expect the weight on the CPU")   # TORCH_INTERNAL_ASSERT, ter_spmm_wrapper.cu:47
        w = w.detach().numpy()
    w = np.ascontiguousarray(w)
    if w.dtype != np.int32:
        if w.dtype.kind not in "iu":
            raise RuntimeError("ter_spmm packers expect an integer weight tensor")
        w = w.astype(np.int32)
    return w


def _ret(arrays, as_numpy):
    return list(arrays) if as_numpy else [a.tolist() for a in arrays]


def convert_to_ter_csc(w, columns, inners, cnt_pos, cnt_neg, as_numpy=False):
    """-> [neg_idx, neg_off, pos_idx, pos_off]  (ter_spmm_wrapper.cu:39-78)"""
    w = _as_w(w)
    ni, no = np.zeros(int(cnt_neg), np.int32), np.zeros(columns + 1, np.int32)
    pi, po = np.zeros(int(cnt_pos), np.int32), np.zeros(columns + 1, np.int32)
    check(lib().tllm_convert_to_ter_csc(np_ptr(w), columns, inners, np_ptr(ni), np_ptr(no), np_ptr(pi), np_ptr(po)))
    return _ret((ni, no, pi, po), as_numpy)


def convert_to_ter_tiled_csc(w, columns, inners, cnt_pos, cnt_neg, TILE_K, as_numpy=False):
    """-> [neg_idx (tile-local), neg_off_tiled, pos_idx, pos_off_tiled]  (ter_spmm_wrapper.cu:92-152)"""
    w = _as_w(w)
    tiles = -(-inners // TILE_K)
    ni, no = np.zeros(int(cnt_neg), np.int32), np.zeros(columns * tiles * 2, np.int32)
    pi, po = np.zeros(int(cnt_pos), np.int32), np.zeros(columns * tiles * 2, np.int32)
    check(lib().tllm_convert_to_ter_tiled_csc(np_ptr(w), columns, inners, TILE_K, np_ptr(ni), np_ptr(no), np_ptr(pi), np_ptr(po)))
    return _ret((ni, no, pi, po), as_numpy)


def convert_to_ter_tiled_mcsc(w, columns, inners, cnt_pos, cnt_neg, TILE_K, padding, padding_size, compat=False,
                              as_numpy=False):
    """-> [merged_idx, merged_off (4 per (column, tile)), col_tile_indices]  (ter_spmm_wrapper.cu:156-315)"""
    w = _as_w(w)
    mode = 1 if compat else 0
    n = lib().tllm_ter_tiled_mcsc_len(np_ptr(w), columns, inners, TILE_K, int(bool(padding)), int(padding_size), mode)
    if n < 0:
        check(int(n))
    tiles = -(-inners // TILE_K)
    idx = np.zeros(int(n), np.int32)
    off = np.zeros(columns * tiles * 4, np.int32)
    til = np.zeros(columns * tiles, np.int32)
    check(lib().tllm_convert_to_ter_tiled_mcsc(np_ptr(w), columns, inners, TILE_K, int(bool(padding)), int(padding_size), mode,
                                               np_ptr(idx), int(n), np_ptr(off), np_ptr(til)))
    return _ret((idx, off, til), as_numpy)


AUTO_PREPARE = False


def ter_spmm(X, w_tiled_merged_row_indice, w_tiled_merged_col_offset, w_col_tile_indices, batch_size, rows, columns,
             inners, uniformed, padded, scale=1.0, out=None, tile_k=None):
    """Product on the reference's merged tiled CSC arrays; returns [batch_size, rows, columns].

    Same positional signature as the reference (ter_spmm_wrapper.cu:318-348).  Raises RuntimeError when a
    tensor is not on a CUDA device or has the wrong dtype, like the reference's TORCH_INTERNAL_ASSERT /
    data_ptr<T>() checks (:326-333).
    """
    import torch

    for t, name in ((X, "X"), (w_tiled_merged_row_indice, "row indices"), (w_tiled_merged_col_offset, "col offsets")):
        if t.device.type != "cuda":
            raise RuntimeError(f"ter_spmm: {name} must be a CUDA tensor")
    if w_tiled_merged_row_indice.dtype != torch.int16:
        raise RuntimeError("ter_spmm: row indices must be int16")
    if w_tiled_merged_col_offset.dtype != torch.int32:
        raise RuntimeError("ter_spmm: col offsets must be int32")
    if X.dtype not in (torch.float32, torch.float16, torch.bfloat16, torch.int8):
        raise RuntimeError(f"ter_spmm: unsupported activation dtype {X.dtype}")
    X = X.contiguous()
    y_dtype = torch.int32 if X.dtype == torch.int8 else X.dtype
    layout = _lib.ROW_MAJOR if X.shape[-1] == inners else _lib.COL_MAJOR
    if layout == _lib.COL_MAJOR and not (X.dim() >= 2 and X.shape[-2] == inners):
        raise RuntimeError(f"ter_spmm: activation of shape {tuple(X.shape)} has no dimension of {inners} inners")
    if X.numel() != max(batch_size, 0) * rows * inners and batch_size > 0:
        raise RuntimeError("ter_spmm: activation size does not match batch_size*rows*inners")
    if tile_k is None:
        tile_k = tile_size_for(inners)
    tiles = -(-inners // tile_k)
    if w_tiled_merged_col_offset.numel() != columns * tiles * 4:
        raise RuntimeError("ter_spmm: col offsets do not have columns*ceil(inners/TILE_K)*4 entries")
    if out is None:
        out = torch.empty((batch_size, rows, columns), device=X.device, dtype=y_dtype)
    elif out.dtype != y_dtype or out.numel() != batch_size * rows * columns or not out.is_contiguous():
        raise RuntimeError("ter_spmm: out has the wrong dtype, size or strides")
    if batch_size == 0:
        return out                      # the reference launches nothing for an empty batch (TernaryLinear.py:168)
    tile_ptr = w_col_tile_indices.data_ptr() if w_col_tile_indices is not None and w_col_tile_indices.numel() else None
    if AUTO_PREPARE and not torch.cuda.is_current_stream_capturing():
        prepare(w_tiled_merged_row_indice, w_tiled_merged_col_offset, columns, inners, tile_k)
    with torch.cuda.device(X.device):
        check(lib().tllm_ter_spmm(X.data_ptr(), _lib.torch_dtype_code(X.dtype), layout, w_tiled_merged_row_indice.data_ptr(),
                                  w_tiled_merged_col_offset.data_ptr(), tile_ptr, out.data_ptr(), _lib.torch_dtype_code(y_dtype),
                                  int(batch_size), int(rows), int(columns), int(inners), int(tile_k), float(scale),
                                  int(bool(uniformed)), int(bool(padded)), torch.cuda.current_stream().cuda_stream), "ter_spmm")
    return out


def prepare(w_tiled_merged_row_indice, w_tiled_merged_col_offset, columns, inners, tile_k=None):
    """Repack one weight held in the reference's device arrays, once (tllm_ter_spmm_prepare): later `ter_spmm` calls with
    the same two tensors run the packed kernels.  The tensors must stay alive and unchanged; `forget` drops the copy."""
    import torch

    if tile_k is None:
        tile_k = tile_size_for(inners)
    with torch.cuda.device(w_tiled_merged_row_indice.device):
        check(lib().tllm_ter_spmm_prepare(w_tiled_merged_row_indice.data_ptr(), w_tiled_merged_col_offset.data_ptr(), int(columns), int(inners),
                                          int(tile_k)), "ter_spmm.prepare")


def forget(w_tiled_merged_row_indice=None, w_tiled_merged_col_offset=None):
    """Drops the packed copy made by `prepare` for these tensors (no arguments: all of them); returns how many."""
    a = w_tiled_merged_row_indice.data_ptr() if w_tiled_merged_row_indice is not None else None
    b = w_tiled_merged_col_offset.data_ptr() if w_tiled_merged_col_offset is not None else None
    return int(lib().tllm_ter_spmm_forget(a, b))


def install(auto_prepare=False):
    """Make `import ter_spmm` resolve to this module (for unmodified reference code).  With auto_prepare, the first
    `ter_spmm` call that sees a pair of weight tensors outside a stream capture repacks it (see `prepare`)."""
    global AUTO_PREPARE
    AUTO_PREPARE = bool(auto_prepare)
    """Make `import ter_spmm` resolve to this module (for unmodified reference code)."""
    sys.modules.setdefault("ter_spmm", sys.modules[__name__])
    return sys.modules["ter_spmm"]
