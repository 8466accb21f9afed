"""PackedWeight / PackedMLP: thin owners of the C-ABI handles (tllm_weight, tllm_mlp)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import PackOpts, WeightInfo, check, lib, np_ptr


def _opts(tile_rows=0, num_ctas=0, max_rows=0, k_splits=0, no_bit_tiles=0, no_nibbles=0):
    return PackOpts(int(tile_rows), int(num_ctas), 0, int(max_rows), int(k_splits), int(no_bit_tiles), int(no_nibbles))


def _dense_i8(w):
    if hasattr(w, "detach"):
        w = w.detach().cpu().numpy()
    w = np.ascontiguousarray(w)
    if w.dtype != np.int8:
        if np.any((w < -1) | (w > 1)):
            raise ValueError("weight is not ternary")
        w = w.astype(np.int8)
    return w


class PackedWeight:
    """A ternary matrix W [inners, columns] packed into the bank-stream format on the current CUDA device."""

    def __init__(self, handle, device_index):
        self._h = handle
        self.device_index = device_index

    # ---- constructors -------------------------------------------------------------------------------
    @classmethod
    def from_dense(cls, w, scale=1.0, device=None, **opts):
        w = _dense_i8(w)
        K, N = w.shape
        return cls._create(lambda o, h: lib().tllm_weight_create_dense(np_ptr(w), K, N, float(scale), C.byref(o), C.byref(h)),
                           device, opts)

    @classmethod
    def from_ssr(cls, image, inners, columns, scale=1.0, device=None, **opts):
        """From the library's sparse-segment image (`ternaryllm_b200.ssr.encode`): validated and decoded on the host."""
        img = np.ascontiguousarray(np.asarray(image), dtype=np.uint8)
        return cls._create(lambda o, h: lib().tllm_weight_create_ssr(np_ptr(img), img.size, int(inners), int(columns), float(scale),
                                                                     C.byref(o), C.byref(h)),
                           device, opts)

    @classmethod
    def from_mcsc(cls, row_idx, col_off, columns, inners, tile_k, scale=1.0, device=None, **opts):
        ri = np.ascontiguousarray(np.asarray(row_idx), dtype=np.int32)
        co = np.ascontiguousarray(np.asarray(col_off), dtype=np.int32)
        return cls._create(lambda o, h: lib().tllm_weight_create_mcsc(np_ptr(ri), np_ptr(co), int(columns), int(inners),
                                                                      int(tile_k), float(scale), C.byref(o), C.byref(h)),
                           device, opts)

    @classmethod
    def from_cpu_format(cls, kind, group, chunk, metadata, row_index, columns, inners, aux=0, scale=1.0, device=None, **opts):
        meta = np.ascontiguousarray(np.asarray(metadata), dtype=np.int32)
        ri = np.ascontiguousarray(np.asarray(row_index))
        if ri.dtype not in (np.int16, np.int32):
            raise ValueError("row_index must be int16 or int32")
        return cls._create(lambda o, h: lib().tllm_weight_create_cpu_format(int(kind), int(group), int(chunk), np_ptr(meta), np_ptr(ri),
                                                                            int(ri.dtype == np.int32), int(aux), int(columns),
                                                                            int(inners), float(scale), C.byref(o), C.byref(h)),
                           device, opts)

    @classmethod
    def _create(cls, fn, device, opts):
        import torch

        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        if dev.type != "cuda":
            raise RuntimeError("PackedWeight lives on a CUDA device; there is no CPU implementation")
        h = C.c_void_p()
        o = _opts(**opts)
        with torch.cuda.device(dev):
            check(fn(o, h), "PackedWeight")
        return cls(h, dev.index if dev.index is not None else torch.cuda.current_device())

    @classmethod
    def load(cls, path, device=None):
        """A handle from a file written by `save` (no repacking)."""
        import torch

        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        h = C.c_void_p()
        with torch.cuda.device(dev):
            check(lib().tllm_weight_load(str(path).encode(), C.byref(h)), "PackedWeight.load")
        return cls(h, dev.index if dev.index is not None else torch.cuda.current_device())

    def save(self, path):
        check(lib().tllm_weight_save(self._h, str(path).encode()), "PackedWeight.save")

    # ---- use ---------------------------------------------------------------------------------------
    @property
    def info(self):
        i = WeightInfo()
        check(lib().tllm_weight_get_info(self._h, C.byref(i)))
        return i.as_dict()

    def set_scale(self, s):
        check(lib().tllm_weight_set_scale(self._h, float(s)))

    def check(self):
        check(lib().tllm_weight_check(self._h), "PackedWeight")

    def matmul(self, x, out=None, col_major=False):
        """y = x @ W * s for a 2-D CUDA tensor x [rows, inners] (or [inners, rows] with col_major)."""
        import torch

        if x.device.type != "cuda" or x.device.index != self.device_index:
            raise RuntimeError("activation must be on the CUDA device that holds the packed weight")
        if x.dim() != 2:
            raise RuntimeError("matmul expects a 2-D activation")
        x = x.contiguous()
        info = self.info
        rows = x.shape[1] if col_major else x.shape[0]
        if (x.shape[0] if col_major else x.shape[1]) != info["inners"]:
            raise RuntimeError(f"activation has {x.shape} but the weight has {info['inners']} inners")
        ydt = torch.int32 if x.dtype == torch.int8 else x.dtype
        if out is None:
            out = torch.empty((rows, info["columns"]), device=x.device, dtype=ydt)
        elif (out.dtype != ydt and not (out.dtype == torch.float32 and ydt != torch.int32)) or \
                tuple(out.shape) != (rows, info["columns"]) or not out.is_contiguous():
            raise RuntimeError("out has the wrong dtype, shape or strides")
        with torch.cuda.device(x.device):
            check(lib().tllm_spmm(self._h, x.data_ptr(), _lib.torch_dtype_code(x.dtype), _lib.COL_MAJOR if col_major else _lib.ROW_MAJOR,
                                  rows, out.data_ptr(), _lib.torch_dtype_code(out.dtype), torch.cuda.current_stream().cuda_stream), "tllm_spmm")
        return out

    def matmul_host(self, x, col_major=False, y_col_major=False):
        """Same on numpy host arrays (copies in, runs, copies out, synchronises): the CPU entry points' form."""
        import torch

        x = np.ascontiguousarray(x)
        code = {np.dtype(np.float32): _lib.F32, np.dtype(np.float16): _lib.F16, np.dtype(np.int8): _lib.I8}[x.dtype]
        info = self.info
        rows = x.shape[1] if col_major else x.shape[0]
        ydt = np.int32 if x.dtype == np.int8 else x.dtype
        y = np.empty((info["columns"], rows) if y_col_major else (rows, info["columns"]), ydt)
        with torch.cuda.device(self.device_index):
            check(lib().tllm_spmm_host(self._h, np_ptr(x), code, _lib.COL_MAJOR if col_major else _lib.ROW_MAJOR, rows, np_ptr(y),
                                       _lib.I32 if x.dtype == np.int8 else code, _lib.COL_MAJOR if y_col_major else _lib.ROW_MAJOR),
                  "tllm_spmm_host")
        return y

    def close(self):
        if self._h:
            lib().tllm_weight_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def ternarize(w, sparsity=None, threshold_factor=0.7):
    """Float weights [inners, columns] -> (int8 ternary weights, per-tensor scale); see tllm_ternarize."""
    if hasattr(w, "detach"):
        w = w.detach().float().cpu().numpy()
    w = np.ascontiguousarray(w, dtype=np.float32)
    if w.ndim != 2:
        raise ValueError("ternarize expects a 2-D weight")
    out = np.empty(w.shape, np.int8)
    scale = C.c_float()
    check(lib().tllm_ternarize(np_ptr(w), w.shape[0], w.shape[1], float(threshold_factor), float(sparsity or 0.0), np_ptr(out), C.byref(scale)),
          "tllm_ternarize")
    return out, float(scale.value)


class PackedMLP:
    """gate / up / down of one ternary MLP block, fused (see tllm_mlp_* in include/tllm.h)."""

    def __init__(self, w_gate, w_up, w_down, s_gate=1.0, s_up=1.0, s_down=1.0, device=None, **opts):
        import torch

        g, u, d = _dense_i8(w_gate), _dense_i8(w_up), _dense_i8(w_down)
        hidden, inter = g.shape
        if u.shape != (hidden, inter) or d.shape != (inter, hidden):
            raise ValueError("gate/up must be [hidden, intermediate] and down [intermediate, hidden]")
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.device_index = dev.index if dev.index is not None else torch.cuda.current_device()
        self.hidden, self.inter = hidden, inter
        h = C.c_void_p()
        o = _opts(**opts)
        with torch.cuda.device(dev):
            check(lib().tllm_mlp_create(np_ptr(g), np_ptr(u), np_ptr(d), hidden, inter, float(s_gate), float(s_up), float(s_down),
                                        C.byref(o), C.byref(h)), "PackedMLP")
        self._h = h

    @property
    def info(self):
        a, b = WeightInfo(), WeightInfo()
        check(lib().tllm_mlp_get_info(self._h, C.byref(a), C.byref(b)))
        return a.as_dict(), b.as_dict()

    def forward(self, x, out=None, h=None):
        import torch

        if x.device.type != "cuda" or x.dim() != 2 or x.shape[1] != self.hidden:
            raise RuntimeError("PackedMLP.forward expects a 2-D CUDA activation [rows, hidden]")
        x = x.contiguous()
        rows = x.shape[0]
        if out is None:
            out = torch.empty((rows, self.hidden), device=x.device, dtype=x.dtype)
        elif out.dtype not in (x.dtype, torch.float32) or tuple(out.shape) != (rows, self.hidden) or not out.is_contiguous():
            raise RuntimeError("out has the wrong dtype, shape or strides")
        if h is None and rows > 16:
            h = torch.empty((rows, self.inter), device=x.device, dtype=x.dtype)
        with torch.cuda.device(x.device):
            check(lib().tllm_mlp_forward_ex(self._h, x.data_ptr(), _lib.torch_dtype_code(x.dtype), rows, out.data_ptr(),
                                            _lib.torch_dtype_code(out.dtype), h.data_ptr() if h is not None else None,
                                            torch.cuda.current_stream().cuda_stream), "tllm_mlp_forward")
        return out

    def close(self):
        if self._h:
            lib().tllm_mlp_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
