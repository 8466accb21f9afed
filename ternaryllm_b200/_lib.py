"""ctypes binding of libtllm.so, the C-ABI shared library declared in include/tllm.h.

There is no fallback: if the library has not been built, loading raises with the build command; if it
has been built but no CUDA device is usable, the device-side entry points return an error which
`check()` turns into a RuntimeError.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libtllm.so")

F32, F16, BF16, I8, I32 = 0, 1, 2, 3, 4
ROW_MAJOR, COL_MAJOR = 0, 1


class PackOpts(C.Structure):
    _fields_ = [("tile_rows", C.c_int), ("num_ctas", C.c_int), ("reserved0", C.c_int), ("max_rows", C.c_int),
                ("k_splits", C.c_int), ("no_bit_tiles", C.c_int), ("no_nibbles", C.c_int), ("reserved", C.c_int * 1)]


class WeightInfo(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("inners", "columns", "tile_rows", "tiles", "col_blocks", "k_splits",
                                       "tiles_per_cta", "num_ctas", "units", "max_rows")] + [
        (n, C.c_int64) for n in ("nnz", "stream_bytes", "meta_bytes", "scratch_bytes", "algorithmic_bytes", "bit_tile_bytes", "nibble_bytes")] + [
        ("scale", C.c_float)]

    def as_dict(self):
        return {n: getattr(self, n) for n, _ in self._fields_}


# every symbol include/tllm.h declares, with its signature
_P, _I, _L, _F = C.c_void_p, C.c_int, C.c_int64, C.c_float
SIGNATURES = {
    "tllm_last_error": (C.c_char_p, []),
    "tllm_version": (_I, []),
    "tllm_launch_count": (_L, []),
    "tllm_mma_launch_count": (_L, []),
    "tllm_set_mma_min_rows": (_I, [_I]),
    "tllm_set_nibble_max_rows": (_I, [_I]),
    "tllm_nibble_launch_count": (_L, []),
    "tllm_count_nnz": (_I, [_P, _I, _I, _P, _P]),
    "tllm_convert_to_ter_csc": (_I, [_P, _I, _I, _P, _P, _P, _P]),
    "tllm_convert_to_ter_tiled_csc": (_I, [_P, _I, _I, _I, _P, _P, _P, _P]),
    "tllm_ter_tiled_mcsc_len": (_L, [_P, _I, _I, _I, _I, _I, _I]),
    "tllm_convert_to_ter_tiled_mcsc": (_I, [_P, _I, _I, _I, _I, _I, _I, _P, _L, _P, _P]),
    "tllm_ter_spmm": (_I, [_P, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _I, _P]),
    "tllm_ter_spmm_prepare": (_I, [_P, _P, _I, _I, _I]),
    "tllm_ter_spmm_forget": (_I, [_P, _P]),
    "tllm_ternarize": (_I, [_P, _I, _I, _F, _F, _P, _P]),
    "tllm_ssr_encode": (_I, [_P, _I, _I, _P, C.c_size_t, _P]),
    "tllm_ssr_decode": (_I, [_P, C.c_size_t, _I, _I, _P]),
    "tllm_weight_create_ssr": (_I, [_P, C.c_size_t, _I, _I, _F, _P, _P]),
    "tllm_weight_save": (_I, [_P, C.c_char_p]),
    "tllm_weight_load": (_I, [C.c_char_p, _P]),
    "tllm_weight_create_dense": (_I, [_P, _I, _I, _F, _P, _P]),
    "tllm_weight_create_mcsc": (_I, [_P, _P, _I, _I, _I, _F, _P, _P]),
    "tllm_weight_create_mcsc_device": (_I, [_P, _L, _P, _I, _I, _I, _F, _P, _P]),
    "tllm_weight_create_cpu_format": (_I, [_I, _I, _I, _P, _P, _I, _L, _I, _I, _F, _P, _P]),
    "tllm_pack_roundtrip": (_I, [_P, _I, _I, _P, _I, _P, _P]),
    "tllm_nibble_schedule": (_I, [_I, _I, _I, _P, _P, C.c_size_t]),
    "tllm_pack_corrupt_check": (_I, [_P, _I, _I, _P, _I, _I, _L, C.c_uint32]),
    "tllm_weight_destroy": (_I, [_P]),
    "tllm_weight_get_info": (_I, [_P, _P]),
    "tllm_weight_set_scale": (_I, [_P, _F]),
    "tllm_weight_check": (_I, [_P]),
    "tllm_spmm": (_I, [_P, _P, _I, _I, _I, _P, _I, _P]),
    "tllm_spmm_host": (_I, [_P, _P, _I, _I, _I, _P, _I, _I]),
    "tllm_spmm_host_bias": (_I, [_P, _P, _I, _I, _I, _P, _P, _I, _I]),
    "tllm_spmm_static_scratch": (_I, [_P, _P, _I, _I, _I, _P, _I, _P]),
    "tllm_mlp_create": (_I, [_P, _P, _P, _I, _I, _F, _F, _F, _P, _P]),
    "tllm_mlp_destroy": (_I, [_P]),
    "tllm_mlp_forward": (_I, [_P, _P, _I, _I, _P, _P, _P]),
    "tllm_mlp_forward_ex": (_I, [_P, _P, _I, _I, _P, _I, _P, _P]),
    "tllm_mlp_forward_host": (_I, [_P, _P, _I, _I, _I, _P]),
    "tllm_mlp_create_cpu_format": (_I, [_I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _I, _I, _P, _P]),
    "tllm_mlp_get_info": (_I, [_P, _P, _P]),
    "tllm_silu_mul": (_I, [_P, _P, _I, _L, _P]),
    "tllm_add_rmsnorm": (_I, [_P, _P, _P, _P, _I, _I, _I, _F, _P]),
    "tllm_comm_create": (_I, [_I, _I, _I, _I, _P]),
    "tllm_comm_handle_bytes": (_I, []),
    "tllm_comm_export": (_I, [_P, _P]),
    "tllm_comm_connect": (_I, [_P, _P]),
    "tllm_comm_attach": (_I, [_P, _I, _P, _P]),
    "tllm_comm_buffers": (_I, [_P, _P, _P, _P, _P]),
    "tllm_comm_set_wait_limit": (_I, [_P, C.c_double]),
    "tllm_comm_check": (_I, [_P]),
    "tllm_comm_destroy": (_I, [_P]),
    "tllm_allreduce_add_rmsnorm": (_I, [_P, _P, _P, _P, _P, _I, _I, _F, _P]),
}

_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m ternaryllm_b200.build` "
                "(needs nvcc; there is no CPU fallback for this library)")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(rc: int, what: str = "libtllm"):
    if rc != 0:
        msg = lib().tllm_last_error()
        raise RuntimeError(f"{what}: {msg.decode() if msg else 'error'} (code {rc})")


def np_ptr(a):
    return a.ctypes.data_as(C.c_void_p)


def torch_dtype_code(dt):
    import torch

    return {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16, torch.int8: I8, torch.int32: I32}[dt]
