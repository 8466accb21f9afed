"""CPU oracle for the ternary sparse product path -- TEST INFRASTRUCTURE ONLY.

`oracle.c` restates the reference's algorithms in plain C; `ref_shim.cpp` compiles the reference's own
CPU kernels in place (into oracle/_ref/).  This module loads both with ctypes and wraps them in numpy
signatures.  Only tests, the smoke check and the benchmark's CPU-baseline leg import it; the shipped
package never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_BUILD = os.path.join(HERE, "_build")
_LIB = os.path.join(_BUILD, "liboracle.so")
_REF = os.path.join(HERE, "_ref", "libtllm_ref.so")

_lib = None
_ref = None


def build(force: bool = False) -> str:
    """Compile oracle.c with gcc into oracle/_build/liboracle.so (a second or so)."""
    src = os.path.join(HERE, "oracle.c")
    if force or not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(src):
        os.makedirs(_BUILD, exist_ok=True)
        subprocess.check_call(["gcc", "-O2", "-std=c11", "-fPIC", "-shared", src, "-o", _LIB, "-lm"])
    return _LIB


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _lib.orc_ter_tiled_mcsc.restype = C.c_int64
        _lib.orc_merged_group.restype = C.c_int64
        _lib.orc_round.restype = C.c_double
        _lib.orc_round.argtypes = [C.c_double, C.c_int]
    return _lib


def reference_root() -> str:
    """Where a checkout of the reference project is looked for: $TLLM_REFERENCE_ROOT, else a directory named
    `reference` beside this repository.  It need not exist; callers test for the sources they want."""
    env = os.environ.get("TLLM_REFERENCE_ROOT")
    return env if env else os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def have_ref() -> bool:
    return os.path.exists(_REF)


def host_has_avx512() -> bool:
    try:
        flags = open("/proc/cpuinfo").read()
    except OSError:
        return False
    return all(f in flags for f in (" avx512f", " avx512bw", " avx512vl", " avx2", " fma"))


def ref():
    """The compiled reference (None when absent or when this host cannot run its AVX-512 code)."""
    global _ref
    if _ref is None and have_ref() and host_has_avx512():
        _ref = C.CDLL(_REF)
        for n in ("ref_sparse_format", "ref_merged_tcsc", "ref_merged_group"):
            getattr(_ref, n).restype = C.c_int64
    return _ref


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


# ------------------------------------------------------------------------------------------------
# ground truth
# ------------------------------------------------------------------------------------------------
def dense_f64(X, W, scale=1.0):
    """Y = (X as fp64) @ W * scale; X [M,K], W [K,N] in {-1,0,1}."""
    X = _c(X, np.float64)
    W = _c(W, np.int8)
    M, K = X.shape
    N = W.shape[1]
    Y = np.empty((M, N), np.float64)
    lib().orc_dense_f64(_p(X), _p(W), C.c_double(float(scale)), _p(Y), M, N, K)
    return Y


def dense_i64(X, W):
    X = _c(X, np.int8)
    W = _c(W, np.int8)
    M, K = X.shape
    N = W.shape[1]
    Y = np.empty((M, N), np.int64)
    lib().orc_dense_i64(_p(X), _p(W), _p(Y), M, N, K)
    return Y


def int8_wrap(X, W):
    X = _c(X, np.int8)
    W = _c(W, np.int8)
    M, K = X.shape
    N = W.shape[1]
    Y = np.empty((M, N), np.int8)
    lib().orc_int8_wrap(_p(X), _p(W), _p(Y), M, N, K)
    return Y


def round_to(a, mode):
    """mode: 0 none, 1 fp16, 2 bf16, 3 fp32 (round-to-nearest-even), elementwise on fp64."""
    a = np.asarray(a, np.float64)
    f = np.vectorize(lambda v: lib().orc_round(float(v), int(mode)), otypes=[np.float64])
    return f(a)


def silu_mul_f32(x, xb):
    x = _c(x, np.float32).copy()
    xb = _c(xb, np.float32)
    lib().orc_silu_mul_f32(x.size, _p(x), _p(xb))
    return x


def mlp_f64(X, Wg, Wu, Wd, sg, su, sd, h_round=0):
    X = _c(X, np.float64)
    Wg, Wu, Wd = _c(Wg, np.int8), _c(Wu, np.int8), _c(Wd, np.int8)
    M, hidden = X.shape
    inter = Wg.shape[1]
    Y = np.empty((M, hidden), np.float64)
    lib().orc_mlp_f64(_p(X), _p(Wg), _p(Wu), _p(Wd), C.c_double(sg), C.c_double(su), C.c_double(sd),
                      int(h_round), _p(Y), M, hidden, inter)
    return Y


# ------------------------------------------------------------------------------------------------
# GPU-side formats
# ------------------------------------------------------------------------------------------------
def ter_csc(w):
    w = _c(w, np.int32)
    K, N = w.shape
    pos = int((w == 1).sum())
    neg = int((w == -1).sum())
    ni, no = np.zeros(neg, np.int32), np.zeros(N + 1, np.int32)
    pi, po = np.zeros(pos, np.int32), np.zeros(N + 1, np.int32)
    lib().orc_ter_csc(_p(w), N, K, _p(ni), _p(no), _p(pi), _p(po))
    return ni, no, pi, po


def ter_tiled_csc(w, T):
    w = _c(w, np.int32)
    K, N = w.shape
    tiles = -(-K // T)
    pos = int((w == 1).sum())
    neg = int((w == -1).sum())
    ni, no = np.zeros(neg, np.int32), np.zeros(N * tiles * 2, np.int32)
    pi, po = np.zeros(pos, np.int32), np.zeros(N * tiles * 2, np.int32)
    lib().orc_ter_tiled_csc(_p(w), N, K, T, _p(ni), _p(no), _p(pi), _p(po))
    return ni, no, pi, po


def ter_tiled_mcsc(w, T, padding=False, padding_size=4, lossy=False):
    w = _c(w, np.int32)
    K, N = w.shape
    tiles = -(-K // T)
    nnz = int((w != 0).sum())
    cap = nnz + (2 * padding_size * N * tiles if padding else 0) + 8
    idx = np.zeros(cap, np.int32)
    off = np.zeros(N * tiles * 4, np.int32)
    til = np.zeros(N * tiles, np.int32)
    n = lib().orc_ter_tiled_mcsc(_p(w), N, K, T, int(padding), int(padding_size), int(lossy), _p(idx),
                                 C.c_int64(cap), _p(off), _p(til))
    assert n >= 0
    return idx[:n].copy(), off, til


def mcsc_product_f64(X, idx, off, N, K, T, scale=1.0, x_colmajor=False):
    X = _c(X, np.float64)
    M = X.shape[1] if x_colmajor else X.shape[0]
    idx = _c(idx, np.int32)
    off = _c(off, np.int32)
    Y = np.empty((M, N), np.float64)
    lib().orc_mcsc_product_f64(_p(X), int(x_colmajor), _p(idx), _p(off), M, N, K, T, C.c_double(scale), _p(Y))
    return Y


# ------------------------------------------------------------------------------------------------
# CPU-side formats
# ------------------------------------------------------------------------------------------------
def sparse_format(W):
    W = _c(W, np.int8)
    K, N = W.shape
    pos = int((W >= 1).sum())
    neg = int((W <= -1).sum())
    csp, csn = np.zeros(N + 1, np.int32), np.zeros(N + 1, np.int32)
    rip, rin = np.zeros(pos, np.int16), np.zeros(neg, np.int16)
    lib().orc_sparse_format(_p(W), K, N, _p(csp), _p(csn), _p(rip), _p(rin))
    return csp, csn, rip, rin


def merged_tcsc(W):
    csp, csn, rip, rin = sparse_format(W)
    N = len(csp) - 1
    meta = np.zeros(4 * N, np.int32)
    ri = np.zeros(len(rip) + len(rin), np.int16)
    lib().orc_merged_tcsc(_p(csp), _p(csn), _p(rip), _p(rin), N, _p(meta), _p(ri))
    return meta, ri


METHODS = {"min": 0, "mid": 1, "max": 2, "uniform": 3}


def merged_group(W, G, method="min", interleaved=True, simd=0):
    csp, csn, rip, rin = sparse_format(W)
    K, N = np.asarray(W).shape
    meta_cap = (N // G + 1) * (2 + 2 * G) + 8
    ri_cap = 2 * (len(rip) + len(rin)) + 2 * N * K // max(1, G) + 64
    ri_cap = max(ri_cap, 4 * N * 64)
    meta = np.zeros(meta_cap, np.int32)
    ri = np.zeros(ri_cap, np.int16)
    ml = C.c_int64(0)
    n = lib().orc_merged_group(_p(csp), _p(csn), _p(rip), _p(rin), N, G, METHODS[method], int(interleaved),
                               int(simd), _p(meta), C.c_int64(meta_cap), _p(ri), C.c_int64(ri_cap), C.byref(ml))
    assert n >= 0, "capacity"
    return meta[: ml.value].copy(), ri[:n].copy()


def cpu_decode_dense(kind, G, chunk, meta, ri, N, K, aux=0):
    meta = _c(meta, np.int32)
    ri = np.ascontiguousarray(ri)
    assert ri.dtype in (np.int16, np.int32)
    Wd = np.zeros((K, N), np.int8)
    r = lib().orc_cpu_decode_dense(int(kind), int(G), int(chunk), _p(meta), _p(ri), int(ri.dtype == np.int32),
                                   C.c_int64(aux), N, K, _p(Wd))
    assert r == 0
    return Wd


# ------------------------------------------------------------------------------------------------
# compiled reference (oracle/_ref)
# ------------------------------------------------------------------------------------------------
_FAM = {"F1": 1, "F2": 2, "F3": 3, "F4": 4, "F4U": 5, "F5": 6, "F6": 7, "F6U": 8, "FD": 9}


def ref_names(family):
    r = ref()
    buf = C.create_string_buffer(1 << 16)
    n = r.ref_list(_FAM[family], buf, len(buf))
    return buf.value.decode().split() if n > 0 else []


def ref_merged_tcsc(W):
    W = _c(W, np.int8)
    K, N = W.shape
    meta = np.zeros(4 * N, np.int32)
    cap = int((W != 0).sum()) + 8
    ri = np.zeros(cap, np.int16)
    n = ref().ref_merged_tcsc(_p(W), K, N, _p(meta), _p(ri), C.c_int64(cap))
    return meta, ri[:n].copy()


def ref_sparse_format(W):
    W = _c(W, np.int8)
    K, N = W.shape
    cap = int((W != 0).sum()) + 8
    csp, csn = np.zeros(N + 1, np.int32), np.zeros(N + 1, np.int32)
    rip, rin = np.zeros(cap, np.int16), np.zeros(cap, np.int16)
    nn = C.c_int64(0)
    npos = ref().ref_sparse_format(_p(W), K, N, _p(csp), _p(csn), _p(rip), _p(rin), C.c_int64(cap), C.byref(nn))
    return csp, csn, rip[:npos].copy(), rin[: nn.value].copy()


def ref_merged_group(W, G, method="min", interleaved=True, simd=0):
    W = _c(W, np.int8)
    K, N = W.shape
    meta_cap = (N // G + 1) * (2 + 2 * G) + 8
    ri_cap = max(4 * int((W != 0).sum()) + 64, 4 * N * 64)
    meta = np.zeros(meta_cap, np.int32)
    ri = np.zeros(ri_cap, np.int16)
    ml = C.c_int64(0)
    n = ref().ref_merged_group(_p(W), K, N, G, method.encode(), int(interleaved), int(simd), _p(meta),
                               C.c_int64(meta_cap), _p(ri), C.c_int64(ri_cap), C.byref(ml))
    assert n >= 0 and ml.value >= 0
    return meta[: ml.value].copy(), ri[:n].copy()


def ref_call(family, name, *args):
    """Call a reference kernel by name; args are numpy arrays / ints in the kernel's own order."""
    fn = getattr(ref(), "ref_" + family.lower())
    conv = [name.encode()]
    for a in args:
        if isinstance(a, np.ndarray):
            conv.append(_p(a))
        else:
            conv.append(C.c_int32(int(a)))
    r = fn(*conv)
    if r != 0:
        raise KeyError(name)


def ternarize_f64(w, sparsity=None, threshold_factor=0.7):
    """Restatement of the product's float -> ternary rule (tllm_ternarize; the reference's ternarize_weights is a stub,
    ternaryLLM_GPU/TernaryLLM/TernaryLinear.py:19-20, so parity is unpinned and this numpy version is the definition):
    zero what is at or below the threshold, sign() for the rest, scale = mean |w| of the kept entries."""
    w = np.asarray(w, dtype=np.float32)
    a = np.abs(w).astype(np.float64)
    if sparsity:
        k = int(np.rint(np.float64(np.float32(sparsity)) * a.size))
        thr = -1.0 if k == 0 else np.partition(a.ravel(), k - 1)[k - 1]
    else:
        thr = np.float64(np.float32(threshold_factor if threshold_factor > 0 else 0.7)) * (a.sum() / a.size)
    keep = a > thr
    t = np.where(keep, np.sign(w), 0).astype(np.int8)
    return t, (float(a[keep].mean()) if keep.any() else 0.0)
