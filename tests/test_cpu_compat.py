"""include/tllm_cpu_compat.hpp: the reference's CPU kernels by name (ternaryLLM_CPU/src/GEMM_CPU_FP32.hpp:40-185,
GEMM_CPU_INT8.hpp:11-29) forwarding to the C ABI.  The header must compile on its own; on a GPU, one wrapper of every
parameter-list family is called with the fixture's arrays (built by the reference's own format classes) and must
leave in `result` exactly what the reference kernel of that name left there (tests/golden/cpu_reference.npz)."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INC = os.path.join(ROOT, "include")


def test_header_compiles_standalone_and_names_every_family(tmp_path):
    src = tmp_path / "t.cpp"
    src.write_text('#include "tllm_cpu_compat.hpp"\nint main() { return 0; }\n')
    subprocess.check_call(["g++", "-std=c++17", "-fsyntax-only", "-I", INC, str(src)])
    text = open(os.path.join(INC, "tllm_cpu_compat.hpp")).read()
    for name in ("GEMM_CPU_FP32_colMajor_TCSC_Merged_GroupMin_8xG16_AVX2_OpenMP", "GEMM_CPU_FP32_colMajor_TCSC_Uniform_16xG16_AVX512_OpenMP",
                 "GEMM_CPU_FP32_rowMajor_TCSC_Merged_GroupMin_4xG8_AVX2_OpenMP", "GEMV_CPU_FP32_rowMajor_TCSC_Merged_GroupMin_G128_CS16_AVX512_OpenMP",
                 "GEMV_CPU_FP32_rowMajor_TCSC_Uniform_G16_CS8_AVX2_OpenMP", "GEMM_CPU_FP32_colMajor_TCSC_Naive",
                 "GEMM_CPU_INT8_colMajor_TCSC_Merged_GroupMin_64xG4_AVX2_OpenMP"):
        assert f"inline void {name}(" in text


def _build_helper(tmp_path):
    from ternaryllm_b200 import _lib

    so = tmp_path / "libcompat_check.so"
    subprocess.check_call(["g++", "-std=c++17", "-O1", "-fPIC", "-shared", "-I", INC, os.path.join(ROOT, "tests", "compat_check.cpp"),
                           "-o", str(so), _lib.LIB_PATH, f"-Wl,-rpath,{os.path.dirname(_lib.LIB_PATH)}"])
    _lib.lib()                                    # libtllm first, so that the helper binds to the same copy
    return C.CDLL(str(so))


def test_group_format_builder_matches_the_reference_builder(cpu_reference, tmp_path):
    """tllm_compat::build_group_format (what TernaryMLP keeps in its W*_metadata / W*_rowindex members) against the
    arrays the reference's own MergedTCSC_Group constructor produced for the fixture matrices (TCSC.hpp:99-243):
    "min" interleaved and not, "uniform" interleaved and not.  Host code only."""
    L = _build_helper(tmp_path)
    fx = cpu_reference
    P = lambda a: a.ctypes.data_as(C.c_void_p)
    for wname, G, method, inter in (("W", 16, "min", 1), ("W", 8, "min", 0), ("W", 32, "min", 0), ("W", 4, "min", 1),
                                    ("Wun", 16, "uniform", 1), ("Wun", 16, "uniform", 0)):
        key = f"grp.{wname}.G{G}.{method}.i{inter}.s0"
        if key + ".meta" not in fx.files:
            continue
        w = np.ascontiguousarray(fx[wname], np.int8)
        K, N = w.shape
        want_meta, want_ri = fx[key + ".meta"].astype(np.int32), fx[key + ".ri"].astype(np.int16)
        meta, ri = np.zeros(len(want_meta) + 64, np.int32), np.zeros(len(want_ri) + 64, np.int16)
        nm, nr = C.c_int(len(meta)), C.c_int(len(ri))
        assert L.chk_build_group16(P(w), K, N, G, int(method == "uniform"), inter, P(meta), C.byref(nm), P(ri), C.byref(nr)) == 0, key
        assert np.array_equal(meta[: nm.value], want_meta), key
        assert np.array_equal(ri[: nr.value], want_ri), key
    # a matrix that is not uniform is refused as such
    w = np.ascontiguousarray(fx["W"], np.int8)
    nm, nr = C.c_int(4096), C.c_int(1 << 16)
    assert L.chk_build_group16(P(w), w.shape[0], w.shape[1], 16, 1, 1, P(np.zeros(4096, np.int32)), C.byref(nm), P(np.zeros(1 << 16, np.int16)),
                               C.byref(nr)) == -1


@pytest.mark.gpu
def test_sparse_gemm_with_bias_and_ternary_mlp_classes(cpu_reference, tmp_path):
    """tllm_compat::sparseGEMM (TCSC.hpp:413-430: the naive product plus a bias per column) and the TernaryMLP classes
    (LlamaModel.hpp:92-454: X overwritten with down(silu(X.WG) * X.WU)) against the oracle."""
    import oracle
    from conftest import random_ternary

    L = _build_helper(tmp_path)
    P = lambda a: a.ctypes.data_as(C.c_void_p)
    fx = cpu_reference
    K, N = fx["W"].shape
    X = np.ascontiguousarray(fx["X"][:5])
    bias = np.arange(N, dtype=np.float32) - 7
    Y = np.zeros((5, N), np.float32)
    i32 = lambda a: np.ascontiguousarray(a, np.int32)
    assert L.chk_sparse_gemm(P(X.copy()), P(fx["sf_rin"].astype(np.int16)), P(i32(fx["sf_csn"])), P(fx["sf_rip"].astype(np.int16)), P(i32(fx["sf_csp"])),
                             P(bias), P(Y), 5, N, K) == 0
    assert np.array_equal(Y, (oracle.dense_f64(X.astype(np.float64), fx["W"]) + bias).astype(np.float32))
    if oracle.have_ref() and oracle.host_has_avx512():
        r = oracle.ref()
        if hasattr(r, "ref_sparse_gemm_f32"):
            Yr = np.zeros((5, N), np.float32)
            r.ref_sparse_gemm_f32(P(X.copy()), P(np.ascontiguousarray(fx["W"], np.int8)), P(bias), P(Yr), 5, N, K)
            assert np.array_equal(Y, Yr)

    rng = np.random.default_rng(17)
    K, N = 256, 512
    wu, wg, wd = random_ternary(rng, K, N, 0.6), random_ternary(rng, K, N, 0.6), random_ternary(rng, N, K, 0.6)
    x = (rng.standard_normal((1, K)) * 0.25).astype(np.float32)
    once = oracle.mlp_f64(x.astype(np.float64), wg, wu, wd, 1.0, 1.0, 1.0, h_round=3)
    twice = oracle.mlp_f64(once.astype(np.float32).astype(np.float64), wg, wu, wd, 1.0, 1.0, 1.0, h_round=3)
    xb, ya, yb, grp = x.copy(), np.zeros(N, np.float32), np.zeros(N, np.float32), C.c_int(0)
    assert L.chk_mlp32(P(wu), P(wg), P(wd), K, N, 0, P(xb), P(ya), P(yb), C.byref(grp)) == 0
    assert grp.value == 64
    assert np.max(np.abs(xb.astype(np.float64) - twice)) <= 2e-5 * np.max(np.abs(twice))
    # the GEMM class: 32 rows, X and the result column-major [K][M]
    M = 32
    xm = (rng.standard_normal((M, K)) * 0.25).astype(np.float32)
    want = oracle.mlp_f64(xm.astype(np.float64), wg, wu, wd, 1.0, 1.0, 1.0, h_round=3)
    xt, ya, yb = np.ascontiguousarray(xm.T), np.zeros((N, M), np.float32), np.zeros((N, M), np.float32)
    assert L.chk_mlp16(P(wu), P(wg), P(wd), K, N, M, P(xt), P(ya), P(yb), C.byref(grp)) == 0
    assert grp.value == 16
    assert np.max(np.abs(xt.T.astype(np.float64) - want)) <= 2e-5 * np.max(np.abs(want))
    # silu(X.WG) * X.WU is left in Yb (the buffer the reference leaves it in for non-uniform weights), column-major
    g = xm.astype(np.float64) @ wg.astype(np.float64)
    h = g / (1 + np.exp(-g)) * (xm.astype(np.float64) @ wu.astype(np.float64))
    assert np.max(np.abs(yb.T.astype(np.float64) - h)) <= 2e-5 * np.max(np.abs(h))
    # the reference's constructor signature: random weights, one row, finite output; two rows are refused
    xr, ya, yb = (rng.standard_normal((1, K)) * 0.25).astype(np.float32), np.zeros(N, np.float32), np.zeros(N, np.float32)
    for uniform in (0, 1):
        assert L.chk_mlp_random(K, N, C.c_float(0.5), uniform, P(xr), P(ya), P(yb)) == 0
        assert np.isfinite(xr).all()


@pytest.mark.gpu
def test_named_wrappers_reproduce_the_reference_kernels(cpu_reference, tmp_path):
    from ternaryllm_b200 import _lib

    so = tmp_path / "libcompat_check.so"
    subprocess.check_call(["g++", "-std=c++17", "-O1", "-fPIC", "-shared", "-I", INC, os.path.join(ROOT, "tests", "compat_check.cpp"),
                           "-o", str(so), _lib.LIB_PATH, f"-Wl,-rpath,{os.path.dirname(_lib.LIB_PATH)}"])
    _lib.lib()                                    # libtllm first, so that the helper binds to the same copy
    L = C.CDLL(str(so))
    fx = cpu_reference
    K, N = fx["W"].shape
    X = np.ascontiguousarray(fx["X"])             # [M][K]
    XT = np.ascontiguousarray(X.T)                # [K][M]: the colMajor kernels' argument
    M = X.shape[0]
    P = lambda a: a.ctypes.data_as(C.c_void_p)

    def i32(a):
        return np.ascontiguousarray(a, dtype=np.int32)

    out = np.zeros((N, M), np.float32)
    k = "grp.W.G16.min.i1.s0"
    assert L.chk_f1(P(XT), P(i32(fx[k + ".meta"])), P(fx[k + ".ri"]), P(out), M, N, K) == 0
    assert np.array_equal(out, fx["direct_col.W"])
    out[:] = 0
    k = "grp.Wun.G16.uniform.i1.s0"
    assert L.chk_f2(P(XT), int(fx[k + ".meta"][0]), P(fx[k + ".ri"]), P(out), M, N, K) == 0
    assert np.array_equal(out, fx["direct_col.Wun"])
    outr = np.zeros((M, N), np.float32)
    k = "grp.W.G8.min.i0.s0"
    assert L.chk_f3(P(X.copy()), P(i32(fx[k + ".meta"])), P(i32(fx[k + ".ri"])), P(outr), M, N, K) == 0
    assert np.array_equal(outr, fx["direct_col.W"].T)
    y = np.zeros(N, np.float32)
    k = "grp.W.G32.min.i0.s0"
    assert L.chk_f4(P(X[0].copy()), P(i32(fx[k + ".meta"])), P(i32(fx[k + ".ri"])), P(y), N, K) == 0
    assert np.array_equal(y, fx["direct_col.W"][:, 0])
    k = "grp.Wun.G16.uniform.i0.s8"
    assert L.chk_f4u(P(X[0].copy()), int(fx[k + ".meta"][0]), P(i32(fx[k + ".ri"])), P(y), N, K) == 0
    assert np.array_equal(y, fx["direct_col.Wun"][:, 0])
    out[:] = 0
    assert L.chk_f5(P(XT.copy()), P(fx["sf_rin"].astype(np.int16)), P(i32(fx["sf_csn"])), P(fx["sf_rip"].astype(np.int16)), P(i32(fx["sf_csp"])),
                    P(out), M, N, K) == 0
    assert np.array_equal(out, fx["direct_col.W"])
    X8T = np.ascontiguousarray(fx["X8"].T)
    o8 = np.zeros((N, M), np.int8)
    k = "grp.W.G4.min.i0.s0"
    assert L.chk_f6(P(X8T), P(i32(fx[k + ".meta"])), P(fx[k + ".ri"]), P(o8), M, N, K) == 0
    assert np.array_equal(o8, fx["int8_col.W"])
    k = "grp.Wun.G4.uniform.i0.s0"
    assert L.chk_f6u(P(X8T), int(fx[k + ".meta"][0]), P(fx[k + ".ri"]), P(o8), M, N, K) == 0
    assert np.array_equal(o8, fx["int8_col.Wun"])
