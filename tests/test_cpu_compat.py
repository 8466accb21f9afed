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
