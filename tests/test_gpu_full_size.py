"""The benchmark configurations at their full sizes: the reference's own CPU case (C1), the fused Llama-7B-shaped MLP
block (C3) and the Llama-2-13B-shaped attention projections at prefill length (C4).

Pins: the oracle's fp64 products (bit-exact on integer-valued activations, every partial sum being an integer below
2^24; within the stated tolerance on N(0,1) activations) and, where the reference's CPU kernels were compiled on this
host (oracle/_ref), the reference kernel itself on the same seeded inputs.
"""
import numpy as np
import pytest
import torch

import oracle
from conftest import random_ternary
from ternaryllm_b200 import PackedMLP, PackedWeight, _lib

pytestmark = pytest.mark.gpu


def dev():
    return torch.device("cuda", 0)


def test_c1_reference_cpu_case_exactly():
    """M = 8, K = N = 2048, fp32 N(0,1), 50 % zeros, seed 0, through the host-buffer entry point with the column-major
    layout of the reference's colMajor kernels (GEMM_CPU_FP32.cpp:509-538): within 1e-5 of the fp64 product, bit-exact on
    integers in +-512 (the reference's own verification inputs, main.cpp:1403), and -- when the reference's kernels are
    available -- equal to GEMM_CPU_FP32_colMajor_TCSC_Merged_GroupMin_8xG16_AVX2_OpenMP on the same arrays."""
    rng = np.random.default_rng(0)
    M, K, N = 8, 2048, 2048
    w = random_ternary(rng, K, N, 0.5)
    pw = PackedWeight.from_dense(w, scale=1.0, tile_rows=512)
    X = rng.standard_normal((M, K)).astype(np.float32)
    XT = np.ascontiguousarray(X.T)                                   # [K][M]
    Y = pw.matmul_host(XT, col_major=True, y_col_major=True)         # [N][M]
    ref = oracle.dense_f64(X.astype(np.float64), w, 1.0).T
    assert np.max(np.abs(Y.astype(np.float64) - ref)) <= 1e-5 * np.max(np.abs(ref))
    Xi = rng.integers(-512, 513, size=(M, K)).astype(np.float32)
    Yi = pw.matmul_host(np.ascontiguousarray(Xi.T), col_major=True, y_col_major=True)
    assert np.array_equal(Yi.astype(np.float64), oracle.dense_f64(Xi.astype(np.float64), w, 1.0).T)
    if oracle.have_ref() and oracle.host_has_avx512():
        meta, ri = oracle.ref_merged_group(w, 16, "min", interleaved=True)
        for x, y in ((XT, Y), (np.ascontiguousarray(Xi.T), Yi)):
            out = np.zeros((N, M), np.float32)
            oracle.ref_call("F1", "GEMM_CPU_FP32_colMajor_TCSC_Merged_GroupMin_8xG16_AVX2_OpenMP", x, meta, ri, out, M, N, K)
            assert np.max(np.abs(out.astype(np.float64) - y.astype(np.float64))) <= 1e-5 * np.max(np.abs(ref))
        # and the same arrays through the library's reader of that format
        pg = PackedWeight.from_cpu_format(2, 16, 0, meta, ri, N, K)
        assert np.array_equal(pg.matmul_host(np.ascontiguousarray(Xi.T), col_major=True, y_col_major=True), Yi)
        pg.close()
    pw.check()
    pw.close()


@pytest.mark.parametrize("M", [1, 8, 32])
def test_c3_fused_mlp_block_full_size(M):
    """4096 -> 11008 -> 4096, 60 % zeros, fp16, per-tensor scales in U(0.01, 0.05): every row against the fp64 oracle
    (h rounded to fp16 where the block rounds it), tolerance 1e-3 + one fp16 rounding of the output."""
    rng = np.random.default_rng(33)
    hidden, inter = 4096, 11008
    wg, wu, wd = (random_ternary(rng, *s, 0.6) for s in ((hidden, inter), (hidden, inter), (inter, hidden)))
    sg, su, sd = (float(np.float16(v)) for v in rng.uniform(0.01, 0.05, 3))
    mlp = PackedMLP(wg, wu, wd, sg, su, sd)
    X = torch.tensor(rng.standard_normal((M, hidden)), dtype=torch.float16, device=dev())
    Y = mlp.forward(X)
    ref = oracle.mlp_f64(X.double().cpu().numpy(), wg, wu, wd, sg, su, sd, h_round=1)
    err = np.max(np.abs(Y.double().cpu().numpy() - ref)) / np.max(np.abs(ref))
    assert err <= 1e-3 + 2.0 ** -10, err
    mlp.close()


@pytest.mark.parametrize("N,name", [(15360, "QKV"), (5120, "O")])
def test_c4_prefill_projections_full_size(N, name):
    """X [2048, 5120] bf16 against W [5120, N], 50 % zeros: bit-exact on integer activations against a dense fp64
    product on the device, within 1e-3 (+ one bf16 rounding) on N(0,1)."""
    rng = np.random.default_rng(44 + N)
    K, M = 5120, 2048
    w = random_ternary(rng, K, N, 0.5)
    pw = PackedWeight.from_dense(w, scale=1.0)
    Wd = torch.tensor(w, device=dev()).double()
    Xi = torch.tensor(rng.integers(-3, 4, size=(M, K)), dtype=torch.bfloat16, device=dev())
    Y = pw.matmul(Xi, out=torch.empty((M, N), dtype=torch.float32, device=dev()))
    assert torch.equal(Y.double(), Xi.double() @ Wd)
    X = torch.tensor(rng.standard_normal((M, K)), dtype=torch.bfloat16, device=dev())
    Y = pw.matmul(X)
    ref = X.double() @ Wd
    err = float((Y.double() - ref).abs().max() / ref.abs().max())
    assert err <= 1e-3 + 2.0 ** -8, err
    pw.check()
    pw.close()


def test_non_finite_activations_on_the_three_kernels():
    """What each kernel does with an Inf in the activations.  The gather kernel adds only the rows a column refers to:
    columns that do not touch the row stay finite, the others become +-Inf (or NaN where +Inf and -Inf meet).  The
    tensor-core kernels multiply every entry, zeros included, and 0 * Inf is NaN: no column of that activation row stays
    finite (NaN where the column does not use the row, Inf or NaN where it does).  Either way a non-finite input is
    visible in the output; rows without one are unaffected."""
    rng = np.random.default_rng(8)
    K, N = 1024, 256
    w = random_ternary(rng, K, N, 0.75)
    w[5, :] = 0
    w[5, :64] = 1                                     # row 5 is used by the first 64 columns only
    pw = PackedWeight.from_dense(w, scale=1.0)
    L = _lib.lib()
    X = torch.randn((9, K), device=dev()).half()
    X[0, 5] = float("inf")
    for nib, mma, tensor in ((0, 0, False), (64, -1, True), (0, 8, True)):
        prev = L.tllm_set_nibble_max_rows(nib), L.tllm_set_mma_min_rows(mma)
        Y = pw.matmul(X, out=torch.empty((9, N), dtype=torch.float32, device=dev()))
        L.tllm_set_nibble_max_rows(prev[0]), L.tllm_set_mma_min_rows(prev[1])
        assert torch.isfinite(Y[1:]).all()
        if tensor:
            assert not torch.isfinite(Y[0]).any() and torch.isnan(Y[0, 64:]).all()
        else:
            assert torch.isinf(Y[0, :64]).all() and torch.isfinite(Y[0, 64:]).all()
    pw.close()
