"""The tensor-core (tcgen05) product against the oracle, through the C ABI.

From a configurable number of activation rows on, fp16 / bf16 products run on the dense two-bit copy of W with
tcgen05.mma instead of the gather kernel.  The reference has no counterpart (its kernels gather for every M,
ternaryLLM_GPU/csrc/ter_spmm_kernel.cuh:106-308), so the pin is the oracle's dense fp64 product: bit-exact on
integer-valued activations (every product and every partial sum is an integer below 2^24, so the order of the
sums cannot matter), and within 1e-3 of the largest output on N(0,1) activations.
"""
import numpy as np
import pytest
import torch

import oracle
from conftest import random_ternary
from ternaryllm_b200 import PackedMLP, PackedWeight, _lib

pytestmark = pytest.mark.gpu
DT = {"f16": torch.float16, "bf16": torch.bfloat16}
TOL = 1e-3


def dev():
    return torch.device("cuda", 0)


@pytest.fixture(autouse=True)
def tensor_kernel_from_eight_rows():
    """A fixed crossover, so that which kernel runs does not depend on the cost model (tested on its own below)."""
    L = _lib.lib()
    prev = L.tllm_set_mma_min_rows(8)
    yield
    L.tllm_set_mma_min_rows(prev)


def mma_launches():
    return _lib.lib().tllm_mma_launch_count()


SHAPES = [(64, 128, 0.5), (128, 256, 0.5), (1000, 70, 0.6), (4096, 1024, 0.75), (2056, 386, 0.5), (8192, 512, 0.9), (512, 4096, 0.5)]
ROWS = [8, 16, 17, 33, 64, 65, 130, 256, 300, 700]


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("K,N,s", SHAPES)
def test_exact_on_integer_activations(K, N, s, dtype):
    rng = np.random.default_rng(K + N)
    w = random_ternary(rng, K, N, s)
    pw = PackedWeight.from_dense(w, scale=1.0)
    assert pw.info["bit_tile_bytes"] == ((N + 127) // 128) * ((K + 63) // 64) * 2048
    for M in (ROWS if K * N <= 2 ** 20 else (8, 40, 129, 300)):
        xs = rng.integers(-4, 5, size=(M, K)).astype(np.float64)
        X = torch.tensor(xs, dtype=DT[dtype], device=dev())
        Y = torch.full((M, N), float("nan"), dtype=torch.float32, device=dev())
        n0 = mma_launches()
        pw.matmul(X, out=Y)
        assert mma_launches() == n0 + 1, "the call did not run on the tensor-core kernel"
        want = oracle.dense_f64(xs, w, 1.0)
        assert np.array_equal(Y.double().cpu().numpy(), want), (K, N, M)
    pw.check()
    pw.close()


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_tolerance_on_gaussian_activations_and_agreement_with_the_gather_kernel(dtype):
    rng = np.random.default_rng(11)
    K, N = 4096, 2816
    w = random_ternary(rng, K, N, 0.6)
    s = float(np.float16(0.0371))
    pw = PackedWeight.from_dense(w, scale=s)
    L = _lib.lib()
    for M in (8, 16, 48, 100, 512):
        X = torch.tensor(rng.standard_normal((M, K)), dtype=DT[dtype], device=dev())
        ref = oracle.dense_f64(X.double().cpu().numpy(), w, s)
        n0 = mma_launches()
        Y = pw.matmul(X)
        assert mma_launches() == n0 + 1
        eps = {"f16": 2.0 ** -11, "bf16": 2.0 ** -8}[dtype]
        err = np.max(np.abs(Y.double().cpu().numpy() - ref)) / np.max(np.abs(ref))
        assert err <= TOL + eps, (M, err)
        # the gather kernel on the same handle, same inputs: both are within rounding of the fp64 product
        L.tllm_set_mma_min_rows(0)
        Yg = pw.matmul(X)
        L.tllm_set_mma_min_rows(8)
        assert mma_launches() == n0 + 1
        assert np.max(np.abs(Yg.double().cpu().numpy() - Y.double().cpu().numpy())) / np.max(np.abs(ref)) <= 2 * eps + 1e-5
    pw.check()
    pw.close()


def test_repeated_calls_and_row_counts_share_the_split_scratch():
    """Back-to-back launches with different row counts on one handle (programmatic dependent launch lets the
    next kernel start before the previous one has drained): counters and partial sums must not leak."""
    rng = np.random.default_rng(12)
    K, N = 8192, 1024                      # 8 column tiles over all SMs: every tile is shared by many blocks
    w = random_ternary(rng, K, N, 0.5)
    pw = PackedWeight.from_dense(w)
    outs = []
    for rep in range(3):
        for M in (64, 8, 33, 16):
            xs = rng.integers(-3, 4, size=(M, K)).astype(np.float64)
            X = torch.tensor(xs, dtype=torch.bfloat16, device=dev())
            Y = torch.empty((M, N), dtype=torch.float32, device=dev())
            pw.matmul(X, out=Y)
            outs.append((xs, Y))
    torch.cuda.synchronize()
    for xs, Y in outs:
        assert np.array_equal(Y.double().cpu().numpy(), oracle.dense_f64(xs, w, 1.0))
    pw.check()
    pw.close()


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_fused_mlp_on_the_tensor_path(dtype):
    rng = np.random.default_rng(13)
    hidden, inter = 1024, 2752
    wg, wu = random_ternary(rng, hidden, inter, 0.6), random_ternary(rng, hidden, inter, 0.6)
    wd = random_ternary(rng, inter, hidden, 0.6)
    sg, su, sd = (float(np.float16(v)) for v in rng.uniform(0.01, 0.05, 3))
    mlp = PackedMLP(wg, wu, wd, sg, su, sd)
    mode = {"f16": 1, "bf16": 2}[dtype]
    for M in (8, 32, 200):
        X = torch.tensor(rng.standard_normal((M, hidden)), dtype=DT[dtype], device=dev())
        ref = oracle.mlp_f64(X.double().cpu().numpy(), wg, wu, wd, sg, su, sd, h_round=mode)
        n0 = mma_launches()
        Y = mlp.forward(X).double().cpu().numpy()
        assert mma_launches() == n0 + 2
        eps = {"f16": 2.0 ** -11, "bf16": 2.0 ** -8}[dtype]
        err = np.max(np.abs(Y - ref)) / np.max(np.abs(ref))
        assert err <= TOL + 4 * eps, (M, err)
    mlp.close()


def test_crossover_setting_and_fallbacks():
    L = _lib.lib()
    rng = np.random.default_rng(14)
    K, N = 1024, 256
    w = random_ternary(rng, K, N, 0.5)
    pw = PackedWeight.from_dense(w)
    X = torch.tensor(rng.integers(-4, 5, size=(32, K)).astype(np.float32), device=dev())
    n0 = mma_launches()
    pw.matmul(X)                                            # fp32 activations stay on the gather kernel
    pw.matmul(X.to(torch.float16)[:4].contiguous())         # below the crossover
    assert mma_launches() == n0
    prev = L.tllm_set_mma_min_rows(2)
    assert prev == 8
    pw.matmul(X.to(torch.float16)[:4].contiguous())
    assert mma_launches() == n0 + 1
    assert L.tllm_set_mma_min_rows(8) == 2
    narrow = PackedWeight.from_dense(random_ternary(rng, 40, 256, 0.5))     # fewer rows of W than one TMA box: gather kernel
    Xn = torch.tensor(rng.integers(-4, 5, size=(32, 40)).astype(np.float32), dtype=torch.float16, device=dev())
    L.tllm_set_mma_min_rows(2)
    narrow.matmul(Xn)
    L.tllm_set_mma_min_rows(8)
    assert mma_launches() == n0 + 1
    narrow.close()
    lean = PackedWeight.from_dense(w, no_bit_tiles=1)       # no dense copy: always the gather kernel
    assert lean.info["bit_tile_bytes"] == 0
    Y = lean.matmul(X.to(torch.float16))
    assert mma_launches() == n0 + 1
    assert np.array_equal(Y.double().cpu().numpy(), oracle.dense_f64(X.double().cpu().numpy(), w, 1.0))
    pw.close()
    lean.close()


def test_cost_model_dispatch():
    """Default setting: one row always gathers; many rows of a matrix dense enough go to the tensor cores; a
    90 %-sparse matrix keeps a few rows on the gather kernel (its index lists are shorter than the dense copy)."""
    L = _lib.lib()
    L.tllm_set_mma_min_rows(-1)
    rng = np.random.default_rng(15)
    K, N = 4096, 2816
    for s, rows_gather, rows_tensor in ((0.5, (1,), (8, 64, 300)), (0.9, (1, 2, 4), (64, 300))):
        w = random_ternary(rng, K, N, s)
        pw = PackedWeight.from_dense(w)
        for M in rows_gather + rows_tensor:
            X = torch.tensor(rng.integers(-4, 5, size=(M, K)).astype(np.float32), dtype=torch.bfloat16, device=dev())
            Y = torch.empty((M, N), dtype=torch.float32, device=dev())
            n0 = mma_launches()
            pw.matmul(X, out=Y)
            assert (mma_launches() - n0 == 1) == (M in rows_tensor), (s, M)
            assert np.array_equal(Y.double().cpu().numpy(), oracle.dense_f64(X.double().cpu().numpy(), w, 1.0))
        pw.close()
