"""The decode tensor-core product (four-bit planes of W streamed by TMA into tcgen05.mma.kind::f8f6f4) against the
oracle, through the C ABI.

The reference gathers for every M (ternaryLLM_GPU/csrc/ter_spmm_kernel.cuh:24-78, :106-308); this kernel multiplies
instead, with the activations split into exact e5m2 pieces, so the pin is the oracle's dense fp64 product: bit-exact on
integer-valued activations (every product and every partial sum is an integer below 2^24), within 1e-3 of the largest
output on N(0,1) activations (the tolerance the task states for fp16 / bf16 after reordering sums), and within rounding
of what the gather kernel gives on the same handle.
"""
import numpy as np
import pytest
import torch

import oracle
from conftest import random_ternary
from ternaryllm_b200 import PackedMLP, PackedWeight, _lib

pytestmark = pytest.mark.gpu
DT = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}
TOL = 1e-3


def dev():
    return torch.device("cuda", 0)


@pytest.fixture(autouse=True)
def nibble_kernel_for_every_small_call():
    """Pins the choice, so that which kernel runs does not depend on the cost model (tested on its own below)."""
    L = _lib.lib()
    prev = L.tllm_set_nibble_max_rows(128)
    yield
    L.tllm_set_nibble_max_rows(prev)


def launches():
    return _lib.lib().tllm_nibble_launch_count()


def expected_launches(M, dtype):
    """up to four rows (two for fp32): one launch of the small kernel; above that the many-row kernel, 64 (32) rows per launch"""
    small, big = (2, 32) if dtype == "f32" else (4, 64)
    return 1 if M <= small else -(-M // big)


# K not a multiple of 128, N not a multiple of 128, one and several K ranges (4096 rows each), one K block
SHAPES = [(64, 128, 0.5), (128, 256, 0.5), (1000, 70, 0.6), (4096, 1024, 0.75), (2056, 386, 0.5), (8192, 512, 0.9), (512, 4096, 0.5),
          (12800, 260, 0.5), (77, 5, 0.3), (4224, 128, 0.0)]


@pytest.mark.parametrize("dtype", ["f16", "bf16", "f32"])
@pytest.mark.parametrize("K,N,s", SHAPES)
def test_exact_on_integer_activations(K, N, s, dtype):
    rng = np.random.default_rng(K + N)
    w = random_ternary(rng, K, N, s)
    pw = PackedWeight.from_dense(w, scale=1.0)
    assert pw.info["nibble_bytes"] == ((N + 127) // 128 * 128) * ((K + 127) // 128 * 128) // 2
    top = {"f16": 512, "bf16": 127, "f32": 100000}[dtype]          # exactly representable magnitudes of each type
    for M in (1, 2, 3, 4, 5, 9, 16, 33, 64, 70):
        xs = rng.integers(-top, top + 1, size=(M, K)).astype(np.float64)
        if dtype == "f32" and K * top * 4 > 2 ** 24:
            xs = np.round(xs / 64)                                  # keep every partial sum below 2^24
        X = torch.tensor(xs, dtype=DT[dtype], device=dev())
        Y = torch.full((M, N), float("nan"), dtype=torch.float32, device=dev())
        n0 = launches()
        pw.matmul(X, out=Y)
        assert launches() == n0 + expected_launches(M, dtype), "the call did not run on the decode tensor-core kernel"
        want = oracle.dense_f64(xs, w, 1.0)
        assert np.array_equal(Y.double().cpu().numpy(), want), (K, N, M)
    pw.check()
    pw.close()


@pytest.mark.parametrize("dtype", ["f16", "bf16", "f32"])
def test_tolerance_on_gaussian_activations_and_agreement_with_the_gather_kernel(dtype):
    rng = np.random.default_rng(11)
    K, N = 4096, 2816
    w = random_ternary(rng, K, N, 0.6)
    s = float(np.float16(0.0371))
    pw = PackedWeight.from_dense(w, scale=s)
    L = _lib.lib()
    for M in (1, 2, 4, 7, 16, 40, 64):
        X = torch.tensor(rng.standard_normal((M, K)), dtype=DT[dtype], device=dev())
        ref = oracle.dense_f64(X.double().cpu().numpy(), w, s)
        n0 = launches()
        Y = pw.matmul(X, out=torch.empty((M, N), dtype=torch.float32, device=dev()))
        assert launches() > n0
        err = np.max(np.abs(Y.double().cpu().numpy() - ref)) / np.max(np.abs(ref))
        assert err <= 1e-5, (M, err)                               # fp32 sums of exact products: far inside the 1e-3 allowed
        prev = L.tllm_set_nibble_max_rows(0)
        Yg = pw.matmul(X, out=torch.empty((M, N), dtype=torch.float32, device=dev()))
        L.tllm_set_nibble_max_rows(prev)
        assert float((Y - Yg).abs().max()) <= 1e-5 * float(Yg.abs().max())
        # results in the activation type carry that type's rounding and nothing more
        Yt = pw.matmul(X)
        eps = {"f16": 2.0 ** -11, "bf16": 2.0 ** -8, "f32": 2.0 ** -23}[dtype]
        err = np.max(np.abs(Yt.double().cpu().numpy() - ref)) / np.max(np.abs(ref))
        assert err <= TOL * 0.01 + eps, (M, err)
    pw.check()
    pw.close()


def test_wide_range_of_magnitudes_in_one_row():
    """The scaling is per row and per K range: a row whose entries span thirty binary orders of magnitude keeps the
    small ones as far as an fp32 sum could."""
    rng = np.random.default_rng(5)
    K, N = 8192, 256
    w = random_ternary(rng, K, N, 0.5)
    pw = PackedWeight.from_dense(w, scale=1.0)
    x = rng.standard_normal((2, K))
    x[0, :4096] *= 2.0 ** -20          # a K range of tiny values next to one of ordinary ones
    x[1, ::7] *= 2.0 ** 12
    for dtype in ("bf16", "f32"):
        X = torch.tensor(x, dtype=DT[dtype], device=dev())
        ref = oracle.dense_f64(X.double().cpu().numpy(), w, 1.0)
        Y = pw.matmul(X, out=torch.empty((2, N), dtype=torch.float32, device=dev()))
        err = np.max(np.abs(Y.double().cpu().numpy() - ref), axis=1) / np.max(np.abs(ref), axis=1)
        assert np.all(err <= 1e-5), err
        # the tiny half on its own: its relative accuracy does not suffer from sharing a row with the other half
        X0 = X.clone()
        X0[:, 4096:] = 0
        ref0 = oracle.dense_f64(X0.double().cpu().numpy(), w, 1.0)
        Y0 = pw.matmul(X0, out=torch.empty((2, N), dtype=torch.float32, device=dev()))
        err0 = np.max(np.abs(Y0[0].double().cpu().numpy() - ref0[0])) / np.max(np.abs(ref0[0]))
        assert err0 <= 1e-5, err0
    pw.check()
    pw.close()


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("M", [1, 3, 6, 16, 64])
def test_fused_mlp_block_on_the_decode_tensor_core_kernel(dtype, M):
    rng = np.random.default_rng(3)
    hidden, inter = 1024, 2816
    wg, wu, wd = (random_ternary(rng, *shape, 0.6) for shape in ((hidden, inter), (hidden, inter), (inter, hidden)))
    sg, su, sd = 0.021, 0.034, 0.027
    mlp = PackedMLP(wg, wu, wd, sg, su, sd)
    X = torch.tensor(rng.standard_normal((M, hidden)), dtype=DT[dtype], device=dev())
    n0 = launches()
    Y = mlp.forward(X)
    assert launches() == n0 + 2, "gate/up and down did not both run on the decode tensor-core kernel"
    ref = oracle.mlp_f64(X.double().cpu().numpy(), wg, wu, wd, sg, su, sd, h_round={"f16": 1, "bf16": 2}[dtype])
    err = np.max(np.abs(Y.double().cpu().numpy() - ref)) / np.max(np.abs(ref))
    assert err <= TOL + {"f16": 2.0 ** -10, "bf16": 2.0 ** -7}[dtype], err
    mlp.close()


def test_cost_model_sends_large_dense_weights_to_this_kernel_and_small_sparse_ones_to_the_gather_kernel():
    L = _lib.lib()
    prev = L.tllm_set_nibble_max_rows(-1)
    try:
        rng = np.random.default_rng(9)
        big = PackedWeight.from_dense(random_ternary(rng, 8192, 8192, 0.5), scale=1.0, no_bit_tiles=1)
        small = PackedWeight.from_dense(random_ternary(rng, 2048, 2048, 0.9), scale=1.0, no_bit_tiles=1)
        for pw, K, expect in ((big, 8192, 1), (small, 2048, 0)):
            X = torch.randn((1, K), dtype=torch.float16, device=dev())
            n0 = launches()
            pw.matmul(X)
            assert launches() - n0 == expect
            pw.close()
    finally:
        L.tllm_set_nibble_max_rows(prev)


def test_handle_without_the_four_bit_copy_gathers():
    rng = np.random.default_rng(2)
    w = random_ternary(rng, 512, 256, 0.5)
    pw = PackedWeight.from_dense(w, scale=1.0, no_nibbles=1)
    assert pw.info["nibble_bytes"] == 0
    X = torch.randn((1, 512), dtype=torch.float16, device=dev())
    n0 = launches()
    Y = pw.matmul(X, out=torch.empty((1, 256), dtype=torch.float32, device=dev()))
    assert launches() == n0
    ref = oracle.dense_f64(X.double().cpu().numpy(), w, 1.0)
    assert np.max(np.abs(Y.double().cpu().numpy() - ref)) <= 1e-5 * np.max(np.abs(ref))
    pw.close()
