"""The allocation-free entry point, tllm_spmm_static_scratch, checked against tllm_spmm through the C ABI.

Who needs it: callers that are not allowed to allocate device memory once they are running -- an inference
server whose memory pool was divided up at start-up, code under a framework allocator that must not see a
stray cudaMalloc, a latency-critical loop where an allocation could stall the device.  For them the product
keeps its split-K scratch in a fixed array inside the library instead of in memory the handle obtained from
cudaMalloc.  The test runs both entry points on the same device buffers, twice in a row (the array is
shared between calls and keeps the previous call's contents), and expects the same bits; it also checks
that a request beyond the array's size is refused with a message instead of being run.

This file is collected last on purpose: if it fails, every other test has already run.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from conftest import random_ternary
from ternaryllm_b200 import PackedWeight, _lib

pytestmark = pytest.mark.gpu


def _call(fn, pw, X, Y):
    rc = fn(pw._h, X.data_ptr(), _lib.torch_dtype_code(X.dtype), _lib.ROW_MAJOR, X.shape[0], Y.data_ptr(),
            _lib.torch_dtype_code(Y.dtype), torch.cuda.current_stream().cuda_stream)
    return rc


def test_static_scratch_matches_the_allocating_entry_point_twice_in_a_row():
    assert torch.cuda.is_available()
    dev = torch.device("cuda", 0)
    L = _lib.lib()
    prev = L.tllm_set_mma_min_rows(0)     # compare like with like: tllm_spmm on the gather kernel too
    rng = np.random.default_rng(77)
    K, N = 4096, 3072
    w = random_ternary(rng, K, N, 0.75)
    # four K-tiles of 1024 rows shared by four blocks per column range: the split-K scratch is really used
    pw = PackedWeight.from_dense(w, scale=0.03125, tile_rows=1024, k_splits=4)
    assert pw.info["k_splits"] == 4 and pw.info["max_rows"] == 4
    # 16 rows: more than one launch takes, so the call runs as four launches that share the array
    for call, (M, dtype) in enumerate([(4, torch.float16), (16, torch.float32), (1, torch.bfloat16)]):
        xs = rng.standard_normal((M, K))
        X = torch.tensor(xs, dtype=dtype, device=dev)
        want = torch.empty((M, N), dtype=dtype, device=dev)
        got = torch.full((M, N), float("nan"), dtype=dtype, device=dev)
        assert _call(L.tllm_spmm, pw, X, want) == 0, L.tllm_last_error()
        assert _call(L.tllm_spmm_static_scratch, pw, X, got) == 0, L.tllm_last_error()
        torch.cuda.synchronize()
        # same kernel, same summation order: the two results must be identical, not merely close
        assert torch.equal(got, want), f"call {call}: static-scratch result differs"
        ref = oracle.dense_f64(X.double().cpu().numpy(), w, 0.03125)
        eps = {torch.float32: 2.0 ** -24, torch.float16: 2.0 ** -11, torch.bfloat16: 2.0 ** -8}[dtype]
        err = np.max(np.abs(got.double().cpu().numpy() - ref)) / np.max(np.abs(ref))
        assert err <= 1e-3 + eps          # the tolerance of the other parity tests
    # exact integers, int8 path, straight after the floating-point calls on the same array
    x8 = rng.integers(-128, 128, size=(5, K)).astype(np.int8)
    X8 = torch.tensor(x8, device=dev)
    Y8 = torch.zeros((5, N), dtype=torch.int32, device=dev)
    assert _call(L.tllm_spmm_static_scratch, pw, X8, Y8) == 0, L.tllm_last_error()
    assert np.array_equal(Y8.cpu().numpy().astype(np.int64), oracle.dense_i64(x8, w))
    pw.check()            # the status word this path reports through is the handle's: no wait ran out
    pw.close()
    # more blocks than one wave holds (descriptors past the first 160 come from device memory), two K-splits
    wide = PackedWeight.from_dense(w, scale=1.0, tile_rows=2048, k_splits=2, num_ctas=400)
    assert wide.info["num_ctas"] > 160
    xs = rng.integers(-64, 65, size=(3, K)).astype(np.float64)
    X = torch.tensor(xs, dtype=torch.float32, device=dev)
    got = torch.full((3, N), float("nan"), dtype=torch.float32, device=dev)
    for _ in range(2):
        assert _call(L.tllm_spmm_static_scratch, wide, X, got) == 0, L.tllm_last_error()
    assert np.array_equal(got.double().cpu().numpy(), oracle.dense_f64(xs, w))
    wide.check()
    wide.close()
    L.tllm_set_mma_min_rows(prev)


def test_static_scratch_refuses_what_does_not_fit():
    L = _lib.lib()
    dev = torch.device("cuda", 0)
    K, N = 8192, 8448                     # 32 K-splits x 4 rows per launch x 8448 columns > 1 048 576 partial sums
    w = np.zeros((K, N), np.int8)
    w[::7, ::3] = 1
    pw = PackedWeight.from_dense(w, tile_rows=256, k_splits=32)
    info = pw.info
    assert info["k_splits"] * 4 * N > (1 << 20)
    X = torch.zeros((16, K), dtype=torch.float16, device=dev)
    Y = torch.zeros((16, N), dtype=torch.float16, device=dev)
    rc = _call(L.tllm_spmm_static_scratch, pw, X, Y)
    assert rc == -1 and b"exceed the built-in scratch" in L.tllm_last_error()
    # fewer rows per call fit, and the regular entry point takes the full request
    assert _call(L.tllm_spmm_static_scratch, pw, X[:1], Y[:1]) == 0, L.tllm_last_error()
    assert _call(L.tllm_spmm, pw, X, Y) == 0
    torch.cuda.synchronize()
    pw.close()
