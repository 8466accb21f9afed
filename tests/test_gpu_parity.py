"""Parity of the CUDA path with the oracle -- every call goes through the C ABI (ctypes on libtllm.so).

Bars: bit-exact wherever the arithmetic is exact (integer-valued fp32 / fp16 / bf16 activations as in the
reference's own verify_* functions, main.cpp:1403; int8 activations with int32 accumulation); for N(0,1)
activations  max|Y - Y_ref| <= 1e-3 * max|Y_ref|  with Y_ref the fp64 product of the activations as stored
(the tolerance the task states for fp16/bf16 after reordering sums; fp32 accumulation lands near 1e-6).
"""
import numpy as np
import pytest
import torch

import oracle
from conftest import random_ternary
from ternaryllm_b200 import PackedMLP, PackedWeight, TernaryLinear, _lib, ter_spmm

pytestmark = pytest.mark.gpu

TOL = 1e-3
DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def dev():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    return torch.device("cuda", 0)


@pytest.fixture(autouse=True)
def gather_kernel_only():
    """Everything in this file pins the gather kernel: the tensor-core kernel (tests in test_gpu_tensor_path.py)
    is switched off for the duration of each test."""
    L = _lib.lib()
    prev = L.tllm_set_mma_min_rows(0)
    yield
    L.tllm_set_mma_min_rows(prev)


def int_acts(rng, M, K, lim, dtype):
    x = rng.integers(-lim, lim + 1, size=(M, K)).astype(np.float64)
    return x, torch.tensor(x, dtype=dtype, device=dev())


def rel_err(y, ref):
    return float(np.max(np.abs(y - ref)) / max(1e-30, np.max(np.abs(ref))))


# ------------------------------------------------------------------------------------------------------
# ter_spmm on the reference's arrays (golden fixtures from the reference's Python packer)
# ------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("case", ["a", "b", "c", "d"])
@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
def test_ter_spmm_on_golden_arrays(gpu_packers, case, dtype):
    c = gpu_packers[case]
    K, N = c["w"].shape
    T = int(c["T"])
    rng = np.random.default_rng(11)
    ri = torch.tensor(c["mcsc_idx"].astype(np.int16), device=dev())
    co = torch.tensor(c["mcsc_off"], device=dev())
    til = torch.zeros(1, dtype=torch.int16, device=dev())
    for B, M in ((1, 1), (2, 5), (3, 8)):
        xs = rng.integers(-8, 9, size=(B, M, K)).astype(np.float64)
        X = torch.tensor(xs, dtype=DT[dtype], device=dev())
        Y = ter_spmm.ter_spmm(X, ri, co, til, B, M, N, K, False, False, tile_k=T)
        assert Y.shape == (B, M, N) and Y.dtype == DT[dtype]
        for b in range(B):
            want = oracle.mcsc_product_f64(xs[b], c["mcsc_idx"], c["mcsc_off"], N, K, T)
            assert np.array_equal(Y[b].double().cpu().numpy(), want)
            assert np.array_equal(want, oracle.dense_f64(xs[b], c["w"]))
        # the layout the reference kernel indexes: [K][M] per batch item
        Xt = X.transpose(1, 2).contiguous()
        if M != K:
            Yt = ter_spmm.ter_spmm(Xt, ri, co, til, B, M, N, K, False, False, tile_k=T)
            assert torch.equal(Yt, Y)
    # scale and out=
    out = torch.empty((1, 2, N), dtype=torch.float32, device=dev())
    xs = rng.integers(-8, 9, size=(1, 2, K)).astype(np.float64)
    ter_spmm.ter_spmm(torch.tensor(xs, dtype=torch.float32, device=dev()), ri, co, til, 1, 2, N, K, False, False, scale=0.5, out=out, tile_k=T)
    assert np.array_equal(out[0].double().cpu().numpy(), oracle.dense_f64(xs[0], c["w"], 0.5))


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
def test_ter_spmm_after_prepare_runs_the_packed_kernels(gpu_packers, dtype):
    """tllm_ter_spmm_prepare repacks the reference's device arrays once; the same ter_spmm call then gives the same
    values from the packed kernels (launch counters show which ran), for both activation layouts, and `forget` puts the
    call back on the arrays as they are."""
    L = _lib.lib()
    rng = np.random.default_rng(21)
    for case in ("a", "b", "c", "d", "e", "f"):
        c = gpu_packers[case]
        K, N = c["w"].shape
        T = int(c["T"])
        idx, off = (c["mcsc_idx"], c["mcsc_off"]) if "mcsc_idx" in c else oracle.ter_tiled_mcsc(c["w"].astype(np.int32), T)[:2]
        ri = torch.tensor(np.asarray(idx).astype(np.int16), device=dev())
        co = torch.tensor(np.asarray(off).astype(np.int32), device=dev())
        til = torch.zeros(1, dtype=torch.int16, device=dev())
        B, M = 2, 3
        xs = rng.integers(-8, 9, size=(B, M, K)).astype(np.float64)
        X = torch.tensor(xs, dtype=DT[dtype], device=dev())
        before = ter_spmm.ter_spmm(X, ri, co, til, B, M, N, K, False, False, scale=0.25, tile_k=T)
        ter_spmm.prepare(ri, co, N, K, tile_k=T)
        ter_spmm.prepare(ri, co, N, K, tile_k=T)                  # a second call finds the copy
        prev = L.tllm_set_nibble_max_rows(0), L.tllm_set_mma_min_rows(0)
        n0 = L.tllm_launch_count()
        after = ter_spmm.ter_spmm(X, ri, co, til, B, M, N, K, False, False, scale=0.25, tile_k=T)
        assert L.tllm_launch_count() - n0 == 2                    # six rows: two gather launches of up to four rows, not one per-column launch
        L.tllm_set_mma_min_rows(-1), L.tllm_set_nibble_max_rows(64)
        d0 = L.tllm_nibble_launch_count()
        tensor = ter_spmm.ter_spmm(X, ri, co, til, B, M, N, K, False, False, scale=0.25, tile_k=T)
        assert L.tllm_nibble_launch_count() > d0
        L.tllm_set_nibble_max_rows(prev[0]), L.tllm_set_mma_min_rows(prev[1])
        Xt = X.transpose(1, 2).contiguous()
        turned = ter_spmm.ter_spmm(Xt, ri, co, til, B, M, N, K, False, False, scale=0.25, tile_k=T) if M != K else after
        want = np.stack([oracle.dense_f64(xs[b], c["w"], 0.25) for b in range(B)])
        for y in (before, after, tensor, turned):
            assert np.array_equal(y.double().cpu().numpy(), want), case
        assert ter_spmm.forget(ri, co) == 1 and ter_spmm.forget(ri, co) == 0
        n0 = L.tllm_launch_count()
        ter_spmm.ter_spmm(X, ri, co, til, B, M, N, K, False, False, scale=0.25, tile_k=T)
        assert L.tllm_launch_count() - n0 == 1


def test_ter_spmm_error_behaviour(gpu_packers):
    c = gpu_packers["a"]
    K, N = c["w"].shape
    ri = torch.tensor(c["mcsc_idx"].astype(np.int16), device=dev())
    co = torch.tensor(c["mcsc_off"], device=dev())
    X = torch.zeros((1, 2, K), device=dev())
    with pytest.raises(RuntimeError):
        ter_spmm.ter_spmm(X.cpu(), ri, co, ri, 1, 2, N, K, False, False, tile_k=16)          # X not on CUDA
    with pytest.raises(RuntimeError):
        ter_spmm.ter_spmm(X, ri.int(), co, ri, 1, 2, N, K, False, False, tile_k=16)          # wrong index dtype
    with pytest.raises(RuntimeError):
        ter_spmm.ter_spmm(X, ri, co, ri, 1, 2, N, K, False, False, tile_k=32)                # offsets do not match TILE_K
    # batch 0: nothing is launched and an empty [0, M, N] tensor comes back, as in the reference
    Y0 = ter_spmm.ter_spmm(X[:0], ri, co, ri, 0, 2, N, K, False, False, tile_k=16)
    assert Y0.shape == (0, 2, N)


def test_ter_spmm_int8(gpu_packers):
    c = gpu_packers["b"]
    K, N = c["w"].shape
    T = int(c["T"])
    rng = np.random.default_rng(2)
    x8 = rng.integers(-128, 128, size=(1, 7, K)).astype(np.int8)
    ri = torch.tensor(c["mcsc_idx"].astype(np.int16), device=dev())
    co = torch.tensor(c["mcsc_off"], device=dev())
    Y = ter_spmm.ter_spmm(torch.tensor(x8, device=dev()), ri, co, ri, 1, 7, N, K, False, False, tile_k=T)
    assert Y.dtype == torch.int32
    assert np.array_equal(Y[0].cpu().numpy().astype(np.int64), oracle.dense_i64(x8[0], c["w"]))


# ------------------------------------------------------------------------------------------------------
# gather kernel on the bank-stream format
# ------------------------------------------------------------------------------------------------------
SHAPES = [
    # K, N, sparsity, pack options
    (64, 8, 0.5, {}),
    (1000, 70, 0.75, {}),
    (2048, 256, 0.5, {}),
    (1536, 130, 0.9, {}),
    (4096, 344, 0.75, {}),
    (3000, 2, 0.5, {}),
    (700, 40, 0.7, {"tile_rows": 256}),                   # three tiles resident at once (one row), one at a time (four rows)
    (700, 40, 0.7, {"tile_rows": 64, "k_splits": 1}),     # eleven tiles in one block: several table refills
    (700, 40, 0.7, {"tile_rows": 64, "k_splits": 4}),     # the same through the split-K hand-over
    (700, 40, 0.0, {"num_ctas": 3}),                      # dense
    (2500, 64, 0.6, {"num_ctas": 2, "tile_rows": 512}),
    (5000, 24, 0.8, {"num_ctas": 1}),                     # one block, two tiles
    (9000, 36, 0.8, {}),                                  # three tiles, K-split chosen by the packer
    (4096, 200, 0.97, {"num_ctas": 1}),                   # one warp walks many columns: ring wrap-around and reduce points
    (128, 16, 1.0, {}),                                   # all-zero weight
    (999, 77, 0.6, {}),                                   # K not a multiple of 16 (no vector loads of X), odd N
]


@pytest.mark.parametrize("K,N,s,opts", SHAPES)
def test_gather_bit_exact_on_integer_activations(K, N, s, opts):
    rng = np.random.default_rng(K * 31 + N)
    w = random_ternary(rng, K, N, s)
    if N > 12:
        w[:, 3] = 0
        w[:, 9] = 1
        w[:, 10] = -1
    pw = PackedWeight.from_dense(w, scale=1.0, **opts)
    for M in (1, 2, 3, 4, 5, 8, 13, 16, 17, 40):
        xs, X = int_acts(rng, M, K, 512, torch.float32)      # |sum| < 2^24: exact in fp32, as in main.cpp:1403
        want = oracle.dense_f64(xs, w)
        Y = pw.matmul(X)
        assert np.array_equal(Y.double().cpu().numpy(), want), (M,)
        if M in (1, 4, 16):
            Yc = pw.matmul(X.t().contiguous(), col_major=True)
            assert torch.equal(Yc, Y)
    for dtype, lim in (("f16", 1), ("bf16", 1)):
        # +-1/0 activations keep every sum exactly representable in the narrow output type for small K
        xs, X = int_acts(rng, 4, K, lim, DT[dtype])
        want = oracle.round_to(oracle.dense_f64(xs, w), 1 if dtype == "f16" else 2)
        assert np.array_equal(pw.matmul(X).double().cpu().numpy(), want)
    x8 = rng.integers(-128, 128, size=(6, K)).astype(np.int8)
    Y8 = pw.matmul(torch.tensor(x8, device=dev()))
    assert Y8.dtype == torch.int32 and np.array_equal(Y8.cpu().numpy().astype(np.int64), oracle.dense_i64(x8, w))
    pw.check()
    pw.close()


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("M", [1, 4, 16])
def test_gather_tolerance_on_gaussian_activations(dtype, M):
    rng = np.random.default_rng(M)
    K, N, s = 4096, 688, 0.75
    w = random_ternary(rng, K, N, s)
    scale = float(np.float16(rng.uniform(0.01, 0.05)))
    pw = PackedWeight.from_dense(w, scale=scale)
    X = torch.tensor(rng.standard_normal((M, K)), dtype=DT[dtype], device=dev())
    ref = oracle.dense_f64(X.double().cpu().numpy(), w, scale)          # activations as stored
    Y = pw.matmul(X).double().cpu().numpy()
    # the result is rounded once to the output dtype: allow that rounding on top of the stated tolerance
    eps = {"f32": 2.0 ** -24, "f16": 2.0 ** -11, "bf16": 2.0 ** -8}[dtype]
    assert rel_err(Y, ref) <= TOL * (1.0 if dtype == "f32" else 1.0) + eps
    if dtype == "f32":
        assert rel_err(Y, ref) < 1e-5
    pw.close()


def test_repeated_calls_and_scale_update():
    rng = np.random.default_rng(3)
    K, N = 2048, 512
    w = random_ternary(rng, K, N, 0.6)
    pw = PackedWeight.from_dense(w, scale=2.0)
    xs, X = int_acts(rng, 4, K, 16, torch.float32)
    want = oracle.dense_f64(xs, w, 2.0)
    for _ in range(20):     # back to back on one stream: split-K counters must return to zero every time
        Y = pw.matmul(X)
    assert np.array_equal(Y.double().cpu().numpy(), want)
    pw.set_scale(0.25)
    assert np.array_equal(pw.matmul(X).double().cpu().numpy(), oracle.dense_f64(xs, w, 0.25))
    info = pw.info
    assert info["nnz"] == int((w != 0).sum()) and info["scratch_bytes"] > 0
    pw.check()


def test_host_buffer_entry_point():
    rng = np.random.default_rng(4)
    K, N = 1024, 96
    w = random_ternary(rng, K, N, 0.5)
    pw = PackedWeight.from_dense(w)
    x = rng.integers(-512, 513, size=(8, K)).astype(np.float32)
    want = oracle.dense_f64(x, w)
    assert np.array_equal(pw.matmul_host(x).astype(np.float64), want)
    # the col-major CPU kernels' convention: X [K][M] in, Y [N][M] out (GEMM_CPU_FP32.cpp:509-538)
    yt = pw.matmul_host(np.ascontiguousarray(x.T), col_major=True, y_col_major=True)
    assert np.array_equal(yt.T.astype(np.float64), want)
    x8 = rng.integers(-10, 11, size=(64, K)).astype(np.int8)
    y32 = pw.matmul_host(x8)
    assert np.array_equal(y32.astype(np.int64), oracle.dense_i64(x8, w))
    # the reference's int8 kernels wrap modulo 256 (GEMM_CPU_INT8.cpp:33-40): truncating the int32 result gives the same bytes
    assert np.array_equal(y32.astype(np.int8), oracle.int8_wrap(x8, w))


# ------------------------------------------------------------------------------------------------------
# reference CPU formats in, reference CPU kernels' results out (golden fixture from the compiled reference)
# ------------------------------------------------------------------------------------------------------
def test_cpu_formats_reproduce_reference_kernel_outputs(cpu_reference):
    import re

    fx = cpu_reference
    K, N = fx["W"].shape
    X = np.ascontiguousarray(fx["X"])                       # [M][K] integer-valued fp32
    XT = np.ascontiguousarray(X.T)
    seen = {}
    for name, fmt in zip(fx["kernel_names"], fx["kernel_formats"]):
        if fmt in seen:
            continue
        if fmt == "merged":
            pw = PackedWeight.from_cpu_format(1, 1, 0, fx["merged_meta"], fx["merged_ri"], N, K)
            wname = "W"
        elif fmt == "naive":
            meta = np.concatenate([fx["sf_csn"], fx["sf_csp"]])
            ri = np.concatenate([fx["sf_rin"], fx["sf_rip"]])
            pw = PackedWeight.from_cpu_format(0, 1, 0, meta, ri, N, K, aux=len(fx["sf_rin"]))
            wname = "W"
        else:
            m = re.match(r"grp\.(\w+)\.G(\d+)\.(\w+)\.i(\d)\.s(\d+)", fmt)
            wname, G, method, inter, simd = m.group(1), int(m.group(2)), m.group(3), int(m.group(4)), int(m.group(5))
            kind = {"min": 2, "mid": 3, "max": 4, "uniform": 5}[method]
            chunk = 0 if inter else (simd if simd else G)
            ri = fx[fmt + ".ri"]
            if "GEMV" in name or "rowMajor" in name:
                ri = ri.astype(np.int32)                     # the gather kernels take int32 ids (main.cpp:1446-1449)
            pw = PackedWeight.from_cpu_format(kind, G, chunk, fx[fmt + ".meta"], ri, N, K)
        seen[fmt] = True
        want_col = fx[f"direct_col.{wname}"]                 # [N][M], what every reference kernel reproduced
        got = pw.matmul_host(XT, col_major=True, y_col_major=True)
        assert np.array_equal(got, want_col), (name, fmt)
        pw.close()
    assert len(seen) >= 20
    # int8 family
    for wname in ("W", "Wun"):
        key = f"int8_col.{wname}"
        if key in fx.files:
            pw = PackedWeight.from_dense(fx[wname])
            y = pw.matmul_host(np.ascontiguousarray(fx["X8"].T), col_major=True, y_col_major=True)
            assert np.array_equal(y.astype(np.int8), fx[key])


# ------------------------------------------------------------------------------------------------------
# modules
# ------------------------------------------------------------------------------------------------------
def test_ternary_linear_module():
    g = torch.Generator().manual_seed(0)
    lin = TernaryLinear(512, 96, sparsity=0.7, bias=False, scale=0.5, generator=g)
    w = lin.ternary_weight.numpy()
    assert lin.w_row_indices.dtype == torch.int16 and lin.w_col_offsets.dtype == torch.int32
    rng = np.random.default_rng(0)
    xs = rng.integers(-16, 17, size=(2, 5, 512)).astype(np.float64)
    X = torch.tensor(xs, dtype=torch.float32, device=dev())
    Y = lin(X)
    assert Y.shape == (2, 5, 96)
    for b in range(2):
        assert np.array_equal(Y[b].double().cpu().numpy(), oracle.dense_f64(xs[b], w, 0.5))
    assert torch.equal(lin(X.transpose(1, 2).contiguous()), Y)          # (batch, K, rows) form
    assert torch.equal(lin(X[0]), Y[0])                                  # 2-D input
    # the reference-layout buffers feed ter_spmm and give the same numbers (scale passed explicitly)
    lin = lin.to(dev())
    Y2 = ter_spmm.ter_spmm(X, lin.w_row_indices, lin.w_col_offsets, lin.w_col_tile_indices, 2, 5, 96, 512, False, False, scale=0.5)
    assert torch.equal(Y2, Y)
    with pytest.raises(RuntimeError):
        lin(X.cpu())
    # uniform weights: balanced +1 / -1 in every 512-block of a column
    lu = TernaryLinear(1024, 32, sparsity=0.75, uniform=True, bias=False, generator=g)
    wu = lu.ternary_weight.numpy()
    assert np.all((wu[:512] == 1).sum(0) == (wu[:512] == -1).sum(0)) and abs((wu == 0).mean() - 0.75) < 1e-3


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
def test_fused_mlp(dtype):
    rng = np.random.default_rng(9)
    hidden, inter = 1024, 2752
    wg, wu = random_ternary(rng, hidden, inter, 0.6), random_ternary(rng, hidden, inter, 0.6)
    wd = random_ternary(rng, inter, hidden, 0.6)
    sg, su, sd = (float(np.float16(v)) for v in rng.uniform(0.01, 0.05, 3))
    mlp = PackedMLP(wg, wu, wd, sg, su, sd)
    mode = {"f32": 3, "f16": 1, "bf16": 2}[dtype]
    for M in (1, 8, 32):
        X = torch.tensor(rng.standard_normal((M, hidden)), dtype=DT[dtype], device=dev())
        ref = oracle.mlp_f64(X.double().cpu().numpy(), wg, wu, wd, sg, su, sd, h_round=mode)
        Y = mlp.forward(X).double().cpu().numpy()
        eps = {"f32": 2.0 ** -24, "f16": 2.0 ** -11, "bf16": 2.0 ** -8}[dtype]
        # h is rounded to the activation dtype between the two products, exactly like the oracle does
        assert rel_err(Y, ref) <= TOL + 4 * eps, (M, rel_err(Y, ref))
    # exact check of the epilogue alone on values where SiLU is benign: x = 0 -> h = 0 -> y = 0
    Z = torch.zeros((3, hidden), dtype=DT[dtype], device=dev())
    assert not mlp.forward(Z).any()
    mlp.close()


def test_wide_matrix_runs_as_several_waves_of_blocks():
    """8192 x 57344 (the fused gate|up width of a 70B-class MLP) packed for 400 thread blocks: more blocks than one
    wave holds, and the blocks past the first 160 read their descriptors from device memory.  Exact on integer
    activations, against a dense product on the device."""
    from ternaryllm_b200.synthetic import make_weight

    K, N = 8192, 57344
    w = make_weight(3, K, N, 0.875)
    pw = PackedWeight.from_dense(w, scale=1.0, num_ctas=400)
    info = pw.info
    assert info["num_ctas"] > 160 and info["num_ctas"] == info["col_blocks"] * info["k_splits"] and info["tiles"] == 2
    rng = np.random.default_rng(3)
    Wd = torch.tensor(w, device=dev()).float()
    for M in (1, 5, 16):
        xs, X = int_acts(rng, M, K, 8, torch.float32)
        Y = pw.matmul(X)
        want = X @ Wd                                      # integer sums far below 2^24: the fp32 GEMM is exact
        want64 = oracle.dense_f64(xs[:1].astype(np.float64), w, 1.0) if M == 1 else None
        assert torch.equal(Y, want)
        if want64 is not None:
            assert np.array_equal(Y.double().cpu().numpy(), want64)
    pw.check()
    pw.close()


# ------------------------------------------------------------------------------------------------------
# full benchmark size: size-independent properties + a dense fp64 product on the device
# ------------------------------------------------------------------------------------------------------
def test_full_size_llama7b_up_projection():
    rng = np.random.default_rng(0)
    K, N = 4096, 11008
    r = rng.integers(0, 256, size=(K, N), dtype=np.uint8)
    w = np.zeros((K, N), np.int8)
    w[(r >= 192) & (r < 224)] = -1
    w[r >= 224] = 1                                        # 75 % zeros, +-1 equiprobable
    pw = PackedWeight.from_dense(w, scale=1.0)
    Wd = torch.tensor(w, device=dev()).double()
    for M in (1, 4, 16):
        xs, X = int_acts(rng, M, K, 64, torch.float32)
        Y = pw.matmul(X)
        assert torch.equal(Y.double(), X.double() @ Wd)                  # exact: integer sums below 2^24
        # linearity: (a+b) W = aW + bW  (exact on integers)
        xs2, X2 = int_acts(rng, M, K, 64, torch.float32)
        assert torch.equal(pw.matmul(X + X2), Y + pw.matmul(X2))
    Xg = torch.tensor(rng.standard_normal((1, K)), dtype=torch.float16, device=dev())
    Yg = pw.matmul(Xg).double()
    ref = Xg.double() @ Wd
    assert float((Yg - ref).abs().max() / ref.abs().max()) <= TOL + 2.0 ** -11
    pw.check()


def test_packed_weight_file_round_trip(tmp_path):
    """tllm_weight_save / tllm_weight_load: the loaded handle reports the same layout and gives the same bits as
    the one that was saved, on both kernels; a damaged file is refused with a message."""
    rng = np.random.default_rng(31)
    K, N = 3000, 1100
    w = random_ternary(rng, K, N, 0.7)
    pw = PackedWeight.from_dense(w, scale=0.0625)
    path = tmp_path / "w.tllm"
    pw.save(path)
    pl = PackedWeight.load(path)
    assert pl.info == pw.info
    xs, X = int_acts(rng, 5, K, 16, torch.float32)
    assert torch.equal(pl.matmul(X), pw.matmul(X))
    assert np.array_equal(pl.matmul(X).double().cpu().numpy(), oracle.dense_f64(xs, w, 0.0625))
    L = _lib.lib()
    L.tllm_set_mma_min_rows(8)
    xs, Xh = int_acts(rng, 40, K, 4, torch.float16)
    Y = torch.empty((40, N), dtype=torch.float32, device=dev())
    m0 = L.tllm_mma_launch_count()
    pl.matmul(Xh, out=Y)
    assert L.tllm_mma_launch_count() == m0 + 1
    assert np.array_equal(Y.double().cpu().numpy(), oracle.dense_f64(xs, w, 0.0625))
    L.tllm_set_mma_min_rows(0)
    raw = path.read_bytes()
    bad = tmp_path / "bad.tllm"
    bad.write_bytes(raw[: len(raw) // 2])
    with pytest.raises(RuntimeError, match="not a packed-weight file|truncated"):
        PackedWeight.load(bad)
    pw.close()
    pl.close()


def test_linear_from_float_weights():
    """TernaryLinear.from_float: ternarise an nn.Linear weight (threshold rule), keep the per-tensor scale, and get
    scale * x @ sign-pattern -- checked against the oracle's restatement of the rule and its dense product."""
    g = torch.Generator().manual_seed(5)
    lin = torch.nn.Linear(768, 320, bias=False)
    with torch.no_grad():
        lin.weight.copy_(torch.randn(lin.weight.shape, generator=g) * 0.02)
    tl = TernaryLinear.from_float(lin.weight, sparsity=0.6, bias=False, reference_buffers=False)
    t_ref, s_ref = oracle.ternarize_f64(lin.weight.detach().t().contiguous().numpy(), sparsity=0.6)
    assert np.array_equal(tl.ternary_weight.numpy(), t_ref.astype(np.int32)) and abs(tl.scale - s_ref) <= 1e-6 * s_ref
    x = torch.randn((7, 768), generator=g)
    y = tl(x.to(dev())).double().cpu().numpy()
    ref = oracle.dense_f64(x.double().numpy(), t_ref, tl.scale)
    assert rel_err(y, ref) <= TOL
    # the ternarised layer approximates the float layer (sanity of the scale): correlation of the outputs is high
    yf = (x @ lin.weight.detach().t()).double().numpy()
    assert np.corrcoef(y.ravel(), yf.ravel())[0, 1] > 0.8
