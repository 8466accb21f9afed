"""Pin the C oracle (oracle/oracle.c) against fixtures produced by the reference itself.

Fixtures: tests/golden/gpu_packers.npz (the reference's Python packers, TernaryCSC.py) and
tests/golden/cpu_reference.npz (the reference's C++ format builders and CPU kernels compiled in place);
both are written by tests/golden/make_golden.py.  Everything here is integer / index work or exact
integer-valued fp32, so every comparison is bit-exact.
"""
import re

import numpy as np
import pytest

import oracle


@pytest.mark.parametrize("case", ["a", "b", "c", "d"])
def test_gpu_packers_match_reference_python(gpu_packers, case):
    c = gpu_packers[case]
    w = c["w"].astype(np.int32)
    T = int(c["T"])
    ni, no, pi, po = oracle.ter_csc(w)
    assert np.array_equal(ni, c["csc_neg_idx"]) and np.array_equal(no, c["csc_neg_off"])
    assert np.array_equal(pi, c["csc_pos_idx"]) and np.array_equal(po, c["csc_pos_off"])
    tni, tno, tpi, tpo = oracle.ter_tiled_csc(w, T)
    assert np.array_equal(tni, c["tcsc_neg_idx"]) and np.array_equal(tno, c["tcsc_neg_off"])
    assert np.array_equal(tpi, c["tcsc_pos_idx"]) and np.array_equal(tpo, c["tcsc_pos_off"])
    mi, mo, _ = oracle.ter_tiled_mcsc(w, T)
    assert np.array_equal(mi, c["mcsc_idx"]) and np.array_equal(mo, c["mcsc_off"])


@pytest.mark.parametrize("case", ["a", "b", "c", "d"])
def test_mcsc_product_equals_dense(gpu_packers, case):
    c = gpu_packers[case]
    w = c["w"]
    K, N = w.shape
    T = int(c["T"])
    rng = np.random.default_rng(1)
    X = rng.integers(-512, 513, size=(5, K)).astype(np.float64)
    want = oracle.dense_f64(X, w, 1.0)
    assert np.array_equal(want, X @ w.astype(np.float64))
    got = oracle.mcsc_product_f64(X, c["mcsc_idx"], c["mcsc_off"], N, K, T)
    assert np.array_equal(got, want)
    got_t = oracle.mcsc_product_f64(np.ascontiguousarray(X.T), c["mcsc_idx"], c["mcsc_off"], N, K, T, x_colmajor=True)
    assert np.array_equal(got_t, want)


def test_lossy_packer_loses_entries_lossless_does_not():
    """The extension's C++ packer truncates list lengths (ter_spmm_wrapper.cu:277-291); the restatement
    reproduces that, and the lossless mode does not lose anything."""
    rng = np.random.default_rng(3)
    K, N, T = 512, 16, 256
    r = rng.random((K, N))
    w = np.zeros((K, N), np.int32)
    w[(r >= 0.5) & (r < 0.75)] = -1
    w[r >= 0.75] = 1
    X = rng.integers(-8, 9, size=(2, K)).astype(np.float64)
    want = X @ w.astype(np.float64)
    idx, off, _ = oracle.ter_tiled_mcsc(w, T)
    assert np.array_equal(oracle.mcsc_product_f64(X, idx, off, N, K, T), want)
    idx2, off2, _ = oracle.ter_tiled_mcsc(w, T, lossy=True)
    o = off2.reshape(-1, 4)
    assert np.all((o[:, 1] - o[:, 0]) % 4 == 0) and np.all((o[:, 2] - o[:, 1]) % 4 == 0)
    assert not np.array_equal(oracle.mcsc_product_f64(X, idx2, off2, N, K, T), want)


def test_cpu_format_builders_match_reference(cpu_reference):
    fx = cpu_reference
    csp, csn, rip, rin = oracle.sparse_format(fx["W"])
    assert np.array_equal(csp, fx["sf_csp"]) and np.array_equal(csn, fx["sf_csn"])
    assert np.array_equal(rip, fx["sf_rip"]) and np.array_equal(rin, fx["sf_rin"])
    meta, ri = oracle.merged_tcsc(fx["W"])
    assert np.array_equal(meta, fx["merged_meta"]) and np.array_equal(ri, fx["merged_ri"])
    n = 0
    for key in fx.files:
        m = re.match(r"grp\.(\w+)\.G(\d+)\.(\w+)\.i(\d)\.s(\d+)\.meta", key)
        if not m:
            continue
        wname, G, method, inter, simd = m.group(1), int(m.group(2)), m.group(3), int(m.group(4)), int(m.group(5))
        meta, ri = oracle.merged_group(fx[wname], G, method, bool(inter), simd)
        base = key[: -len(".meta")]
        assert np.array_equal(meta, fx[key]), key
        assert np.array_equal(ri, fx[base + ".ri"]), key
        n += 1
    assert n > 50


def _decode_args(fmt):
    """fixture format key -> (kind, G, chunk) for oracle.cpu_decode_dense"""
    m = re.match(r"grp\.(\w+)\.G(\d+)\.(\w+)\.i(\d)\.s(\d+)", fmt)
    wname, G, method, inter, simd = m.group(1), int(m.group(2)), m.group(3), int(m.group(4)), int(m.group(5))
    kind = {"min": 2, "mid": 3, "max": 4, "uniform": 5}[method]
    chunk = 0 if inter else (simd if simd else G)
    return wname, kind, G, chunk


def test_decode_semantics_match_every_reference_kernel(cpu_reference):
    """For each reference kernel that reproduced its Direct product on the fixture, decoding the arrays it
    was given the way oracle.c says that kernel family reads them must give back the dense weight."""
    fx = cpu_reference
    K, N = fx["W"].shape
    names, fmts = list(fx["kernel_names"]), list(fx["kernel_formats"])
    assert len(names) >= 100
    seen = set()
    for name, fmt in zip(names, fmts):
        if fmt in seen:
            continue
        seen.add(fmt)
        if fmt == "merged":
            Wd = oracle.cpu_decode_dense(1, 1, 0, fx["merged_meta"], fx["merged_ri"], N, K)
            assert np.array_equal(Wd, fx["W"])
        elif fmt == "naive":
            meta = np.concatenate([fx["sf_csn"], fx["sf_csp"]])
            ri = np.concatenate([fx["sf_rin"], fx["sf_rip"]])
            Wd = oracle.cpu_decode_dense(0, 1, 0, meta, ri, N, K, aux=len(fx["sf_rin"]))
            assert np.array_equal(Wd, fx["W"])
        else:
            wname, kind, G, chunk = _decode_args(fmt)
            Wd = oracle.cpu_decode_dense(kind, G, chunk, fx[fmt + ".meta"], fx[fmt + ".ri"], N, K)
            assert np.array_equal(Wd, fx[wname]), (name, fmt)
            Wd32 = oracle.cpu_decode_dense(kind, G, chunk, fx[fmt + ".meta"], fx[fmt + ".ri"].astype(np.int32), N, K)
            assert np.array_equal(Wd32, fx[wname])


def test_dense_oracle_matches_reference_direct_kernels(cpu_reference):
    fx = cpu_reference
    X = fx["X"].astype(np.float64)
    for wname in ("W", "Wal", "Wun"):
        want = fx[f"direct_col.{wname}"].T.astype(np.float64)     # reference result is [N][M]
        assert np.array_equal(oracle.dense_f64(X, fx[wname], 1.0), want)
    for wname in ("W", "Wun"):
        key = f"int8_col.{wname}"
        if key in fx.files:
            assert np.array_equal(oracle.int8_wrap(fx["X8"], fx[wname]), fx[key].T)
            wide = oracle.dense_i64(fx["X8"], fx[wname])
            assert np.array_equal(wide.astype(np.int8), fx[key].T)     # truncation commutes with the sum


def test_scale_and_rounding_helpers():
    rng = np.random.default_rng(0)
    X = rng.standard_normal((3, 64))
    W = rng.integers(-1, 2, size=(64, 8)).astype(np.int8)
    assert np.allclose(oracle.dense_f64(X, W, 0.03), (X @ W) * 0.03, rtol=0, atol=1e-12)
    v = rng.standard_normal(200) * 10
    import torch

    t = torch.tensor(v, dtype=torch.float64)
    assert np.array_equal(oracle.round_to(v, 1), t.to(torch.float16).double().numpy())
    assert np.array_equal(oracle.round_to(v, 2), t.to(torch.bfloat16).double().numpy())
    assert np.array_equal(oracle.round_to(v, 3), t.to(torch.float32).double().numpy())
    a = rng.standard_normal(50).astype(np.float32)
    b = rng.standard_normal(50).astype(np.float32)
    want = (a.astype(np.float64) * b / (1 + np.exp(-a.astype(np.float64))))
    assert np.allclose(oracle.silu_mul_f32(a, b), want, rtol=1e-6, atol=1e-6)


@pytest.mark.skipif(oracle.ref() is None, reason="compiled reference (oracle/_ref) not present on this host")
def test_live_reference_agrees_with_fixture(cpu_reference):
    """When the compiled reference is available, rebuild two formats live and compare with the fixture."""
    fx = cpu_reference
    meta, ri = oracle.ref_merged_tcsc(fx["W"])
    assert np.array_equal(meta, fx["merged_meta"]) and np.array_equal(ri, fx["merged_ri"])
    meta, ri = oracle.ref_merged_group(fx["W"], 8, "min", True, 0)
    assert np.array_equal(meta, fx["grp.W.G8.min.i1.s0.meta"]) and np.array_equal(ri, fx["grp.W.G8.min.i1.s0.ri"])
