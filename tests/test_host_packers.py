"""Host-side logic of the library, no GPU needed: the C ABI loads and exports every declared symbol, the
three reference packers behind it reproduce the reference (golden fixtures + the C oracle), and the
tile-stream packer round-trips and keeps the invariants its kernel relies on."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import oracle
from conftest import ROOT, random_ternary
from ternaryllm_b200 import _lib, ter_spmm


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "tllm.h")).read()
    declared = set(re.findall(r"\b(tllm_[a-z0-9_]+)\s*\(", header))
    declared -= {"tllm_weight", "tllm_mlp"}
    assert len(declared) >= 20
    L = _lib.lib()
    for name in sorted(declared):
        assert hasattr(L, name), f"{name} is declared in include/tllm.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert L.tllm_version() >= 100
    assert L.tllm_launch_count() == 0 or L.tllm_launch_count() > 0


@pytest.mark.parametrize("case", ["a", "b", "c", "d"])
def test_packers_match_reference_python(gpu_packers, case):
    c = gpu_packers[case]
    w = c["w"].astype(np.int32)
    K, N = w.shape
    T = int(c["T"])
    pos, neg = int((w == 1).sum()), int((w == -1).sum())
    cp, cn = C.c_int64(), C.c_int64()
    _lib.check(_lib.lib().tllm_count_nnz(_lib.np_ptr(w), N, K, C.byref(cp), C.byref(cn)))
    assert (cp.value, cn.value) == (pos, neg)
    ni, no, pi, po = ter_spmm.convert_to_ter_csc(w, N, K, pos, neg, as_numpy=True)
    assert np.array_equal(ni, c["csc_neg_idx"]) and np.array_equal(no, c["csc_neg_off"])
    assert np.array_equal(pi, c["csc_pos_idx"]) and np.array_equal(po, c["csc_pos_off"])
    tni, tno, tpi, tpo = ter_spmm.convert_to_ter_tiled_csc(w, N, K, pos, neg, T, as_numpy=True)
    assert np.array_equal(tni, c["tcsc_neg_idx"]) and np.array_equal(tno, c["tcsc_neg_off"])
    assert np.array_equal(tpi, c["tcsc_pos_idx"]) and np.array_equal(tpo, c["tcsc_pos_off"])
    mi, mo, mt = ter_spmm.convert_to_ter_tiled_mcsc(w, N, K, pos, neg, T, False, 4, as_numpy=True)
    assert np.array_equal(mi, c["mcsc_idx"]) and np.array_equal(mo, c["mcsc_off"])
    # python-list return shape of the reference binding (std::vector<std::vector<int32_t>>)
    as_lists = ter_spmm.convert_to_ter_tiled_mcsc(w, N, K, pos, neg, T, False, 4)
    assert isinstance(as_lists, list) and isinstance(as_lists[0], list) and as_lists[0] == mi.tolist()
    # tile order: non-decreasing list length per column
    tiles = -(-K // T)
    o = mo.reshape(N, tiles, 4)
    lens = (o[:, :, 2] - o[:, :, 0])
    order = mt.reshape(N, tiles)
    assert np.all(np.diff(np.take_along_axis(lens, order, 1), axis=1) >= 0)


@pytest.mark.parametrize("K,N,T,s,pad", [(512, 16, 256, 0.5, False), (512, 16, 256, 0.5, True), (300, 12, 64, 0.8, True),
                                         (128, 8, 32, 0.0, False), (64, 8, 64, 1.0, False)])
def test_mcsc_modes_against_oracle(K, N, T, s, pad):
    rng = np.random.default_rng(K + N)
    w = random_ternary(rng, K, N, s, np.int32)
    pos, neg = int((w == 1).sum()), int((w == -1).sum())
    X = rng.integers(-9, 10, size=(3, K)).astype(np.float64)
    want = X @ w.astype(np.float64)
    # lossless mode (with and without padding) always encodes W
    idx, off, _ = ter_spmm.convert_to_ter_tiled_mcsc(w, N, K, pos, neg, T, pad, 8, as_numpy=True)
    assert np.array_equal(oracle.mcsc_product_f64(X, idx, off, N, K, T), want)
    if pad:
        o = off.reshape(-1, 4)
        assert np.all((o[:, 1] - o[:, 0]) % 8 == 0)
    # compat mode equals the restatement of the reference's C++ packer, entry for entry
    for padsz in (4, 8):
        cidx, coff, _ = ter_spmm.convert_to_ter_tiled_mcsc(w, N, K, pos, neg, T, pad, padsz, compat=True, as_numpy=True)
        oidx, ooff, _ = oracle.ter_tiled_mcsc(w, T, padding=pad, padding_size=padsz, lossy=True)
        assert np.array_equal(coff, ooff)
        n = min(len(cidx), len(oidx))
        assert len(cidx) == len(oidx) and np.array_equal(cidx[:n], oidx[:n])


@pytest.mark.parametrize("case", ["a", "b", "c", "d", "e", "f"])
def test_packers_against_the_reference_cpp_packers(gpu_packers, case):
    """The arrays the reference's own C++ packers returned for the fixture matrices (the host side of
    ternaryLLM_GPU/csrc/ter_spmm_wrapper.cu, compiled where it lies and called by tests/golden/make_golden.py):
    convert_to_ter_csc and convert_to_ter_tiled_csc entry for entry, and convert_to_ter_tiled_mcsc in its truncating
    form (mode 1) entry for entry -- offsets, tile order, and every row id a list still refers to -- without padding
    and with padding to 4 and to 8.  The C restatement in oracle/ is held to the same arrays."""
    c = gpu_packers[case]
    w = c["w"].astype(np.int32)
    K, N = w.shape
    T = int(c["T"])
    pos, neg = int((w == 1).sum()), int((w == -1).sum())
    ni, no, pi, po = ter_spmm.convert_to_ter_csc(w, N, K, pos, neg, as_numpy=True)
    for got, key in ((ni, "cpp_csc_neg_idx"), (no, "cpp_csc_neg_off"), (pi, "cpp_csc_pos_idx"), (po, "cpp_csc_pos_off")):
        assert np.array_equal(got, c[key]), key
    ni, no, pi, po = ter_spmm.convert_to_ter_tiled_csc(w, N, K, pos, neg, T, as_numpy=True)
    for got, key in ((ni, "cpp_tcsc_neg_idx"), (no, "cpp_tcsc_neg_off"), (pi, "cpp_tcsc_pos_idx"), (po, "cpp_tcsc_pos_off")):
        assert np.array_equal(got, c[key]), key
    for tag, pad, padsz in (("nopad", False, 4), ("pad4", True, 4), ("pad8", True, 8)):
        want_idx, want_off, want_til = c[f"cpp_mcsc_{tag}_idx"], c[f"cpp_mcsc_{tag}_off"], c[f"cpp_mcsc_{tag}_til"]
        for name, (idx, off, til) in (("library", ter_spmm.convert_to_ter_tiled_mcsc(w, N, K, pos, neg, T, pad, padsz, compat=True, as_numpy=True)),
                                      ("oracle", oracle.ter_tiled_mcsc(w, T, padding=pad, padding_size=padsz, lossy=True))):
            assert np.array_equal(off, want_off), (name, tag)
            assert np.array_equal(til, want_til), (name, tag)
            # every entry a list refers to; what lies between the truncated lists is whatever the next tile wrote
            o = want_off.reshape(-1, 4)
            for s0, s1 in zip(o[:, 0], o[:, 2]):
                assert np.array_equal(idx[s0:s1], want_idx[s0:s1]), (name, tag)


def _roundtrip(w, **opts):
    w = np.ascontiguousarray(w, np.int8)
    K, N = w.shape
    out = np.full_like(w, 7)
    info = _lib.WeightInfo()
    o = _lib.PackOpts(opts.get("tile_rows", 0), opts.get("num_ctas", 0), opts.get("reserved0", 0), 0, opts.get("k_splits", 0))
    rc = _lib.lib().tllm_pack_roundtrip(_lib.np_ptr(w), K, N, C.byref(o), opts.get("num_sms", 148), _lib.np_ptr(out), C.byref(info))
    return rc, out, info.as_dict()


@pytest.mark.parametrize("K,N,s", [(64, 8, 0.5), (1000, 70, 0.75), (2048, 256, 0.5), (4096, 344, 0.75), (1536, 130, 0.9),
                                   (11008 // 4, 96, 0.6), (33, 5, 0.3), (8, 2, 0.0), (3000, 2, 0.5), (9000, 37, 0.6)])
def test_bank_stream_roundtrip(K, N, s):
    rng = np.random.default_rng(K * 7 + N)
    w = random_ternary(rng, K, N, s)
    rc, out, info = _roundtrip(w)
    assert rc == 0, _lib.lib().tllm_last_error()
    assert np.array_equal(out, w)
    assert info["nnz"] == int((w != 0).sum())
    assert info["num_ctas"] <= 2 * 148 and info["num_ctas"] == info["col_blocks"] * info["k_splits"]
    assert info["tiles"] == -(-K // 4096)


def test_bank_stream_storage_at_benchmark_density():
    """A quarter of the Llama-7B up-projection columns packed for a quarter of the SMs has the per-block structure
    of the full matrix: one byte per non-zero plus padding to whole words, the flag bytes and the tables stay below
    0.6 of the reference layout's bytes (2 bytes per non-zero + 16 per column and 512-row tile)."""
    rng = np.random.default_rng(0)
    K, N = 4096, 2752
    r = rng.integers(0, 256, size=(K, N), dtype=np.uint8)
    w = np.zeros((K, N), np.int8)
    w[(r >= 192) & (r < 224)] = -1
    w[r >= 224] = 1
    rc, out, info = _roundtrip(w, num_sms=37)
    assert rc == 0 and np.array_equal(out, w)
    assert info["k_splits"] == 1 and info["num_ctas"] == 74 and info["tiles"] == 1      # two blocks per SM
    assert info["stream_bytes"] + info["meta_bytes"] <= 0.6 * info["algorithmic_bytes"], info
    assert info["meta_bytes"] <= 0.02 * info["stream_bytes"]
    # every warp of every block got one unit: the lanes never drift more than a ring apart on random data
    assert info["units"] == 74 * 8


def test_bank_stream_edge_cases():
    rng = np.random.default_rng(5)
    w = random_ternary(rng, 700, 40, 0.7)
    w[:, 3] = 0                # empty column
    w[256:512, :] = 0          # empty rows spanning a tile boundary
    w[:, 9] = 1                # dense +1 column
    w[:, 10] = -1              # dense -1 column
    for opts in (dict(), dict(tile_rows=256), dict(tile_rows=64), dict(num_ctas=8), dict(num_ctas=1), dict(tile_rows=32),
                 dict(tile_rows=1024), dict(k_splits=1), dict(tile_rows=128, k_splits=2), dict(tile_rows=128, k_splits=100)):
        rc, out, info = _roundtrip(w, **opts)
        assert rc == 0, (opts, _lib.lib().tllm_last_error())
        assert np.array_equal(out, w), opts
    # all-zero matrix
    z = np.zeros((128, 16), np.int8)
    rc, out, info = _roundtrip(z)
    assert rc == 0 and not out.any() and info["nnz"] == 0


def test_bank_stream_lanes_that_drift_apart_end_their_unit_early():
    """All non-zeros of 200 columns in the rows of one lane: that lane's lists are long, the 31 others hold one word
    per list and run far ahead.  The packer has to cut the columns into units short enough for the 16-slot ring."""
    K, N = 4096, 200
    w = np.zeros((K, N), np.int8)
    w[5::32, :] = 1
    w[5::64, ::3] = -1
    rc, out, info = _roundtrip(w, num_ctas=1)
    assert rc == 0, _lib.lib().tllm_last_error()
    assert np.array_equal(out, w)
    assert info["units"] > 8


def test_bank_stream_rejects_bad_options():
    w = np.zeros((64, 8), np.int8)
    assert _roundtrip(w, tile_rows=12)[0] != 0           # not a multiple of 32
    assert _roundtrip(w, tile_rows=8192)[0] != 0         # beyond what a one-byte id covers
    assert _roundtrip(w, num_ctas=100000)[0] != 0
    assert b"" != _lib.lib().tllm_last_error()


def _corrupt(w, what, where, value, **opts):
    w = np.ascontiguousarray(w, np.int8)
    o = _lib.PackOpts(opts.get("tile_rows", 0), opts.get("num_ctas", 0), 0, 0, opts.get("k_splits", 0))
    return _lib.lib().tllm_pack_corrupt_check(_lib.np_ptr(w), w.shape[0], w.shape[1], C.byref(o), 8, what, where, value)


def test_damaged_images_are_refused_on_the_host():
    """What tllm_weight_load checks before it uploads anything: every header field, block descriptor, table word
    class and stream byte class, damaged one at a time, must be refused (and nothing may be read out of range
    while finding out)."""
    rng = np.random.default_rng(9)
    w = random_ternary(rng, 600, 48, 0.6)
    kw = dict(tile_rows=256, k_splits=1)
    assert _corrupt(w, 0, 0, 0, **kw) == 0
    bad = [
        (3, 0, 0), (3, 0, 8192), (3, 0, 100), (3, 0, 512),      # tile_rows: zero, too large, not a multiple of 32, wrong
        (4, 0, 0), (4, 0, 7),                                    # tiles
        (5, 0, 0), (5, 0, 1000),                                 # col_blocks
        (6, 0, 0), (6, 0, 3),                                    # k_splits
        (7, 0, 0), (7, 0, 1),                                    # tiles_per_cta
        (8, 0, 0), (8, 0, 0x7fffffff), (8, 0, 8),                # a block's table words
        (9, 0, 0xfffffff0), (9, 1, 3),                           # a block's first vector: out of range, misaligned
        (12, 0, 0xfffffff0), (13, 0, 0xffffffe0),                # table offset, vector count
        (10, 1, 1), (10, 1, 1000), (10, 0, 2),                   # column ranges
        (11, 0, 100),                                            # inners no longer matches the ids
        (1, 0, 5), (1, 1, 4000), (1, 3, 40), (1, 6, 999),        # block header words
        (1, 8, 3), (1, 9, 100000), (1, 16, 0),                   # warp table
        (1, 17, 0xffffff), (1, 18, 0x00ff0001), (1, 18, 0x00030000), (1, 19, 0x7f), (1, 19, 0xffffff00), (1, 20, 0),
        (1, 21, 0xffffffff), (1, 37, 0xffffffff),                # unit descriptor: offset, columns, tile, reduce points, lengths
    ]
    for what, where, value in bad:
        rc = _corrupt(w, what, where, value, **kw)
        assert rc != 0, (what, where, value)
    # stream bytes: an id beyond the tile, a damaged flag byte, a lost list end
    assert _corrupt(w, 2, 0, 200, **kw) != 0
    assert _corrupt(w, 2, 15, 0xf0, **kw) != 0
    assert _corrupt(w, 2, 15, 0x0f, **kw) != 0 or _corrupt(w, 2, 15, 0x00, **kw) != 0


def test_schedule_for_llama_shapes_uses_most_sms():
    """Shapes of the benchmark configs: one wave, >= 88 % of the SMs busy."""
    for K, N in [(4096, 11008), (11008, 4096), (4096, 22016), (2048, 2048), (5120, 15360), (8192, 10240), (8192, 8192)]:
        big = np.zeros((K, N), np.int8)
        info = _lib.WeightInfo()
        o = _lib.PackOpts(0, 0, 0, 0)
        out = np.empty_like(big)
        rc = _lib.lib().tllm_pack_roundtrip(_lib.np_ptr(big), K, N, C.byref(o), 148, _lib.np_ptr(out), C.byref(info))
        assert rc == 0, _lib.lib().tllm_last_error()
        assert info.num_ctas <= 4 * 148 and info.num_ctas >= 130, (K, N, info.as_dict())


def test_cpu_format_decoders_build_the_same_dense_matrix(cpu_reference):
    """Every reference CPU format decodes (in the product code, not the oracle) to the dense weight: checked
    through tllm_weight_create_cpu_format's error path needing no GPU is not possible, so this test drives the
    oracle's decoder and the product's decoder with the same arrays via the pack round-trip of the decoded
    matrix."""
    fx = cpu_reference
    K, N = fx["W"].shape
    Wd = oracle.cpu_decode_dense(2, 8, 0, fx["grp.W.G8.min.i1.s0.meta"], fx["grp.W.G8.min.i1.s0.ri"], N, K)
    rc, out, _ = _roundtrip(Wd)
    assert rc == 0 and np.array_equal(out, fx["W"])


@pytest.mark.parametrize("mode", [dict(sparsity=0.5), dict(sparsity=0.9), dict(threshold_factor=0.7), dict(threshold_factor=0.3)])
def test_ternarize_matches_the_numpy_restatement(mode):
    """tllm_ternarize on the host against oracle.ternarize_f64: identical ternary matrix, scale to fp32 rounding;
    the requested sparsity is met exactly on data without ties."""
    from ternaryllm_b200.weight import ternarize

    rng = np.random.default_rng(21)
    w = (rng.standard_normal((300, 130)) * 0.02).astype(np.float32)
    t, s = ternarize(w, **mode)
    tr, sr = oracle.ternarize_f64(w, **mode)
    assert np.array_equal(t, tr)
    assert abs(s - sr) <= 1e-6 * sr
    assert set(np.unique(t)) <= {-1, 0, 1} and np.all(np.sign(w)[t != 0] == t[t != 0])
    if "sparsity" in mode:
        assert (t == 0).sum() == round(mode["sparsity"] * w.size)
    # the scale minimises |w - s*t| over s for the chosen t
    kept = t != 0
    assert abs(s - np.abs(w[kept]).mean()) <= 1e-6 * s
