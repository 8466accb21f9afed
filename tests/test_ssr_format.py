"""The library's own sparse-segment image (tllm_ssr_encode / tllm_ssr_decode): round trips, the byte counts the design
notes quote, and the validator.  Host only: the reference names such an encoding (SSR/README.md) but defines none, so
the pins are the round trip and the arithmetic of the layout."""
import ctypes as C
import struct

import numpy as np
import pytest

from conftest import random_ternary
from ternaryllm_b200 import _lib, ssr

HEADER = 24     # magic, inners, columns, group, segment, payload bytes


@pytest.mark.parametrize("K,N,s", [(256, 8, 0.9), (1024, 64, 0.9), (4096, 344, 0.95), (300, 13, 0.5), (1000, 70, 0.98), (33, 5, 0.3),
                                   (1, 1, 0.0), (257, 9, 0.99), (512, 16, 0.0), (2048, 2048, 0.95)])
def test_round_trip(K, N, s):
    rng = np.random.default_rng(K * 31 + N)
    w = random_ternary(rng, K, N, s)
    image = ssr.encode(w)
    assert np.array_equal(ssr.decode(image, K, N), w)
    # 2 + 3n bytes (+ a pad byte when n is odd) per (group of 8 columns, segment of 256 rows), n = rows any of the 8 uses
    groups, segments = -(-N // 8), -(-K // 256)
    want = HEADER + 4 * (groups + 1)
    for g in range(groups):
        used = (w[:, g * 8:(g + 1) * 8] != 0).any(axis=1)
        for sgm in range(segments):
            n = int(used[sgm * 256:(sgm + 1) * 256].sum())
            want += 2 + 3 * n + (n & 1)
    assert image.size == want


def test_all_zero_matrix_and_entries_counted_by_sign():
    z = np.zeros((600, 20), dtype=np.int8)
    image = ssr.encode(z)
    assert image.size == HEADER + 4 * 4 + 2 * 3 * 3            # three groups x three segments of an empty list each
    assert not ssr.decode(image, 600, 20).any()
    w = np.zeros((10, 3), dtype=np.int8)
    w[2, 0], w[9, 2], w[4, 1] = 5, -7, 1
    assert np.array_equal(ssr.decode(ssr.encode(w), 10, 3), np.sign(w))


@pytest.mark.parametrize("zeros", [0.9, 0.95, 0.98])
def test_bytes_per_entry_match_the_formula(zeros):
    """256 (1 - zeros^8) listed rows per segment: 0.215 / 0.127 / 0.057 bytes per entry at 90 / 95 / 98 % zeros."""
    K, N = 4096, 1024
    rng = np.random.default_rng(int(zeros * 100))
    w = random_ternary(rng, K, N, zeros)
    per_entry = (ssr.encode(w).size - HEADER - 4 * (N // 8 + 1)) / (K * N)
    assert abs(per_entry - ssr.expected_bytes_per_entry(zeros)) <= 0.03 * per_entry
    assert abs(ssr.expected_bytes_per_entry(zeros) - {0.9: 0.215, 0.95: 0.127, 0.98: 0.057}[zeros]) < 1e-3
    assert per_entry < 0.25                                     # the two-bit tiles, which it beats from 90 % zeros on


def test_where_the_image_is_smaller_than_the_index_stream():
    """Against the bank stream the gather kernel reads (a byte per non-zero plus bank padding and block tables, all
    counted) on a quarter of the Llama-7B up-projection: larger at 90 % zeros, smaller from about 97 % on; smaller than
    the reference layout (2 bytes per non-zero + 16 per column and 512 rows) at all of them."""
    K, N = 4096, 2752
    sizes = {}
    for zeros in (0.9, 0.98):
        rng = np.random.default_rng(int(zeros * 100))
        w = random_ternary(rng, K, N, zeros)
        out = np.empty_like(w)
        info = _lib.WeightInfo()
        o = _lib.PackOpts(0, 0, 0, 0, 0)
        assert _lib.lib().tllm_pack_roundtrip(_lib.np_ptr(w), K, N, C.byref(o), 37, _lib.np_ptr(out), C.byref(info)) == 0
        sizes[zeros] = (ssr.encode(w).size, info.stream_bytes + info.meta_bytes, info.algorithmic_bytes)
    image, stream, reference = sizes[0.9]
    assert stream < image < reference
    image, stream, reference = sizes[0.98]
    assert image < 0.85 * stream and image < reference


def _image():
    rng = np.random.default_rng(5)
    w = random_ternary(rng, 600, 20, 0.9)
    return w, ssr.encode(w)


def _first_block_with_rows(image, groups):
    """Byte position of the first (group 0) segment list that holds at least two rows."""
    at = HEADER + 4 * (groups + 1)
    while True:
        n = struct.unpack_from("<H", image, at)[0]
        if n >= 2:
            return at, n
        at += 2 + 3 * n + (n & 1)


def test_decode_refuses_damaged_images():
    w, image = _image()
    K, N = w.shape
    groups = 3

    def refused(img, k=K, n=N):
        with pytest.raises(RuntimeError):
            ssr.decode(img, k, n)

    refused(image[:10])                                         # shorter than a header
    refused(image[:-1])                                         # size does not match the header
    refused(np.concatenate([image, np.zeros(2, np.uint8)]))
    refused(image, K + 1, N)                                    # another shape than the image's
    refused(image, K, N + 8)
    bad = image.copy(); bad[0] ^= 1; refused(bad)               # magic
    bad = image.copy(); struct.pack_into("<I", bad, HEADER + 4, 3); refused(bad)        # group 1 starts inside group 0's lists
    bad = image.copy(); struct.pack_into("<I", bad, HEADER, 2); refused(bad)            # first offset not 0
    at, n = _first_block_with_rows(image, groups)
    bad = image.copy(); struct.pack_into("<H", bad, at, 300); refused(bad)              # more rows than a segment has
    bad = image.copy(); struct.pack_into("<H", bad, at, n + 1); refused(bad)            # the lists no longer tile the group
    bad = image.copy(); struct.pack_into("<H", bad, at + 2, 0); refused(bad)            # a listed row without an entry
    bad = image.copy(); struct.pack_into("<H", bad, at + 2, 3); refused(bad)            # code 3
    rows_at = at + 2 + 2 * n
    bad = image.copy(); bad[rows_at + 1] = bad[rows_at]; refused(bad)                   # row ids not ascending
    # the last group has 4 columns: a code for a fifth one is refused
    w2 = np.zeros((256, 12), dtype=np.int8); w2[7, 9] = 1
    img2 = ssr.encode(w2)
    second = HEADER + 4 * 3 + 2                                 # group 0: one empty list; group 1: n = 1
    assert struct.unpack_from("<H", img2, second)[0] == 1
    bad = img2.copy(); struct.pack_into("<H", bad, second + 2, 1 << (2 * 5)); refused(bad, 256, 12)
    assert np.array_equal(ssr.decode(img2, 256, 12), w2)        # the undamaged images still decode
    assert np.array_equal(ssr.decode(image, K, N), w)


def test_encode_reports_the_size_first_and_refuses_a_short_buffer():
    w, image = _image()
    K, N = w.shape
    n = C.c_size_t(0)
    L = _lib.lib()
    assert L.tllm_ssr_encode(_lib.np_ptr(w), K, N, None, 0, C.byref(n)) == 0 and n.value == image.size
    short = np.empty(image.size - 1, dtype=np.uint8)
    assert L.tllm_ssr_encode(_lib.np_ptr(w), K, N, _lib.np_ptr(short), short.size, C.byref(n)) != 0
    assert L.tllm_ssr_encode(None, K, N, None, 0, C.byref(n)) != 0
    assert L.tllm_ssr_encode(_lib.np_ptr(w), 0, N, None, 0, C.byref(n)) != 0


def test_handle_creation_refuses_a_damaged_image_before_touching_the_device():
    w, image = _image()
    K, N = w.shape
    h = C.c_void_p()
    o = _lib.PackOpts(0, 0, 0, 0, 0)
    rc = _lib.lib().tllm_weight_create_ssr(_lib.np_ptr(image[:-1].copy()), image.size - 1, K, N, 1.0, C.byref(o), C.byref(h))
    assert rc == -1 and not h.value                             # TLLM_ERR_ARG from the validator, no CUDA call made
    assert b"tllm_ssr_decode" in _lib.lib().tllm_last_error()


@pytest.mark.gpu
def test_handle_from_an_image_multiplies_like_the_handle_from_the_matrix():
    import torch

    import oracle
    from ternaryllm_b200 import PackedWeight

    rng = np.random.default_rng(11)
    K, N = 1500, 200
    w = random_ternary(rng, K, N, 0.97)
    a = PackedWeight.from_ssr(ssr.encode(w), K, N, scale=0.5)
    b = PackedWeight.from_dense(w, scale=0.5)
    assert a.info["nnz"] == b.info["nnz"] == int((w != 0).sum())
    xs = rng.integers(-64, 65, size=(3, K)).astype(np.float64)
    X = torch.tensor(xs, dtype=torch.float32, device=torch.device("cuda", 0))
    Ya, Yb = a.matmul(X), b.matmul(X)
    assert torch.equal(Ya, Yb)
    assert np.array_equal(Ya.double().cpu().numpy(), oracle.dense_f64(xs, w, 0.5))
    a.close()
    b.close()
