"""The host-made schedule of the decode tensor-core kernel (tllm_nibble_schedule) against a restatement of what the
kernel's thread blocks do with it: block c of K range j owns the units [total * c / gj, total * (c + 1) / gj) of that
range, tile-major; the last block to arrive at a column tile adds the parts of all blocks the schedule names, reading
slot `tile + c` of range j.  Host only: every shape here is checked without a GPU, the tensor-parallel shards of the
70B-shaped decoder at every degree included."""
import ctypes as C

import numpy as np
import pytest

from ternaryllm_b200 import _lib


def schedule(K, N, sms):
    dims = (C.c_int * 6)()
    L = _lib.lib()
    assert L.tllm_nibble_schedule(K, N, sms, dims, None, 0) == 0
    kb, tiles, kbs, splits, gj, uk = list(dims)
    words = np.zeros((1 + splits) * tiles, dtype=np.uint32)
    assert L.tllm_nibble_schedule(K, N, sms, dims, _lib.np_ptr(words), words.size) == 0
    return kb, tiles, kbs, splits, gj, uk, words


def check(K, N, sms):
    kb, tiles, kbs, splits, gj, uk, words = schedule(K, N, sms)
    assert kb == -(-K // 128) and tiles == -(-N // 128) and uk == 2
    assert 1 <= kbs <= 32 and splits == -(-kb // kbs)            # a range's activation pieces fit the kernel's shared memory
    assert 1 <= gj and (splits * gj <= sms or gj == 1)           # one thread block per SM
    parts = np.zeros(tiles, dtype=np.int64)
    for j in range(splits):
        kbj = min(kbs, kb - j * kbs)
        assert kbj >= 1
        kuj = -(-kbj // uk)
        total = tiles * kuj
        holders = [[] for _ in range(tiles)]
        slots = set()
        for c in range(gj):
            u0, u1 = total * c // gj, total * (c + 1) // gj
            assert u1 > u0, "a thread block without a unit would be counted by nobody"
            for t in range(u0 // kuj, (u1 - 1) // kuj + 1):
                holders[t].append(c)
                slot = t + c                                   # where block c leaves its part of tile t
                assert slot < tiles + gj and slot not in slots
                slots.add(slot)
        for t in range(tiles):
            run = int(words[(1 + j) * tiles + t])
            first, last = run & 0xFFFF, run >> 16
            assert holders[t] == list(range(first, last + 1)), (K, N, sms, j, t)
            parts[t] += len(holders[t])
    assert np.array_equal(parts, words[:tiles].astype(np.int64))


SHAPES = [(4096, 11008), (11008, 4096), (8192, 28672), (28672, 8192), (8192, 10240), (8192, 8192), (2048, 2048), (5120, 15360),
          (128, 128), (77, 5), (1000, 300), (28672, 520), (3584, 8192), (129, 257), (40000, 128), (256, 100000)]


@pytest.mark.parametrize("K,N", SHAPES)
def test_schedule_names_exactly_the_blocks_that_hold_a_part(K, N):
    for sms in (148, 132, 37, 1, 7, 1000):
        check(K, N, sms)


def test_tensor_parallel_shards_of_the_70b_shape():
    hidden, ffn, q, kv = 8192, 28672, 64 * 128, 8 * 128
    for world in (1, 2, 4, 8):
        for K, N in ((hidden, (q + 2 * kv) // world), (q // world, hidden), (hidden, 2 * ffn // world), (ffn // world, hidden)):
            check(K, N, 148)


def test_random_shapes():
    rng = np.random.default_rng(0)
    for _ in range(300):
        K, N = int(rng.integers(1, 40000)), int(rng.integers(1, 6000))
        check(K, N, int(rng.integers(1, 300)))


def test_bad_arguments_are_refused():
    dims = (C.c_int * 6)()
    L = _lib.lib()
    assert L.tllm_nibble_schedule(0, 128, 148, dims, None, 0) != 0
    assert L.tllm_nibble_schedule(128, 128, 0, dims, None, 0) != 0
    assert L.tllm_nibble_schedule(128, 128, 148, None, None, 0) != 0
    words = np.zeros(1, dtype=np.uint32)
    assert L.tllm_nibble_schedule(4096, 11008, 148, dims, _lib.np_ptr(words), 1) != 0
