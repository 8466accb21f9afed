"""Tensor-parallel partitioning.

CPU (gloo, two ranks): column shards concatenate to the full product, row shards all-reduce to it -- the packed GPU
product is replaced by the oracle's dense product there -- and the blocked weight generator gives every
tensor-parallel degree the same model.
GPU (one device): the decoder layer against the same layer in dense fp32 PyTorch, with both reduction paths; the
peer all-reduce kernel against a stand-in peer whose slot and flag the host fills, and its bounded wait when the
flag is withheld (the kernel gives up after the limit, reports through the status word, and the context stays
usable).  The multi-GPU run of the same code is bench.py under torch.distributed.run, which asserts TP-N against the
dense layer before it times anything."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import random_ternary


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _oracle_matmul(x, w_local, scale):
    import oracle

    y = oracle.dense_f64(x.double().numpy(), w_local, scale)
    return torch.from_numpy(y)


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ternaryllm_b200.tensor_parallel import (ColumnParallelTernaryLinear, RowParallelTernaryLinear, shard_heads,
                                                     shard_rows)

        rng = np.random.default_rng(5)                     # same weights and activations on every rank
        K, N, M = 256, 96, 3
        w1 = random_ternary(rng, K, N, 0.6)
        w2 = random_ternary(rng, N, K, 0.5)
        x = torch.from_numpy(rng.integers(-8, 9, size=(M, K)).astype(np.float64))
        col = ColumnParallelTernaryLinear(w1, world, rank, scale=0.5, matmul=_oracle_matmul)
        row = RowParallelTernaryLinear(w2, world, rank, scale=2.0, matmul=_oracle_matmul)
        h_local = col(x)                                    # [M, N/world]
        gathered = [torch.empty_like(h_local) for _ in range(world)]
        dist.all_gather(gathered, h_local)
        h_full = torch.cat(gathered, dim=1)
        want_h = (x.numpy() @ w1.astype(np.float64)) * 0.5
        ok = np.array_equal(h_full.numpy(), want_h)
        y = row(h_local)                                    # consumes the local feature slice, all-reduces
        want_y = (want_h @ w2.astype(np.float64)) * 2.0
        ok = ok and np.array_equal(y.numpy(), want_y)
        # head-wise column shard keeps whole heads
        wh = shard_heads(w1, 6, 16, world, rank)
        ok = ok and wh.shape == (K, 96 // world) and np.array_equal(wh, w1[:, rank * 48:(rank + 1) * 48])
        ok = ok and np.array_equal(shard_rows(w2, world, rank), w2[rank * 48:(rank + 1) * 48])
        out.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_column_and_row_parallel_on_two_gloo_ranks():
    world = 2
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = [out.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(0, True), (1, True)]


def test_shard_errors():
    from ternaryllm_b200.tensor_parallel import shard_columns, shard_rows

    w = np.zeros((10, 6), np.int8)
    with pytest.raises(ValueError):
        shard_columns(w, 4, 0)
    with pytest.raises(ValueError):
        shard_rows(w, 3, 0)


def test_blocked_weights_are_the_same_model_at_every_degree():
    from ternaryllm_b200.tensor_parallel import DecoderWeights

    W = DecoderWeights(256, 512, 8, 2, 16, 0.5, seed=3)
    for name, axis in (("q", 1), ("o", 0), ("gate", 1), ("up", 1), ("down", 0)):
        full = getattr(W, name)()
        for world in (2, 4, 8):
            parts = [getattr(W, name)(world, r) for r in range(world)]
            assert np.array_equal(np.concatenate(parts, axis=axis), full), (name, world)
    for which in (0, 1):
        full = W.kv(which)
        assert full.shape == (256, 32)
        assert np.array_equal(np.concatenate([W.kv(which, 2, r) for r in range(2)], axis=1), full)
        # more ranks than KV heads: neighbouring ranks hold the same head
        for r in range(8):
            assert np.array_equal(W.kv(which, 8, r), full[:, (r // 4) * 16:(r // 4 + 1) * 16])
    assert abs((W.gate() == 0).mean() - 0.5) < 0.02


@pytest.mark.gpu
@pytest.mark.parametrize("reduce", ["peer", "nccl"])
def test_decoder_layer_single_rank_matches_dense_reference(reduce):
    """One decode step of the Llama-shaped layer (fused QKV, grouped-query attention over a synthetic cache, O, fused
    MLP, the reduction glue with world = 1) against the same layer with dense fp32 matrices.  Tolerance 2e-2 relative
    to the largest output: both round to bf16 between their stages, at slightly different places."""
    from ternaryllm_b200.tensor_parallel import TernaryDecoderLayerTP, reference_decoder_layer

    dev = torch.device("cuda", 0)
    hidden, ffn, hq, hkv, hd, S, M, L = 1024, 2816, 8, 2, 128, 0.5, 3, 64
    layer = TernaryDecoderLayerTP(hidden, ffn, hq, hkv, hd, S, 1, 0, dev, kv_len=L, max_batch=4, seed=40, reduce=reduce)
    g = torch.Generator(device="cpu").manual_seed(5)
    x = torch.randn((M, hidden), generator=g).to(dev, torch.bfloat16)
    want = reference_decoder_layer(layer.weights, x.float(), L, 4, 40)
    xs, pending = layer(x.clone())
    got = layer.finish(xs, pending).float()
    torch.cuda.synchronize()
    err = (got - want).abs().max().item() / want.abs().max().item()
    assert err < 2e-2, err
    # two layers in a row: the pending MLP output travels into the next layer's fused add + norm
    xs, pending = layer(x.clone())
    xs, pending = layer(xs, pending)
    assert torch.isfinite(layer.finish(xs, pending).float()).all()
    if layer.peer is not None:
        layer.peer.check()


def _comm(world, rank, rows, hidden):
    import ctypes as C

    from ternaryllm_b200 import _lib

    h = C.c_void_p()
    _lib.check(_lib.lib().tllm_comm_create(world, rank, rows, hidden, C.byref(h)))
    return h


@pytest.mark.gpu
@pytest.mark.parametrize("hidden,world,slices", [(1024, 2, 1), (8192, 2, 1), (8192, 4, 8)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_peer_allreduce_with_a_stand_in_peer(dtype, hidden, world, slices):
    """Rank 0 of a two- or four-rank communicator on one GPU.  The peers are one pair of buffers of this process: the
    kernel pushes rank 0's rows into them (checked), and finds the other ranks' rows and flags already in its own receive
    buffer, where the host put them -- the data path of real peers without a second kernel that this one would have to
    wait for.  x += p0 + p1 (+ p2 + p3), in rank order, in fp32, rounded once; h = RMSNorm(x) * weight.  Three calls in a
    row: the epochs and the two buffer sets advance.  From four ranks on, a row of 8192 values is shared by eight
    thread blocks that meet at a barrier in global memory for the sum of squares."""
    import ctypes as C

    from ternaryllm_b200 import _lib

    L = _lib.lib()
    dev = torch.device("cuda", 0)
    rows = 3                     # from four ranks on a row of 8192 values is shared by eight thread blocks
    h = _comm(world, 0, rows, hidden)
    recv, flags, rb, fb = C.c_void_p(), C.c_void_p(), C.c_int64(), C.c_int64()
    _lib.check(L.tllm_comm_buffers(h, C.byref(recv), C.byref(flags), C.byref(rb), C.byref(fb)))
    assert rb.value == 2 * world * rows * hidden * 4 and fb.value == 2 * world * rows * 8 * 4      # a flag per (set, rank, row, slice)
    peer_recv = torch.zeros(rb.value // 4, dtype=torch.float32, device=dev)
    peer_flags = torch.zeros(fb.value // 4, dtype=torch.int32, device=dev)
    for peer in range(1, world):
        _lib.check(L.tllm_comm_attach(h, peer, peer_recv.data_ptr(), peer_flags.data_ptr()))
    g = torch.Generator(device="cpu").manual_seed(1)
    x = torch.randn((rows, hidden), generator=g).to(dev, dtype)
    wgt = (1 + 0.1 * torch.randn(hidden, generator=g)).to(dev, dtype)
    for call in range(3):
        epoch, st = call + 1, (call + 1) & 1
        p0 = torch.randn((rows, hidden), generator=g).to(dev)
        total = p0.clone()
        for src in range(1, world):
            # a peer's part: its rows into slot [set][source] of rank 0's receive buffer, then its flags (one per slice)
            pk = torch.randn((rows, hidden), generator=g).to(dev)
            _copy(recv.value + ((st * world + src) * rows) * hidden * 4, pk.contiguous())
            _copy(flags.value + ((st * world + src) * rows) * 8 * 4, torch.full((rows * 8,), epoch, dtype=torch.int32, device=dev))
            total = total + pk
        want_x = (x.float() + total).to(dtype)
        hh = torch.empty_like(x)
        _lib.check(L.tllm_allreduce_add_rmsnorm(h, p0.data_ptr(), x.data_ptr(), wgt.data_ptr(), hh.data_ptr(), _lib.torch_dtype_code(dtype), rows,
                                                1e-6, torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        _lib.check(L.tllm_comm_check(h))
        assert torch.equal(x, want_x), call
        v = want_x.float()
        want_h = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + 1e-6) * wgt.float()
        assert (hh.float() - want_h).abs().max().item() <= 2e-2 * want_h.abs().max().item()
        # what rank 0 pushed to its peer: its rows in slot [set][src = 0], and the flags
        got = peer_recv[((st * world + 0) * rows) * hidden:((st * world + 0) * rows + rows) * hidden].view(rows, hidden)
        assert torch.equal(got, p0)
        assert torch.all(peer_flags[(st * world + 0) * rows * 8:((st * world + 0) * rows + rows) * 8].view(rows, 8)[:, :slices] == epoch)
    L.tllm_comm_destroy(h)


def _copy(dst_ptr, src):
    """device-to-device copy of a tensor to a raw device address"""
    from cuda.bindings import runtime as rt

    (err,) = rt.cudaMemcpy(dst_ptr, src.data_ptr(), src.numel() * src.element_size(), rt.cudaMemcpyKind.cudaMemcpyDeviceToDevice)
    assert int(err) == 0, err


@pytest.mark.gpu
def test_peer_allreduce_gives_up_when_a_flag_never_comes():
    """The peer's flag is never set: after the wait limit (set to 20 ms) the kernel stops waiting, finishes and writes
    the status word; the host reads it as an error, and the GPU keeps working."""
    import ctypes as C

    from ternaryllm_b200 import _lib

    L = _lib.lib()
    dev = torch.device("cuda", 0)
    rows, hidden = 2, 512
    h = _comm(2, 0, rows, hidden)
    rb, fb = C.c_int64(), C.c_int64()
    _lib.check(L.tllm_comm_buffers(h, None, None, C.byref(rb), C.byref(fb)))
    peer_recv = torch.zeros(rb.value // 4, dtype=torch.float32, device=dev)
    peer_flags = torch.zeros(fb.value // 4, dtype=torch.int32, device=dev)
    _lib.check(L.tllm_comm_attach(h, 1, peer_recv.data_ptr(), peer_flags.data_ptr()))
    _lib.check(L.tllm_comm_set_wait_limit(h, 20.0))
    x = torch.zeros((rows, hidden), dtype=torch.bfloat16, device=dev)
    p0 = torch.ones((rows, hidden), dtype=torch.float32, device=dev)
    hh = torch.empty_like(x)
    _lib.check(L.tllm_allreduce_add_rmsnorm(h, p0.data_ptr(), x.data_ptr(), None, hh.data_ptr(), _lib.BF16, rows, 1e-6,
                                            torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert L.tllm_comm_check(h) == -3 and b"never arrived" in L.tllm_last_error()
    assert L.tllm_comm_check(h) == 0                   # reported once
    assert float((torch.ones(8, device=dev) * 2).sum()) == 16.0     # the context is alive
    L.tllm_comm_destroy(h)
    # an unconnected communicator is refused on the host
    h2 = _comm(2, 1, rows, hidden)
    assert L.tllm_allreduce_add_rmsnorm(h2, p0.data_ptr(), x.data_ptr(), None, hh.data_ptr(), _lib.BF16, rows, 1e-6, None) == -1
    L.tllm_comm_destroy(h2)
