"""Tensor-parallel sharding logic on two CPU ranks (gloo): column shards concatenate to the full product, row
shards all-reduce to it.  The packed GPU product is replaced by the oracle's dense product here (tests only);
the GPU path of the same classes is covered by the decoder benchmark on real devices."""
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


@pytest.mark.gpu
def test_decoder_layer_single_rank_matches_fp32_reference():
    """One decode step of the Llama-shaped layer (fused QKV, grouped-query attention over a synthetic cache, O,
    fused MLP) against the same arithmetic in plain fp32 PyTorch on dense weights.  Tolerance 2e-2 relative to the
    largest output: the layer rounds to bf16 between its stages, the reference does not."""
    import torch.nn.functional as F

    from ternaryllm_b200.synthetic import make_weight
    from ternaryllm_b200.tensor_parallel import TernaryDecoderLayerTP, rms_norm

    dev = torch.device("cuda", 0)
    hidden, ffn, hq, hkv, hd, S, M, L = 1024, 2816, 8, 2, 128, 0.5, 3, 64
    layer = TernaryDecoderLayerTP(hidden, ffn, hq, hkv, hd, S, 1, 0, dev, kv_len=L, max_batch=4, seed=40, make_weight=make_weight)
    g = torch.Generator(device="cpu").manual_seed(5)
    x = torch.randn((M, hidden), generator=g).to(dev, torch.bfloat16)
    xs, delta = layer(x.clone())
    got = (xs + delta).float()
    torch.cuda.synchronize()

    def W(i, k, n):
        return torch.tensor(make_weight(40 + i, k, n, S), dtype=torch.float32, device=dev) * 0.02

    xf = x.float()
    h = rms_norm(xf)
    q, k, v = h @ W(1, hidden, hq * hd), h @ W(2, hidden, hkv * hd), h @ W(3, hidden, hkv * hd)
    kc, vc = layer.k_cache[:M].float().clone(), layer.v_cache[:M].float().clone()
    kc[:, :, L], vc[:, :, L] = k.view(M, hkv, hd), v.view(M, hkv, hd)
    a = F.scaled_dot_product_attention(q.view(M, hq, 1, hd), kc.repeat_interleave(hq // hkv, 1), vc.repeat_interleave(hq // hkv, 1))
    x1 = (xf + a.reshape(M, hq * hd) @ W(4, hq * hd, hidden)).bfloat16().float()    # the stream is stored in bf16
    h2 = rms_norm(x1)
    want = x1 + (F.silu(h2 @ W(5, hidden, ffn)) * (h2 @ W(6, hidden, ffn))) @ W(7, ffn, hidden)
    err = (got - want).abs().max().item() / want.abs().max().item()
    assert err < 2e-2, err


@pytest.mark.gpu
def test_attention_projections_fused_qkv_matches_three_products_and_fp32_reference():
    """LlamaTernaryAttention: one fused q|k|v product against the reference's three separate products
    (ternaryLLM_GPU/TernaryLLM/TernaryAttn.py:73-75) and against plain fp32 PyTorch on the dense weights;
    decode with a (k, v) cache and a causal multi-token call.  Tolerance 2e-2 of the largest output (fp16 rounding
    between the stages)."""
    import torch.nn.functional as F

    from ternaryllm_b200 import LlamaTernaryAttention, TernaryConfig

    dev = torch.device("cuda", 0)
    cfg = TernaryConfig(hidden_size=1024, intermediate_size=2816, num_attention_heads=8, num_key_value_heads=2, sparsity=0.6)
    g = torch.Generator().manual_seed(3)
    attn = LlamaTernaryAttention(cfg, layer_idx=0, scales=(0.03125,) * 4, generator=g)
    assert attn.fused_qkv
    hd, hq, hkv = cfg.head_dim, 8, 2
    x = torch.randn((2, 5, 1024), generator=g).to(dev, torch.float16)
    y, _, (k, v) = attn(x, use_cache=True)
    attn.fused_qkv = False
    y3, _, _ = attn(x, use_cache=True)
    attn.fused_qkv = True
    assert (y.float() - y3.float()).abs().max() <= 2e-3 * y3.float().abs().max()

    W = {n: getattr(attn, n).ternary_weight.to(dev, torch.float32) * 0.03125 for n in ("q_proj", "k_proj", "v_proj", "o_proj")}

    def ref(xf, past=None, causal=True):
        b, t, _ = xf.shape
        q = (xf @ W["q_proj"]).view(b, t, hq, hd).transpose(1, 2)
        kk = (xf @ W["k_proj"]).view(b, t, hkv, hd).transpose(1, 2)
        vv = (xf @ W["v_proj"]).view(b, t, hkv, hd).transpose(1, 2)
        if past is not None:
            kk, vv = torch.cat([past[0], kk], 2), torch.cat([past[1], vv], 2)
        o = F.scaled_dot_product_attention(q, kk.repeat_interleave(hq // hkv, 1), vv.repeat_interleave(hq // hkv, 1), is_causal=causal and t > 1)
        return o.transpose(1, 2).reshape(b, t, hq * hd) @ W["o_proj"], (kk, vv)

    want, (kr, vr) = ref(x.float())
    assert (y.float() - want).abs().max() <= 2e-2 * want.abs().max()
    # one more token on top of the cache
    x1 = torch.randn((2, 1, 1024), generator=g).to(dev, torch.float16)
    y1, _, _ = attn(x1, past_key_value=(k, v), use_cache=True)
    want1, _ = ref(x1.float(), past=(kr, vr), causal=False)
    assert (y1.float() - want1).abs().max() <= 2e-2 * want1.abs().max()


@pytest.mark.gpu
def test_add_rms_norm_matches_pytorch():
    """tllm_add_rmsnorm against the same arithmetic in PyTorch (fp32 sums, one rounding of the stream, one of the
    normalised output): the stream must be identical, the output within one unit in the last place."""
    from ternaryllm_b200.tensor_parallel import add_rms_norm

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(8)
    for dtype, ulp in ((torch.float32, 2.0 ** -22), (torch.float16, 2.0 ** -10), (torch.bfloat16, 2.0 ** -7)):
        for rows, hidden in ((1, 8192), (5, 1000), (64, 4096)):
            x = torch.randn((rows, hidden), generator=g).to(dev, dtype)
            d = torch.randn((rows, hidden), generator=g).to(dev, dtype)
            w = (torch.rand((hidden,), generator=g) + 0.5).to(dev, dtype)
            x2 = x.clone()
            h = add_rms_norm(x2, d, weight=w)
            xr = (x.float() + d.float()).to(dtype)
            assert torch.equal(x2, xr)
            hr = xr.float() * torch.rsqrt(xr.float().pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()
            assert ((h.float() - hr).abs() <= ulp * hr.abs() + 1e-6).all()
            x3 = x.clone()
            h0 = add_rms_norm(x3, None)
            assert torch.equal(x3, x)
            h0r = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6)
            assert ((h0.float() - h0r).abs() <= ulp * h0r.abs() + 1e-6).all()
