"""Tensor-parallel partitioning of ternary Llama linears across the GPUs of one node.

The reference has no distributed code; this is the usual partitioning of a tensor-parallel decode deployment on
top of the packed product: gate / up / QKV are **column-sharded** (the input is replicated, every rank produces
its slice of the output, no exchange), down / O are **row-sharded** (every rank holds the K-rows that match its
slice of the intermediate activations and produces a full-width partial result that has to be summed over the
ranks).  Shards are cut before packing, so every rank packs and streams only its own index lists.

The sum over ranks is either an NCCL all-reduce followed by the residual-add + RMSNorm kernel (two launches), or
the library's own kernel that does all three over peer-mapped memory in one launch (`PeerReduce`,
tllm_allreduce_add_rmsnorm): every rank pushes its fp32 partial rows into a slot on every peer with plain stores
over NVLink, raises a flag, waits (bounded) for the peers' flags and reduces in rank order.

One process per GPU; `torch.distributed` (NCCL on GPUs, gloo in the CPU tests) carries the rendezvous and the
fallback all-reduce.  `world == 1` makes every collective a no-op.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch
import torch.distributed as dist
from torch import nn

from . import _lib
from .synthetic import block_weight
from .weight import PackedMLP, PackedWeight


def shard_columns(w: np.ndarray, world: int, rank: int) -> np.ndarray:
    """Columns [rank*N/world, (rank+1)*N/world) of W [K, N]."""
    K, N = w.shape
    if N % world:
        raise ValueError(f"{N} columns do not split over {world} ranks")
    c = N // world
    return np.ascontiguousarray(w[:, rank * c:(rank + 1) * c])


def shard_rows(w: np.ndarray, world: int, rank: int) -> np.ndarray:
    """Rows [rank*K/world, (rank+1)*K/world) of W [K, N]."""
    K, N = w.shape
    if K % world:
        raise ValueError(f"{K} rows do not split over {world} ranks")
    r = K // world
    return np.ascontiguousarray(w[rank * r:(rank + 1) * r, :])


def shard_heads(w: np.ndarray, n_heads: int, head_dim: int, world: int, rank: int) -> np.ndarray:
    """Column shard of a projection whose columns are n_heads blocks of head_dim: whole heads per rank."""
    if n_heads % world:
        raise ValueError(f"{n_heads} heads do not split over {world} ranks")
    h = n_heads // world
    return np.ascontiguousarray(w[:, rank * h * head_dim:(rank + 1) * h * head_dim])


def all_reduce_sum(t: torch.Tensor, group=None) -> torch.Tensor:
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return t


class ColumnParallelTernaryLinear(nn.Module):
    """y_local = x @ W[:, shard] * s   (x replicated; no communication)."""

    def __init__(self, weight: np.ndarray, world: int, rank: int, scale: float = 1.0, device=None, matmul=None):
        super().__init__()
        self.world, self.rank = world, rank
        self.local = shard_columns(np.asarray(weight), world, rank)
        self.scale = float(scale)
        self._matmul = matmul
        self._packed = None if matmul else PackedWeight.from_dense(self.local, self.scale, device)

    def forward(self, x):
        if self._matmul:
            return self._matmul(x, self.local, self.scale)
        return self._packed.matmul(x)


class RowParallelTernaryLinear(nn.Module):
    """y = all_reduce_sum( x_local @ W[shard, :] * s )   (x_local = this rank's slice of the features)."""

    def __init__(self, weight: np.ndarray, world: int, rank: int, scale: float = 1.0, device=None, matmul=None, group=None):
        super().__init__()
        self.world, self.rank, self.group = world, rank, group
        self.local = shard_rows(np.asarray(weight), world, rank)
        self.scale = float(scale)
        self._matmul = matmul
        self._packed = None if matmul else PackedWeight.from_dense(self.local, self.scale, device)

    def forward(self, x_local):
        y = self._matmul(x_local, self.local, self.scale) if self._matmul else self._packed.matmul(x_local)
        return all_reduce_sum(y, self.group)


def rms_norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """RMSNorm with unit weight (the benchmark configuration sets the norm weights to 1)."""
    v = x.float()
    return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)


def add_rms_norm(x: torch.Tensor, delta, out: torch.Tensor = None, weight: torch.Tensor = None, eps: float = 1e-6) -> torch.Tensor:
    """One launch: x += delta in place (skipped when delta is None), returns RMSNorm(x) (tllm_add_rmsnorm)."""
    if x.device.type != "cuda" or not x.is_contiguous() or x.dim() != 2:
        raise RuntimeError("add_rms_norm expects a contiguous 2-D CUDA tensor")
    if out is None:
        out = torch.empty_like(x)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().tllm_add_rmsnorm(x.data_ptr(), delta.data_ptr() if delta is not None else None,
                                               weight.data_ptr() if weight is not None else None, out.data_ptr(),
                                               _lib.torch_dtype_code(x.dtype), x.shape[0], x.shape[1], float(eps),
                                               torch.cuda.current_stream().cuda_stream), "tllm_add_rmsnorm")
    return out


class PeerReduce:
    """The all-reduce of a row-sharded product fused with the residual add and RMSNorm that follow it, over
    peer-mapped memory (tllm_comm_* in include/tllm.h).

    Every rank constructs one with the same `max_rows` and `hidden`; the inter-process memory handles travel
    through `torch.distributed` (all_gather_object), everything after that is this library's kernel.
    `reduce(partial, x)`:  x += sum over ranks of partial (fp32 [rows, hidden]);  returns RMSNorm(x).
    """

    def __init__(self, max_rows: int, hidden: int, device, group=None, wait_ms: float | None = None):
        self.device = torch.device(device)
        self.world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.max_rows, self.hidden = int(max_rows), int(hidden)
        L = _lib.lib()
        h = C.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(L.tllm_comm_create(self.world, self.rank, self.max_rows, self.hidden, C.byref(h)), "tllm_comm_create")
            self._h = h
            if self.world > 1:
                n = L.tllm_comm_handle_bytes()
                mine = (C.c_ubyte * n)()
                _lib.check(L.tllm_comm_export(self._h, mine), "tllm_comm_export")
                gathered = [None] * self.world
                dist.all_gather_object(gathered, bytes(mine), group=group)
                blob = b"".join(gathered)
                buf = (C.c_ubyte * len(blob)).from_buffer_copy(blob)
                _lib.check(L.tllm_comm_connect(self._h, buf), "tllm_comm_connect")
                dist.barrier(group=group)       # nobody pushes before everybody has mapped everybody
            if wait_ms is not None:
                _lib.check(L.tllm_comm_set_wait_limit(self._h, float(wait_ms)), "tllm_comm_set_wait_limit")

    def reduce(self, partial: torch.Tensor, x: torch.Tensor, out: torch.Tensor = None, weight: torch.Tensor = None, eps: float = 1e-6):
        if partial.dtype != torch.float32 or partial.shape != x.shape or not partial.is_contiguous() or not x.is_contiguous():
            raise RuntimeError("PeerReduce.reduce expects a contiguous fp32 partial of the shape of x")
        if out is None:
            out = torch.empty_like(x)
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().tllm_allreduce_add_rmsnorm(self._h, partial.data_ptr(), x.data_ptr(),
                                                             weight.data_ptr() if weight is not None else None, out.data_ptr(),
                                                             _lib.torch_dtype_code(x.dtype), x.shape[0], float(eps),
                                                             torch.cuda.current_stream().cuda_stream), "tllm_allreduce_add_rmsnorm")
        return out

    def check(self):
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().tllm_comm_check(self._h), "PeerReduce")

    def close(self):
        if getattr(self, "_h", None):
            _lib.lib().tllm_comm_destroy(self._h)
            self._h = None


class DecoderWeights:
    """The dense ternary matrices of one decoder layer in a canonical form that every tensor-parallel degree cuts the
    same way: each matrix is the concatenation of `blocks` (8) independently seeded blocks along its sharded axis, so a
    rank generates only its own blocks, and TP-1, TP-2, TP-4 and TP-8 all see the same model.

    q: [hidden, heads*hd] in head blocks; k, v: [hidden, kv_heads*hd]; o: [heads*hd, hidden] in row blocks;
    gate, up: [hidden, ffn]; down: [ffn, hidden] in row blocks.
    """

    BLOCKS = 8

    def __init__(self, hidden, ffn, n_heads, n_kv_heads, head_dim, sparsity, seed):
        self.hidden, self.ffn, self.nh, self.nkv, self.hd, self.s, self.seed = hidden, ffn, n_heads, n_kv_heads, head_dim, sparsity, seed
        B = self.BLOCKS
        if n_heads % B or ffn % B or (n_kv_heads % B and B % n_kv_heads):
            raise ValueError("heads / FFN columns do not split into 8 blocks")

    def _take(self, world, rank):
        per = self.BLOCKS // world
        return rank * per, per

    def q(self, world=1, rank=0):
        f, c = self._take(world, rank)
        return block_weight(self.seed + 1, self.hidden, self.nh * self.hd, self.s, 1, self.BLOCKS, f, c)

    def kv(self, which, world=1, rank=0):
        """k (which = 0) or v (1) columns of this rank: its KV heads; with fewer KV heads than ranks, neighbouring ranks
        hold the same head."""
        nb = min(self.BLOCKS, self.nkv)
        if world <= nb:
            per = nb // world
            return block_weight(self.seed + 2 + which, self.hidden, self.nkv * self.hd, self.s, 1, nb, rank * per, per)
        return block_weight(self.seed + 2 + which, self.hidden, self.nkv * self.hd, self.s, 1, nb, rank // (world // nb), 1)

    def o(self, world=1, rank=0):
        f, c = self._take(world, rank)
        return block_weight(self.seed + 4, self.nh * self.hd, self.hidden, self.s, 0, self.BLOCKS, f, c)

    def gate(self, world=1, rank=0):
        f, c = self._take(world, rank)
        return block_weight(self.seed + 5, self.hidden, self.ffn, self.s, 1, self.BLOCKS, f, c)

    def up(self, world=1, rank=0):
        f, c = self._take(world, rank)
        return block_weight(self.seed + 6, self.hidden, self.ffn, self.s, 1, self.BLOCKS, f, c)

    def down(self, world=1, rank=0):
        f, c = self._take(world, rank)
        return block_weight(self.seed + 7, self.ffn, self.hidden, self.s, 0, self.BLOCKS, f, c)


def kv_cache(seed, kv_head, max_batch, kv_len, head_dim):
    """Synthetic cache of one KV head, [max_batch, kv_len + 1, head_dim] fp32 (the last position is the slot the new
    token is written to): a function of (seed, head) only, so every tensor-parallel degree holds the same cache."""
    g = torch.Generator(device="cpu").manual_seed(seed * 1000 + kv_head)
    return torch.randn((max_batch, kv_len + 1, head_dim), generator=g)


class TernaryDecoderLayerTP(nn.Module):
    """One Llama-shaped decoder layer for single-token decode with ternary linears, tensor-parallel.

    Only the linears and the reduction glue are this library's work; the attention core (scaled-dot-product over a
    synthetic KV cache, grouped-query) is stock PyTorch, as in the reference, whose attention is stock Hugging Face
    code (ternaryLLM_GPU/TernaryLLM/TernaryAttn.py:78-120).

    reduce: "peer" -- tllm_allreduce_add_rmsnorm (one launch per reduction, fp32 partial sums over peer memory);
            "nccl" -- NCCL all-reduce of the bf16 partial result + tllm_add_rmsnorm.
    """

    SCALE = 0.02

    def __init__(self, hidden, ffn, n_heads, n_kv_heads, head_dim, sparsity, world, rank, device, dtype=torch.bfloat16,
                 kv_len=1024, max_batch=64, seed=0, reduce="peer", peer: PeerReduce | None = None):
        super().__init__()
        self.hidden, self.ffn, self.hd = hidden, ffn, head_dim
        self.hq, self.hkv = n_heads // world, max(1, n_kv_heads // world)
        if n_heads % world or (n_kv_heads % world and world % n_kv_heads) or ffn % world or DecoderWeights.BLOCKS % world:
            raise ValueError("heads or FFN columns do not split over the ranks")
        self.world, self.rank, self.device, self.dtype = world, rank, torch.device(device), dtype
        self.reduce = reduce if world > 1 or reduce == "peer" else "nccl"
        self.peer = peer
        if self.reduce == "peer" and peer is None:
            self.peer = PeerReduce(max_batch, hidden, device)
        W = DecoderWeights(hidden, ffn, n_heads, n_kv_heads, head_dim, sparsity, seed)
        self.weights = W
        # column-sharded QKV: this rank's query heads, then its key heads, then its value heads, in one packed weight
        self.qkv = PackedWeight.from_dense(np.ascontiguousarray(np.concatenate([W.q(world, rank), W.kv(0, world, rank), W.kv(1, world, rank)], axis=1)),
                                           self.SCALE, device)
        self.o = PackedWeight.from_dense(W.o(world, rank), self.SCALE, device)
        self.mlp = PackedMLP(W.gate(world, rank), W.up(world, rank), W.down(world, rank), self.SCALE, self.SCALE, self.SCALE, device)
        self.nnz_local = int(self.qkv.info["nnz"] + self.o.info["nnz"] + sum(i["nnz"] for i in self.mlp.info))
        self.alg_bytes_local = int(self.qkv.info["algorithmic_bytes"] + self.o.info["algorithmic_bytes"] +
                                   sum(i["algorithmic_bytes"] for i in self.mlp.info))
        self.kv_len = kv_len
        if n_kv_heads >= world:
            heads = list(range(rank * self.hkv, (rank + 1) * self.hkv))
        else:
            heads = [rank // (world // n_kv_heads)]
        self.k_cache = torch.stack([kv_cache(seed + 11, h, max_batch, kv_len, head_dim) for h in heads], 1).to(self.device, dtype)
        self.v_cache = torch.stack([kv_cache(seed + 12, h, max_batch, kv_len, head_dim) for h in heads], 1).to(self.device, dtype)
        self._part = torch.empty((max_batch, hidden), dtype=torch.float32, device=self.device)    # O projection's partial sums
        self._part2 = torch.empty((max_batch, hidden), dtype=torch.float32, device=self.device)   # down projection's

    def attention(self, qkv, M):
        q, k, v = qkv.split([self.hq * self.hd, self.hkv * self.hd, self.hkv * self.hd], dim=1)
        q = q.view(M, self.hq, 1, self.hd)
        kc, vc = self.k_cache[:M], self.v_cache[:M]
        kc[:, :, self.kv_len].copy_(k.view(M, self.hkv, self.hd))
        vc[:, :, self.kv_len].copy_(v.view(M, self.hkv, self.hd))
        a = torch.nn.functional.scaled_dot_product_attention(q, kc, vc, enable_gqa=self.hq != self.hkv)
        return a.reshape(M, self.hq * self.hd)

    def forward(self, x, pending=None):
        """x [M, hidden]: the residual stream, one new token per sequence, **updated in place**; pending: the previous
        layer's MLP output that has not been added (and, with reduce = "peer", not been summed over the ranks) yet.
        Returns (x, this layer's MLP output still to be added): the add travels with the next RMSNorm."""
        M = x.shape[0]
        if self.reduce == "peer":
            h = add_rms_norm(x, None) if pending is None else self.peer.reduce(pending, x)
            a = self.attention(self.qkv.matmul(h), M)
            h2 = self.peer.reduce(self.o.matmul(a, out=self._part[:M]), x)
            return x, self.mlp.forward(h2, out=self._part2[:M])
        h = add_rms_norm(x, pending)
        a = self.attention(self.qkv.matmul(h), M)
        h2 = add_rms_norm(x, all_reduce_sum(self.o.matmul(a)))
        return x, all_reduce_sum(self.mlp.forward(h2))

    def finish(self, x, pending):
        """Adds the last layer's pending MLP output: returns the final residual stream."""
        if pending is None:
            return x
        if self.reduce == "peer":
            self.peer.reduce(pending, x)
            return x
        return x + pending


def reference_decoder_layer(W: DecoderWeights, x, kv_len, max_batch, seed, scale=TernaryDecoderLayerTP.SCALE):
    """The same layer with dense fp32 matrices on the device of x (the full, un-sharded model): what every
    tensor-parallel degree has to reproduce.  x [M, hidden] float32 is not modified; returns the residual stream after
    the layer (MLP output added).  Rounding points follow the packed path: the linears' inputs and the attention core
    run in bf16."""
    dev = x.device
    M = x.shape[0]
    bf = torch.bfloat16

    def lin(a, w):
        return (a.to(bf).float() @ torch.tensor(w, device=dev).float()) * scale

    def norm(v):
        return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + 1e-6)).to(bf)

    xr = x.to(bf).float()
    h = norm(xr)
    q = lin(h, W.q()).to(bf).view(M, W.nh, 1, W.hd)
    k = lin(h, W.kv(0)).to(bf).view(M, W.nkv, W.hd)
    v = lin(h, W.kv(1)).to(bf).view(M, W.nkv, W.hd)
    kc = torch.stack([kv_cache(seed + 11, hh, max_batch, kv_len, W.hd) for hh in range(W.nkv)], 1)[:M].to(dev, bf).clone()
    vc = torch.stack([kv_cache(seed + 12, hh, max_batch, kv_len, W.hd) for hh in range(W.nkv)], 1)[:M].to(dev, bf).clone()
    kc[:, :, kv_len] = k
    vc[:, :, kv_len] = v
    a = torch.nn.functional.scaled_dot_product_attention(q, kc, vc, enable_gqa=W.nh != W.nkv).reshape(M, W.nh * W.hd)
    xr = (xr + lin(a, W.o())).to(bf).float()
    h2 = norm(xr)
    g, u = lin(h2, W.gate()), lin(h2, W.up())
    hh = (g * torch.sigmoid(g) * u).to(bf)
    return (xr + lin(hh, W.down())).to(bf).float()
