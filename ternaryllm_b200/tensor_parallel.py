"""Tensor-parallel partitioning of ternary Llama linears across the GPUs of one node.

The reference has no distributed code; this is the usual partitioning of a tensor-parallel decode deployment on
top of the packed product: gate / up / QKV are **column-sharded** (the input is replicated, every rank produces its slice of the
output, no exchange), down / O are **row-sharded** (every rank holds the K-rows that match its slice of the
intermediate activations and produces a full-width partial result, one all-reduce(sum) per linear).  Shards are
cut before packing, so every rank packs and streams only its own index lists.

One process per GPU; `torch.distributed` (NCCL over NVLink on GPUs, gloo in the CPU tests) carries the
all-reduce.  `world == 1` makes every collective a no-op.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist
from torch import nn

from . import _lib
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


class TernaryDecoderLayerTP(nn.Module):
    """One Llama-shaped decoder layer for single-token decode with ternary linears, tensor-parallel.

    Only the linears are this library's work; RMSNorm, the attention core (scaled-dot-product over a synthetic
    KV cache, grouped-query) and the residual adds are stock PyTorch, as in the reference, whose attention is
    stock Hugging Face code (ternaryLLM_GPU/TernaryLLM/TernaryAttn.py:78-120).
    """

    def __init__(self, hidden, ffn, n_heads, n_kv_heads, head_dim, sparsity, world, rank, device, dtype=torch.bfloat16,
                 kv_len=1024, max_batch=64, seed=0, make_weight=None):
        super().__init__()
        self.hidden, self.ffn, self.hd = hidden, ffn, head_dim
        self.hq, self.hkv = n_heads // world, max(1, n_kv_heads // world)
        if n_heads % world or (n_kv_heads % world and world % n_kv_heads) or ffn % world:
            raise ValueError("heads or FFN columns do not split over the ranks")
        self.world, self.rank, self.device, self.dtype = world, rank, device, dtype
        mk = make_weight
        # Every rank draws its own shards directly (independent seeds per matrix and rank): the masks are i.i.d., so a
        # shard of a big random matrix and a random matrix of the shard's shape are the same thing, and no rank has to
        # generate the other ranks' entries.  Column-sharded QKV: this rank's query heads, then its key heads, then
        # its value heads, in one packed weight.  With fewer KV heads than ranks, the ranks that share a KV head
        # draw it from the same seed.
        kv_owner = rank if n_kv_heads >= world else rank // (world // n_kv_heads)
        sd = seed + 1000 * rank
        wq = mk(sd + 1, hidden, self.hq * head_dim, sparsity)
        wk = mk(seed + 1000 * kv_owner + 2, hidden, self.hkv * head_dim, sparsity)
        wv = mk(seed + 1000 * kv_owner + 3, hidden, self.hkv * head_dim, sparsity)
        self.qkv = PackedWeight.from_dense(np.ascontiguousarray(np.concatenate([wq, wk, wv], axis=1)), 0.02, device)
        del wq, wk, wv
        self.o = PackedWeight.from_dense(mk(sd + 4, self.hq * head_dim, hidden, sparsity), 0.02, device)
        wg = mk(sd + 5, hidden, ffn // world, sparsity)
        wu = mk(sd + 6, hidden, ffn // world, sparsity)
        wd = mk(sd + 7, ffn // world, hidden, sparsity)
        self.mlp = PackedMLP(wg, wu, wd, 0.02, 0.02, 0.02, device)
        self.nnz_local = int(self.qkv.info["nnz"] + self.o.info["nnz"] + sum(i["nnz"] for i in self.mlp.info))
        self.alg_bytes_local = int(self.qkv.info["algorithmic_bytes"] + self.o.info["algorithmic_bytes"] +
                                   sum(i["algorithmic_bytes"] for i in self.mlp.info))
        del wg, wu, wd
        g = torch.Generator(device="cpu").manual_seed(seed)
        # kv_len cached positions plus the slot the new token's key and value are written to
        self.kv_len = kv_len
        self.k_cache = torch.randn((max_batch, self.hkv, kv_len + 1, head_dim), generator=g).to(device, dtype)
        self.v_cache = torch.randn((max_batch, self.hkv, kv_len + 1, head_dim), generator=g).to(device, dtype)

    def forward(self, x, delta=None):
        """x [M, hidden]: the residual stream, one new token per sequence, **updated in place**; delta: the previous
        layer's MLP output that has not been added yet.  Returns (x, this layer's MLP output still to be added):
        the add travels with the next RMSNorm, so a layer launches two glue kernels instead of a dozen."""
        M = x.shape[0]
        h = add_rms_norm(x, delta)
        qkv = self.qkv.matmul(h)
        q, k, v = qkv.split([self.hq * self.hd, self.hkv * self.hd, self.hkv * self.hd], dim=1)
        q = q.view(M, self.hq, 1, self.hd)
        kc, vc = self.k_cache[:M], self.v_cache[:M]
        kc[:, :, self.kv_len].copy_(k.view(M, self.hkv, self.hd))
        vc[:, :, self.kv_len].copy_(v.view(M, self.hkv, self.hd))
        a = torch.nn.functional.scaled_dot_product_attention(q, kc, vc, enable_gqa=self.hq != self.hkv)
        o = all_reduce_sum(self.o.matmul(a.reshape(M, self.hq * self.hd)))
        h2 = add_rms_norm(x, o)
        y = all_reduce_sum(self.mlp.forward(h2))
        return x, y
