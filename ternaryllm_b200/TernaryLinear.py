"""TernaryLinear: the operator module of the reference (ternaryLLM_GPU/TernaryLLM/TernaryLinear.py:115-182),
same constructor arguments and buffer names, running on the library's B200 kernels through a packed handle.

What is kept: `in_features`, `out_features`, `sparsity`, `uniform`, `uniform_blk_size`, `padding`,
`padding_size`, `bias`, `device`, `dtype`; the attribute `ternary_weight` (int32 [K, N] on the CPU); the
non-persistent buffers `w_row_indices` (int16), `w_col_offsets` (int32), `w_col_tile_indices` (int16) in the
reference's merged tiled CSC layout -- built losslessly -- so that code which inspects them or feeds them
to `ter_spmm.ter_spmm` keeps working.

What is added: `scale` (per-tensor s, default 1.0), `weight=` to pack a given ternary matrix instead of a
random one, fp16 / bf16 / int8 activations, any K (the reference raises KeyError for K outside its map,
:9-16), and a correct result for row-major [batch, rows, K] inputs (the reference kernel reads them as
[K][rows], ternaryLLM_GPU/csrc/ter_spmm_kernel.cuh:173).  A 2-D input [rows, K] returns [rows, N]; the
reference launches nothing for it (:168).  `bias=True` creates a float bias that IS applied; the reference
allocates an int32 Parameter (which torch rejects) and never applies it (:137-140).
"""
from __future__ import annotations

import numpy as np
import torch
from torch import Tensor, nn

from . import ter_spmm as _ter_spmm
from .weight import PackedWeight

MapKSizeToTileSize = {8192: 512, 4096: 512, 3072: 512, 2048: 256, 1024: 256, 512: 64}


def ternarize_weights(w: torch.Tensor, sparsity: float = None, threshold_factor: float = 0.7):
    """Float weights [in_features, out_features] -> (int32 ternary weights, per-tensor scale).  The reference's function
    of this name raises NotImplementedError (TernaryLinear.py:19-20); this one applies the threshold rule of ternary
    weight networks (|w| <= threshold_factor * mean|w| -> 0, or the `sparsity` fraction of smallest magnitudes -> 0;
    the rest -> sign(w); scale = mean |w| of the kept entries).  Runs on the host (tllm_ternarize)."""
    from .weight import ternarize

    t, s = ternarize(w, sparsity=sparsity, threshold_factor=threshold_factor)
    return torch.from_numpy(t.astype(np.int32)), s


def random_ternary_weights(size: tuple, sparsity: float = 0.8, uniform: bool = False, block_size: int = 512,
                           generator: torch.Generator | None = None):
    """Random ternary weight [K, N], int32, on the CPU.

    Non-uniform: i.i.d. P(0) = sparsity, P(-1) = P(+1) = (1 - sparsity)/2 (TernaryLinear.py:79-83).
    Uniform: every `block_size`-long run along K of a column holds the same number of +1 and -1
    (TernaryLinear.py:39-77).  `generator` makes it reproducible (the reference uses the global RNG).
    """
    K, N = size
    if not uniform:
        r = torch.rand(size, generator=generator)
        w = torch.zeros(size, dtype=torch.int32)
        w[(r >= sparsity) & (r < (sparsity + 1) / 2)] = -1
        w[r >= (sparsity + 1) / 2] = 1
        return w
    total = K * N
    if total % block_size:
        raise ValueError("uniform weights need K*N to be a multiple of the block size")
    blocks = total // block_size
    nnz_total = int(total * (1 - sparsity)) // 2 * 2
    base = (nnz_total // blocks) // 2 * 2
    counts = np.full(blocks, base, np.int64)
    extra = (nnz_total - base * blocks) // 2
    counts[np.arange(extra) % blocks] += 2
    # one random permutation per block, vectorised: the first `count` positions get the signs
    order = torch.rand((blocks, block_size), generator=generator).argsort(dim=1).numpy()
    flat = np.zeros((blocks, block_size), np.int32)
    rank = np.empty_like(order)
    np.put_along_axis(rank, order, np.arange(block_size)[None, :].repeat(blocks, 0), axis=1)
    half = (counts // 2)[:, None]
    flat[rank < half] = 1
    flat[(rank >= half) & (rank < 2 * half)] = -1
    return torch.from_numpy(flat.reshape(N, K).T.copy())


def convert_ternary_weights(w: torch.Tensor, padding: bool = False, padding_size: int = 4, dtype=torch.int32, device="cpu",
                            tile_k: int | None = None):
    """Merged tiled CSC buffers of a ternary weight [K, N] (TernaryLinear.py:87-113): returns
    (row_indices, col_offsets, col_tile_indices).  Lossless, unlike the reference's packer."""
    w_ = w.detach().to("cpu", torch.int32).contiguous()
    K, N = w_.shape
    tile = tile_k or _ter_spmm.tile_size_for(K)
    idx, off, til = _ter_spmm.convert_to_ter_tiled_mcsc(w_, N, K, int((w_ == 1).sum()), int((w_ == -1).sum()), tile, padding,
                                                        padding_size, as_numpy=True)
    return (torch.from_numpy(idx).to(device).to(dtype), torch.from_numpy(off).to(device),
            torch.from_numpy(til).to(device).to(dtype))


class TernaryLinear(nn.Module):
    __constants__ = ["in_features", "out_features"]

    def __init__(self, in_features: int, out_features: int, sparsity: float = 0.8, uniform: bool = False,
                 uniform_blk_size: int = 512, padding: bool = False, padding_size: int = 4, bias: bool = True, device=None,
                 dtype=torch.int32, scale: float = 1.0, weight: Tensor | None = None, reference_buffers: bool = True,
                 generator: torch.Generator | None = None, pack_opts: dict | None = None) -> None:
        super().__init__()
        if bias:
            self.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=torch.float32))
        else:
            self.register_parameter("bias", None)
        if weight is None:
            weight = random_ternary_weights((in_features, out_features), sparsity, uniform, uniform_blk_size, generator)
        elif tuple(weight.shape) != (in_features, out_features):
            raise ValueError("weight must be [in_features, out_features]")
        self.ternary_weight = weight.detach().to("cpu", torch.int32).contiguous()
        if reference_buffers:
            ri, co, ti = convert_ternary_weights(self.ternary_weight, padding=padding, padding_size=padding_size, device=device,
                                                 dtype=torch.int16)
        else:
            ri = torch.empty(0, dtype=torch.int16, device=device)
            co = torch.empty(0, dtype=torch.int32, device=device)
            ti = torch.empty(0, dtype=torch.int16, device=device)
        self.register_buffer("w_row_indices", ri, False)
        self.register_buffer("w_col_offsets", co, False)
        self.register_buffer("w_col_tile_indices", ti, False)
        self.in_features = in_features
        self.out_features = out_features
        self.uniform = uniform
        self.padding = padding
        self.scale = float(scale)
        self._pack_opts = dict(pack_opts or {})
        self._packed: dict[int, PackedWeight] = {}

    def packed(self, device: torch.device) -> PackedWeight:
        """The packed handle of the weight on `device`, made on first use."""
        idx = device.index if device.index is not None else torch.cuda.current_device()
        pw = self._packed.get(idx)
        if pw is None:
            pw = PackedWeight.from_dense(self.ternary_weight.numpy().astype(np.int8), self.scale, torch.device("cuda", idx),
                                         **self._pack_opts)
            self._packed[idx] = pw
        return pw

    @classmethod
    def from_float(cls, linear_weight: Tensor, sparsity: float = None, threshold_factor: float = 0.7, **kw):
        """A TernaryLinear from the weight of an `nn.Linear` ([out_features, in_features], as PyTorch stores it):
        ternarised with `ternarize_weights`, the per-tensor scale kept in `scale`."""
        w, s = ternarize_weights(linear_weight.detach().t().contiguous(), sparsity=sparsity, threshold_factor=threshold_factor)
        return cls(w.shape[0], w.shape[1], weight=w, scale=s, **kw)

    def forward(self, input: Tensor) -> Tensor:
        """input: (batch, rows, K) | (batch, K, rows) | (rows, K)  ->  (batch, rows, N) | (rows, N)"""
        assert len(input.shape) <= 3, "Input has dim larger than 3"
        if input.device.type != "cuda":
            raise RuntimeError("TernaryLinear runs on CUDA tensors only (there is no CPU path)")
        K = self.in_features
        if input.shape[-1] == K:
            x2 = input.reshape(-1, K)
            lead = tuple(input.shape[:-1])
        elif input.dim() == 3 and input.shape[-2] == K:
            x2 = input.transpose(1, 2).reshape(-1, K)
            lead = (input.shape[0], input.shape[2])
        else:
            raise RuntimeError(f"input of shape {tuple(input.shape)} has no dimension of size in_features={K}")
        y = self.packed(input.device).matmul(x2)
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        return y.reshape(*lead, self.out_features)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, scale={self.scale}, uniform={self.uniform}"


__all__ = ["TernaryLinear", "ternarize_weights", "random_ternary_weights", "convert_ternary_weights"]
