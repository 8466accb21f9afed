"""LlamaTernaryMLP: down(silu(gate(x)) * up(x)) (ternaryLLM_GPU/TernaryLLM/TernaryMLP.py:11-35).

Same sub-module names (`gate_proj`, `up_proj`, `down_proj`).  The reference issues three products and two
element-wise kernels; here the forward pass is two launches: gate and up share one activation table and the
epilogue applies SiLU and the product, and the down projection starts streaming its weights while that
kernel drains.  `fused=False` gives the reference's five-step composition on the same kernels.
"""
from __future__ import annotations

import numpy as np
import torch
from torch import nn

from .configuration_ternary import TernaryConfig
from .TernaryLinear import TernaryLinear
from .weight import PackedMLP


class LlamaTernaryMLP(nn.Module):
    def __init__(self, config: TernaryConfig, scales=(1.0, 1.0, 1.0), fused: bool = True, generator=None, reference_buffers: bool = False):
        super().__init__()
        self.config = config
        self.hidden_size = config.hidden_size
        self.intermediate_size = config.intermediate_size
        if config.hidden_act != "silu":
            raise NotImplementedError("only hidden_act='silu' is supported")
        kw = dict(sparsity=config.sparsity, uniform=config.uniform_sparsity, uniform_blk_size=config.uniform_sparsity_block_size,
                  padding=config.padding, padding_size=config.padding_size, bias=config.mlp_bias, generator=generator,
                  reference_buffers=reference_buffers)
        self.gate_proj = TernaryLinear(self.hidden_size, self.intermediate_size, scale=scales[0], **kw)
        self.up_proj = TernaryLinear(self.hidden_size, self.intermediate_size, scale=scales[1], **kw)
        self.down_proj = TernaryLinear(self.intermediate_size, self.hidden_size, scale=scales[2], **kw)
        self.fused = fused and not config.mlp_bias
        self._packed: dict[int, PackedMLP] = {}

    def packed(self, device) -> PackedMLP:
        idx = device.index if device.index is not None else torch.cuda.current_device()
        pm = self._packed.get(idx)
        if pm is None:
            pm = PackedMLP(self.gate_proj.ternary_weight.numpy().astype(np.int8), self.up_proj.ternary_weight.numpy().astype(np.int8),
                           self.down_proj.ternary_weight.numpy().astype(np.int8), self.gate_proj.scale, self.up_proj.scale,
                           self.down_proj.scale, torch.device("cuda", idx))
            self._packed[idx] = pm
        return pm

    def forward(self, x):
        if not self.fused:
            return self.down_proj(torch.nn.functional.silu(self.gate_proj(x)) * self.up_proj(x))
        lead = tuple(x.shape[:-1])
        y = self.packed(x.device).forward(x.reshape(-1, self.hidden_size))
        return y.reshape(*lead, self.hidden_size)


__all__ = ["LlamaTernaryMLP"]
