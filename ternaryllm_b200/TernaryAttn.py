"""LlamaTernaryAttention: ternary q / k / v / o projections around a stock attention core
(ternaryLLM_GPU/TernaryLLM/TernaryAttn.py:15-120).

Same constructor arguments and sub-module names (`q_proj`, `k_proj`, `v_proj`, `o_proj`).  Only the four linears
are this library's work; rotary embedding, softmax and the value product are plain PyTorch, as in the reference
(whose attention core is the eager Hugging Face code, :96-112).  Differences a user will notice:

* the three input projections run as **one** product on a packed weight whose columns are q | k | v (`fused_qkv`,
  default on; the reference issues three calls, :73-75) -- bias-free projections only;
* the attention core is `scaled_dot_product_attention` (same arithmetic up to summation order), causal when no mask
  is given and more than one query position is passed;
* the key / value cache is a plain `(k, v)` tuple passed in and returned, not a transformers `Cache` object;
* rotary position embeddings are applied only when `position_embeddings=(cos, sin)` is passed; no rotary module is
  instantiated here.
"""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np
import torch
from torch import nn

from .configuration_ternary import TernaryConfig
from .TernaryLinear import TernaryLinear
from .weight import PackedWeight


def _rotate_half(x):
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


class LlamaTernaryAttention(nn.Module):
    def __init__(self, config: TernaryConfig, layer_idx: Optional[int] = None, scales=(1.0, 1.0, 1.0, 1.0), fused_qkv: bool = True,
                 generator=None, reference_buffers: bool = False):
        super().__init__()
        self.config = config
        self.layer_idx = layer_idx
        self.attention_dropout = config.attention_dropout
        self.hidden_size = config.hidden_size
        self.num_heads = config.num_attention_heads
        self.head_dim = config.head_dim
        self.num_key_value_heads = config.num_key_value_heads
        self.num_key_value_groups = self.num_heads // self.num_key_value_heads
        self.is_causal = True
        kw = dict(sparsity=config.sparsity, uniform=config.uniform_sparsity, uniform_blk_size=config.uniform_sparsity_block_size,
                  padding=config.padding, padding_size=config.padding_size, bias=config.attention_bias, generator=generator,
                  reference_buffers=reference_buffers)
        self.q_proj = TernaryLinear(self.hidden_size, self.num_heads * self.head_dim, scale=scales[0], **kw)
        self.k_proj = TernaryLinear(self.hidden_size, self.num_key_value_heads * self.head_dim, scale=scales[1], **kw)
        self.v_proj = TernaryLinear(self.hidden_size, self.num_key_value_heads * self.head_dim, scale=scales[2], **kw)
        self.o_proj = TernaryLinear(self.num_heads * self.head_dim, self.hidden_size, scale=scales[3], **kw)
        # one product for q | k | v needs one scale for the three of them
        self.fused_qkv = fused_qkv and not config.attention_bias and scales[0] == scales[1] == scales[2]
        self._qkv: dict[int, PackedWeight] = {}

    def packed_qkv(self, device) -> PackedWeight:
        idx = device.index if device.index is not None else torch.cuda.current_device()
        pw = self._qkv.get(idx)
        if pw is None:
            w = np.concatenate([p.ternary_weight.numpy().astype(np.int8) for p in (self.q_proj, self.k_proj, self.v_proj)], axis=1)
            pw = PackedWeight.from_dense(np.ascontiguousarray(w), self.q_proj.scale, torch.device("cuda", idx))
            self._qkv[idx] = pw
        return pw

    def forward(self, hidden_states: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                position_embeddings: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                past_key_value: Optional[Tuple[torch.Tensor, torch.Tensor]] = None, use_cache: bool = False, **kwargs):
        bsz, q_len, _ = hidden_states.shape
        nq, nkv = self.num_heads * self.head_dim, self.num_key_value_heads * self.head_dim
        if self.fused_qkv:
            qkv = self.packed_qkv(hidden_states.device).matmul(hidden_states.reshape(bsz * q_len, self.hidden_size))
            q, k, v = qkv.split([nq, nkv, nkv], dim=1)
        else:
            q, k, v = self.q_proj(hidden_states), self.k_proj(hidden_states), self.v_proj(hidden_states)
        q = q.reshape(bsz, q_len, self.num_heads, self.head_dim).transpose(1, 2)
        k = k.reshape(bsz, q_len, self.num_key_value_heads, self.head_dim).transpose(1, 2)
        v = v.reshape(bsz, q_len, self.num_key_value_heads, self.head_dim).transpose(1, 2)
        if position_embeddings is not None:
            cos, sin = (t.unsqueeze(1) for t in position_embeddings)      # [bsz, 1, q_len, head_dim]
            q, k = q * cos + _rotate_half(q) * sin, k * cos + _rotate_half(k) * sin
        if past_key_value is not None:
            k, v = torch.cat([past_key_value[0], k], dim=2), torch.cat([past_key_value[1], v], dim=2)
        present = (k, v) if use_cache else None
        if attention_mask is not None:
            attention_mask = attention_mask[:, :, :, : k.shape[-2]]
        out = nn.functional.scaled_dot_product_attention(
            q, k, v, attn_mask=attention_mask, dropout_p=self.attention_dropout if self.training else 0.0,
            is_causal=attention_mask is None and q_len > 1 and past_key_value is None, enable_gqa=self.num_key_value_groups > 1)
        out = out.transpose(1, 2).reshape(bsz, q_len, nq)
        return self.o_proj(out), None, present


__all__ = ["LlamaTernaryAttention"]
