"""TernaryConfig: the fields the reference adds to a Llama configuration
(ternaryLLM_GPU/TernaryLLM/configuration_ternary.py:28-47), as a plain dataclass.

The reference derives from transformers' LlamaConfig; only the sizes and the ternary switches matter to the
ternary linears, so this class carries those and nothing of the tokenizer / generation machinery.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class TernaryConfig:
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int | None = None
    hidden_act: str = "silu"
    max_position_embeddings: int = 2048
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    attention_bias: bool = False
    attention_dropout: float = 0.0
    mlp_bias: bool = False
    head_dim: int | None = None
    ternary_attn_linear: bool = True
    ternary_mlp: bool = True
    sparsity: float = 0.8
    uniform_sparsity: bool = False
    uniform_sparsity_block_size: int = 512
    padding: bool = False
    padding_size: int = 4

    def __post_init__(self):
        if self.num_key_value_heads is None:
            self.num_key_value_heads = self.num_attention_heads
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.num_attention_heads


__all__ = ["TernaryConfig"]
