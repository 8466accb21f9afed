"""ternaryllm_b200 -- B200-native ternary sparse product Y = X.W.s behind the reference's operator API.

Host side of libtllm.so (C ABI in include/tllm.h): the `ter_spmm` module functions, `TernaryLinear`,
`LlamaTernaryMLP`, `LlamaTernaryAttention`, `TernaryConfig`, the model surgery of `TernaryLlama`, the handle wrappers `PackedWeight` / `PackedMLP`, and the
tensor-parallel pieces of `tensor_parallel`.
"""
from . import ter_spmm
from .configuration_ternary import TernaryConfig
from .TernaryLinear import TernaryLinear, convert_ternary_weights, random_ternary_weights, ternarize_weights
from .TernaryAttn import LlamaTernaryAttention
from .TernaryMLP import LlamaTernaryMLP
from .TernaryLlama import collect_linear_layers, prepare_ternary_model, replace_linear_layers
from .tensor_parallel import ColumnParallelTernaryLinear, RowParallelTernaryLinear, TernaryDecoderLayerTP
from .weight import PackedMLP, PackedWeight, ternarize

__all__ = ["ter_spmm", "TernaryConfig", "TernaryLinear", "LlamaTernaryMLP", "LlamaTernaryAttention", "PackedWeight", "PackedMLP",
           "ColumnParallelTernaryLinear", "RowParallelTernaryLinear", "TernaryDecoderLayerTP",
           "collect_linear_layers", "replace_linear_layers", "prepare_ternary_model",
           "convert_ternary_weights", "random_ternary_weights", "ternarize_weights", "ternarize"]
