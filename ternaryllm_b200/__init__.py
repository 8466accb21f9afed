"""ternaryllm_b200 -- B200-native ternary sparse product Y = X.W.s behind the reference's operator API.

Host side of libtllm.so (C ABI in include/tllm.h): the `ter_spmm` module functions, `TernaryLinear`,
`LlamaTernaryMLP`, `TernaryConfig`, and the handle wrappers `PackedWeight` / `PackedMLP`.
"""
from . import ter_spmm
from .configuration_ternary import TernaryConfig
from .TernaryLinear import TernaryLinear, convert_ternary_weights, random_ternary_weights
from .TernaryMLP import LlamaTernaryMLP
from .weight import PackedMLP, PackedWeight

__all__ = ["ter_spmm", "TernaryConfig", "TernaryLinear", "LlamaTernaryMLP", "PackedWeight", "PackedMLP",
           "convert_ternary_weights", "random_ternary_weights"]
