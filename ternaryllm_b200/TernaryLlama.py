"""Model surgery of the reference (ternaryLLM_GPU/TernaryLLM/TernaryLlama.py:10-34, :69-76): find the
`nn.Linear` modules of a Llama-style model that the configuration marks as ternary, put a `TernaryLinear` in
the place of each, and move the model to the GPU.

Same three names and argument order, so the reference's benchmark script keeps working
(benchmark_ternary_llama.py:48 calls `prepare_ternary_model(model, config)`).  Selection is by module name,
as there: `q_proj`/`k_proj`/`v_proj`/`o_proj` when `config.ternary_attn_linear`, anything under `mlp` when
`config.ternary_mlp` (a module that matches both is listed once; the reference lists it twice and builds it
twice).

Added: `from_float=True` ternarises each layer's own weight (threshold rule, per-tensor scale) instead of
drawing a random ternary matrix as the reference does; `reference_buffers=False` skips building the
reference-layout index buffers nobody reads on this path; `verbose` replaces the reference's unconditional
prints.  Works on any `nn.Module` tree -- transformers is not imported.
"""
from __future__ import annotations

import torch
from torch import nn

from .TernaryLinear import TernaryLinear

_ATTN_NAMES = ("q_proj", "k_proj", "v_proj", "o_proj")


def collect_linear_layers(model: nn.Module, config) -> list[tuple[str, nn.Linear]]:
    """[(qualified name, module)] of the `nn.Linear` modules to replace, in `named_modules()` order."""
    out = []
    for name, module in model.named_modules():
        if not isinstance(module, nn.Linear):
            continue
        attn = bool(getattr(config, "ternary_attn_linear", True)) and any(k in name for k in _ATTN_NAMES)
        mlp = bool(getattr(config, "ternary_mlp", True)) and "mlp" in name
        if attn or mlp:
            out.append((name, module))
    return out


def replace_linear_layers(layers, model: nn.Module, config, from_float: bool = False, reference_buffers: bool = True,
                          verbose: bool = False, generator: torch.Generator | None = None) -> None:
    """Replaces every listed module in `model` by a bias-free `TernaryLinear` of the same shape, built on the
    CPU (TernaryLlama.py:21-34).  With `from_float` the new layer holds the ternarised weight of the module it
    replaces and its scale; a bias of that module is carried over."""
    for name, module in layers:
        parent_name, _, attr = name.rpartition(".")
        parent = model.get_submodule(parent_name) if parent_name else model
        if from_float:
            layer = TernaryLinear.from_float(module.weight, sparsity=getattr(config, "sparsity", None), bias=module.bias is not None,
                                             padding=False, device="cpu", reference_buffers=reference_buffers)
            if module.bias is not None:
                with torch.no_grad():
                    layer.bias.copy_(module.bias.detach().float())
        else:
            layer = TernaryLinear(module.in_features, module.out_features, sparsity=config.sparsity,
                                  uniform=config.uniform_sparsity, uniform_blk_size=config.uniform_sparsity_block_size,
                                  padding=False, bias=False, device="cpu", reference_buffers=reference_buffers,
                                  generator=generator)
        if verbose:
            print(f"{name}: {module} -> {layer}")
        setattr(parent, attr, layer)


def prepare_ternary_model(model: nn.Module, config, device="cuda", **kw) -> nn.Module:
    """collect + replace on the CPU, then `model.to(device)` (TernaryLlama.py:69-76).  The packed weights are
    built on first use on the device the activations live on."""
    model.to("cpu")
    replace_linear_layers(collect_linear_layers(model, config), model, config, **kw)
    model.to(device)
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
    return model


__all__ = ["collect_linear_layers", "replace_linear_layers", "prepare_ternary_model"]
