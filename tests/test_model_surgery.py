"""collect_linear_layers / replace_linear_layers / prepare_ternary_model against the behaviour of the
reference's functions of those names (ternaryLLM_GPU/TernaryLLM/TernaryLlama.py:10-34, :69-76)."""
import numpy as np
import pytest
import torch
from torch import nn

from ternaryllm_b200 import (TernaryConfig, TernaryLinear, collect_linear_layers, prepare_ternary_model,
                             replace_linear_layers)


class _Attn(nn.Module):
    def __init__(self, h):
        super().__init__()
        self.q_proj, self.k_proj, self.v_proj, self.o_proj = (nn.Linear(h, h, bias=False) for _ in range(4))


class _Mlp(nn.Module):
    def __init__(self, h, i):
        super().__init__()
        self.gate_proj, self.up_proj, self.down_proj = nn.Linear(h, i, bias=False), nn.Linear(h, i, bias=False), nn.Linear(i, h, bias=False)

    def forward(self, x):
        return self.down_proj(nn.functional.silu(self.gate_proj(x)) * self.up_proj(x))


class _Layer(nn.Module):
    def __init__(self, h, i):
        super().__init__()
        self.self_attn, self.mlp, self.input_layernorm = _Attn(h), _Mlp(h, i), nn.LayerNorm(h)


class _Model(nn.Module):
    def __init__(self, h=64, i=96, layers=2):
        super().__init__()
        self.layers = nn.ModuleList(_Layer(h, i) for _ in range(layers))
        self.lm_head = nn.Linear(h, 100, bias=False)


def test_collect_follows_the_configuration_switches():
    m = _Model()
    names = [n for n, _ in collect_linear_layers(m, TernaryConfig())]
    assert names == [f"layers.{l}.{p}" for l in range(2) for p in
                     ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
                      "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj")]
    only_mlp = [n for n, _ in collect_linear_layers(m, TernaryConfig(ternary_attn_linear=False))]
    assert only_mlp == [n for n in names if ".mlp." in n]
    only_attn = [n for n, _ in collect_linear_layers(m, TernaryConfig(ternary_mlp=False))]
    assert only_attn == [n for n in names if "self_attn" in n]
    assert collect_linear_layers(m, TernaryConfig(ternary_mlp=False, ternary_attn_linear=False)) == []


def test_replace_builds_random_ternary_layers_of_the_same_shape():
    m = _Model()
    cfg = TernaryConfig(sparsity=0.75)
    layers = collect_linear_layers(m, cfg)
    replace_linear_layers(layers, m, cfg, generator=torch.Generator().manual_seed(1))
    for name, old in layers:
        new = m.get_submodule(name)
        assert isinstance(new, TernaryLinear) and new.bias is None
        assert (new.in_features, new.out_features) == (old.in_features, old.out_features)
        w = new.ternary_weight
        assert tuple(w.shape) == (old.in_features, old.out_features) and set(w.unique().tolist()) <= {-1, 0, 1}
        assert abs(float((w == 0).float().mean()) - 0.75) < 0.06
        # the reference-layout buffers are there for code that inspects them (TernaryLinear.py:150-152)
        assert new.w_row_indices.dtype == torch.int16 and new.w_col_offsets.numel() % 4 == 0
    assert isinstance(m.lm_head, nn.Linear) and isinstance(m.layers[0].input_layernorm, nn.LayerNorm)


def test_replace_from_float_keeps_the_sign_pattern_and_a_scale():
    m = _Model(layers=1)
    cfg = TernaryConfig(sparsity=0.5)
    old = m.layers[0].mlp.up_proj.weight.detach().clone()      # [out, in]
    replace_linear_layers(collect_linear_layers(m, cfg), m, cfg, from_float=True, reference_buffers=False)
    new = m.layers[0].mlp.up_proj
    t = new.ternary_weight.t().float()
    assert torch.all((t == 0) | (torch.sign(old) == t))
    assert abs(float((t == 0).float().mean()) - 0.5) < 0.02
    kept = old.abs()[t != 0]
    assert new.scale == pytest.approx(float(kept.mean()), rel=1e-5)
    assert float(kept.min()) >= float(old.abs()[t == 0].max())
    assert new.w_row_indices.numel() == 0


@pytest.mark.gpu
def test_prepared_model_runs_the_mlp_on_the_packed_kernel():
    from ternaryllm_b200 import _lib

    torch.manual_seed(0)
    m = _Model(h=256, i=512, layers=1)
    ref = _Model(h=256, i=512, layers=1)
    ref.load_state_dict(m.state_dict())
    cfg = TernaryConfig(sparsity=0.6)
    m = prepare_ternary_model(m, cfg, device="cuda", from_float=True, reference_buffers=False)
    mlp, rmlp = m.layers[0].mlp, ref.layers[0].mlp
    for name in ("gate_proj", "up_proj", "down_proj"):
        t = getattr(mlp, name)
        with torch.no_grad():
            getattr(rmlp, name).weight.copy_(t.ternary_weight.t().float() * t.scale)
    x = torch.randn(5, 256)
    before = _lib.lib().tllm_launch_count()
    y = mlp(x.cuda())
    assert _lib.lib().tllm_launch_count() >= before + 3
    want = rmlp.double()(x.double())
    assert float((y.detach().double().cpu() - want.detach()).abs().max()) <= 1e-4 * float(want.detach().abs().max())
