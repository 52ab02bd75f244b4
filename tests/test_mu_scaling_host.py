"""Host-side pieces of the muS / FP8 interface that define the MINT-650M FP8 workload: `unit_variance_init_`,
`compute_tau`, `set_unit_output_scales`, `build_mint_mu(unit_scaled=True)`, `build_mint_fp8`, `build_checkpointed_model`,
the registry's shape limits.  No GPU.  Where the reference checkout is readable (the build container) its own functions
are imported and compared element for element under one seed; elsewhere those comparisons are skipped and the
closed-form checks remain."""
import importlib.util
import math
import os

import pytest
import torch
from torch import nn

import mint_plus_b200 as M
from mint_plus_b200 import esm2, mu_scaling

# the reference checkout, when it sits beside this repository (or where MINT_REFERENCE_ROOT points)
REF_ROOT = os.path.join(os.environ.get("MINT_REFERENCE_ROOT", os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "reference")),
                        "mint_plus", "models", "mu_scaling")


def _ref_module(name):
    """Import one file of the reference's mu_scaling package by path (its package __init__ pulls in GPU-only code)."""
    path = os.path.join(REF_ROOT, name + ".py")
    if not os.path.exists(path):
        pytest.skip("reference checkout not present")
    spec = importlib.util.spec_from_file_location("ref_mu_" + name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class _Tiny(nn.Module):
    def __init__(self):
        super().__init__()
        self.emb = nn.Embedding(33, 16, padding_idx=1)
        self.fc = nn.Linear(16, 48)
        self.nob = nn.Linear(48, 16, bias=False)
        self.ln = nn.LayerNorm(16)
        self.rms = nn.RMSNorm(16)


def test_unit_variance_init_equals_the_reference_function_under_one_seed():
    ref = _ref_module("init")
    a, b = _Tiny(), _Tiny()
    with torch.no_grad():
        for m in (a, b):
            m.ln.weight.fill_(3.0); m.ln.bias.fill_(2.0); m.rms.weight.fill_(5.0); m.fc.bias.fill_(1.0)
    torch.manual_seed(77)
    ref.unit_variance_init_(a)
    torch.manual_seed(77)
    M.unit_variance_init_(b)
    for (n, p), (_, q) in zip(a.state_dict().items(), b.state_dict().items()):
        assert torch.equal(p, q), n
    assert ref.unit_variance_output_multiplier(1280) == 1.0 / math.sqrt(1280)


def test_unit_variance_init_statistics_and_special_rows():
    torch.manual_seed(3)
    m = M.unit_variance_init_(_Tiny())
    assert m.emb.weight[1].abs().max() == 0                      # the padding row stays zero
    assert abs(m.fc.weight.std().item() - 1.0) < 0.1 and abs(m.fc.weight.mean().item()) < 0.1
    assert m.fc.bias.abs().max() == 0
    assert torch.equal(m.ln.weight, torch.ones(16)) and torch.equal(m.ln.bias, torch.zeros(16))
    assert torch.equal(m.rms.weight, torch.ones(16))
    f = mu_scaling.Fp8Linear(16, 8)                              # the swapped-in projection is initialised the same way
    M.unit_variance_init_(f)
    assert f.bias.abs().max() == 0 and f.weight.std() > 0.5


@pytest.mark.parametrize("L", [0, 1, 4, 30, 33, 100])
def test_compute_tau(L):
    assert M.compute_tau(L) == 0.5 / math.sqrt(max(1, L))
    if os.path.exists(REF_ROOT):
        assert _ref_module("optim").compute_tau(L) == M.compute_tau(L)


def test_build_mint_mu_unit_scaled_sets_tau_init_and_output_multipliers():
    torch.manual_seed(0)
    model = M.build_mint_mu("8M", use_fp8=True, unit_scaled=True)
    assert model._mu_config["tau"] == M.compute_tau(6) and model._mu_config["unit_scaled"]
    for layer in model.layers:
        assert isinstance(layer, M.TransformerLayer_MINT_mu) and not hasattr(layer, "self_attn_layer_norm")
        assert abs(float(layer._tau) - M.compute_tau(6)) < 1e-7
        for mod in (layer.self_attn.q_proj, layer.self_attn.out_proj, layer.multimer_attn.k_proj, layer.feed_forward.fc1):
            assert isinstance(mod, M.Fp8Linear) and mod.out_scale == 1.0 / math.sqrt(320)
        assert layer.feed_forward.fc2.out_scale == 1.0 / math.sqrt(1280)
        assert abs(layer.feed_forward.fc1.weight.std().item() - 1.0) < 0.05
    assert isinstance(model.lm_head.dense, nn.Linear) and isinstance(model.embed_tokens, nn.Embedding)   # left alone


def test_build_mint_fp8_is_the_pre_ln_model_with_fp8_projections_in_blocks():
    model = M.build_mint_fp8("8M", checkpoint_block_size=3)
    assert model._fp8_config == {"enabled": True, "static_scale": True} and model._checkpoint_block_size == 3
    assert len(model.layers) == 2 and all(isinstance(b, M.CheckpointedBlock) and len(b) == 3 for b in model.layers)
    for block in model.layers:
        for layer in block.layers:
            assert isinstance(layer, M.TransformerLayer_MINT) and layer._use_fused_multi_pathway
            assert isinstance(layer.self_attn_layer_norm, nn.LayerNorm)                  # Pre-LN, not muS
            for mod in (layer.self_attn.q_proj, layer.self_attn.k_proj, layer.self_attn.v_proj, layer.self_attn.out_proj,
                        layer.multimer_attn.q_proj, layer.feed_forward.fc1, layer.feed_forward.fc2):
                assert isinstance(mod, M.Fp8Linear) and mod.out_scale == 1.0
    # names are those of the plain model inside the blocks, so pre-trained weights map by name
    keys = set(model.state_dict())
    assert "layers.0.layers.0.self_attn.q_proj.weight" in keys and "layers.1.layers.2.feed_forward.fc2.bias" in keys
    flat = M.build_mint_fp8("8M", checkpoint_block_size=0)
    assert len(flat.layers) == 6 and "layers.5.self_attn.out_proj.weight" in flat.state_dict()
    with pytest.raises(ValueError):
        M.build_checkpointed_model(M.MINT(num_layers=4, embed_dim=32, attention_heads=2), block_size=3)


def test_registry_entries_outside_the_kernels_limits_fail_loudly():
    for size, cfg in M.MODEL_REGISTRY.items():
        head_dim = cfg["embed_dim"] // cfg["attention_heads"]
        ok = head_dim in M.SUPPORTED_HEAD_DIMS and cfg["embed_dim"] <= esm2.MAX_EMBED_DIM
        if ok:
            esm2.check_supported_shape(cfg["embed_dim"], cfg["attention_heads"])
        else:
            assert size in ("35M", "3B", "15B")          # head sizes 24, 112, 256
            with pytest.raises(NotImplementedError, match="head size"):
                M.MINT.from_config(size)
    assert M.MINT.from_config("8M").embed_dim == 320
