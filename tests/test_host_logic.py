"""Host-side mirror of the reference interface: module structure, state-dict keys, weight fusion, argument checks.
No GPU: nothing here launches a kernel."""
import pytest
import torch
from torch import nn

import mint_plus_b200 as M
from oracle import multimer_attention as O


class _OldLayer(nn.Module):
    """A layer with separate q/k/v projections, shaped like the reference's TransformerLayer_MINT."""

    def __init__(self, E, H):
        super().__init__()
        self.embed_dim, self.ffn_embed_dim, self.attention_heads = E, 4 * E, H
        self.use_rotary_embeddings, self.use_multimer, self.use_erf_gelu = True, True, True
        self.self_attn = M.MultiHeadAttention(E, H, use_rotary_embeddings=True)
        self.multimer_attn = M.MultiHeadAttention(E, H, use_rotary_embeddings=False, no_proj=True)
        self.feed_forward = M.VanillaFeedForward(E, 4 * E, use_erf_gelu=True)
        self.self_attn_layer_norm = nn.LayerNorm(E)
        self.final_layer_norm = nn.LayerNorm(E)


class _Model(nn.Module):
    def __init__(self, E=32, H=2, L=2):
        super().__init__()
        self.layers = nn.ModuleList([_OldLayer(E, H) for _ in range(L)])


def test_state_dict_keys_follow_the_reference_names():
    layer = M.TransformerLayer_MINT_plus(32, 128, 2, use_multimer=True, use_erf_gelu=True)
    keys = set(layer.state_dict())
    for k in ("self_attn.fused_qkv.weight", "self_attn.fused_qkv.bias", "self_attn.out_proj.weight",
              "self_attn.rot_emb.inv_freq", "multimer_attn.fused_qkv.weight", "feed_forward.fc1.weight",
              "feed_forward.fc2.bias", "self_attn_layer_norm.weight", "final_layer_norm.bias"):
        assert k in keys, k
    sep = M.MultiHeadAttention(32, 2, use_rotary_embeddings=True)
    assert {"q_proj.weight", "k_proj.weight", "v_proj.weight", "out_proj.weight", "rot_emb.inv_freq"} <= set(sep.state_dict())
    assert M.MultiHeadAttention(32, 2, no_proj=True).out_proj is None


def test_build_mint_plus_concatenates_qkv_and_shares_the_rest():
    torch.manual_seed(0)
    model = _Model()
    old = model.layers[0]
    M.build_mint_plus(model)
    new = model.layers[0]
    assert isinstance(new, M.TransformerLayer_MINT_plus)
    w = torch.cat([old.self_attn.q_proj.weight, old.self_attn.k_proj.weight, old.self_attn.v_proj.weight], 0)
    assert torch.equal(new.self_attn.fused_qkv.weight, w)
    wc = torch.cat([old.multimer_attn.q_proj.weight, old.multimer_attn.k_proj.weight, old.multimer_attn.v_proj.weight], 0)
    assert torch.equal(new.multimer_attn.fused_qkv.weight, wc)
    assert new.self_attn.out_proj is old.self_attn.out_proj
    assert new.self_attn.rot_emb is old.self_attn.rot_emb
    assert new.feed_forward is old.feed_forward and new.final_layer_norm is old.final_layer_norm
    # projections agree with the separate ones
    x = torch.randn(5, 2, 32)
    q, k, v = new.self_attn.project_qkv_4d(x)
    q0, k0, v0 = old.self_attn.project_qkv_4d(x)
    torch.testing.assert_close(q, q0)
    torch.testing.assert_close(v, v0)


def test_enable_fused_multi_pathway_reaches_wrapped_layers():
    model = _Model()
    M.build_mint_plus(model)

    class Block(nn.Module):
        def __init__(self, layers):
            super().__init__()
            self.layers = nn.ModuleList(layers)

    model.layers = nn.ModuleList([Block([model.layers[0]]), model.layers[1]])
    M.enable_fused_multi_pathway(model, False)
    assert model.layers[0].layers[0]._use_fused_multi_pathway is False
    assert model.layers[1]._use_fused_multi_pathway is False


def test_before_softmax_contract_matches_the_oracle_logits():
    torch.manual_seed(1)
    E, H, T, B = 32, 2, 12, 2
    sa = M.MultiHeadAttention(E, H, use_rotary_embeddings=True)
    ma = M.MultimerAttention(E, H)
    x = torch.randn(T, B, E)
    pad = torch.zeros(B, T, dtype=torch.bool)
    pad[0, -2:] = True
    il, iv = sa(x, key_padding_mask=pad, before_softmax=True)
    el, ev = ma(x, key_padding_mask=pad, before_softmax=True)
    q_s, k_s, v_s = sa.project_qkv_4d(x)
    q_c, k_c, v_c = ma.project_qkv_4d(x)
    none = torch.zeros(B, T, T, dtype=torch.bool)
    torch.testing.assert_close(il, O.combined_logits(q_s, k_s, q_c, k_c, none, pad), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(el, O.combined_logits(q_s, k_s, q_c, k_c, ~none, pad), rtol=1e-5, atol=1e-6)
    assert torch.equal(iv, v_s) and torch.equal(ev, v_c)
    assert torch.isinf(il[0, :, :, -2:]).all()


def test_cpu_tensors_are_refused():
    t = torch.zeros(1, 1, 8, 16)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        M.multimer_attention(t, t, t, t, t, t, chain_ids=torch.zeros(1, 8, dtype=torch.int32))
    with pytest.raises(NotImplementedError):
        M.fused_multi_pathway_attention(t, t, t, t, t, t, torch.zeros(1, 8, 8, dtype=torch.bool), dropout_p=0.1)


def test_pack_info_lists_unpadded_rows_in_sequence_first_order():
    from mint_plus_b200.ops import PackInfo
    pad = torch.tensor([[False, False, True, True], [False, True, True, True], [False, False, False, True]])   # (B=3, T=4)
    pk = PackInfo(pad)
    # row = t * B + b over the (T, B) grid of the layer's activations
    assert pk.rows64.tolist() == [0, 1, 2, 3, 5, 8] and pk.rows32.dtype == torch.int32
    assert (pk.T, pk.B, pk.n) == (4, 3, 6)


def test_pack_padding_refuses_cpu_tensors():
    model = M.MINT(num_layers=1, embed_dim=32, attention_heads=2, use_multimer=True).eval()
    model.pack_padding = True
    tokens = torch.tensor([[0, 5, 6, 2, 1, 1]])
    with pytest.raises(NotImplementedError):
        model(tokens, torch.zeros_like(tokens))


def test_benchmark_input_generator_draws_the_oracle_generators_numbers():
    """bench.py carries its own copy of the seeded input generator (its measured arm imports nothing from oracle/)."""
    import bench
    a = bench.make_op_inputs(2, 3, 256, 32, seed=2002)
    b = O.make_op_inputs(2, 3, 256, 32, seed=2002)
    for x, y in zip(a[0], b[0]):
        assert torch.equal(x, y)
    assert torch.equal(a[1], b[1]) and torch.equal(a[2], b[2]) and torch.equal(a[3], b[3])


def test_rotary_frequencies_stay_fp32_through_a_model_cast():
    rot = M.RotaryEmbedding(64)
    want = rot.inv_freq.clone()
    rot = rot.to(torch.bfloat16)
    assert rot.inv_freq.dtype == torch.float32 and torch.equal(rot.inv_freq, want)
    layer = M.TransformerLayer_MINT_plus(128, 512, 2, use_multimer=True).to(torch.bfloat16)
    assert layer.self_attn.rot_emb.inv_freq.dtype == torch.float32
    assert layer.self_attn.out_proj.weight.dtype == torch.bfloat16
    assert "self_attn.rot_emb.inv_freq" in layer.state_dict()


def test_e4m3_copy_rides_on_the_tensor_and_expires_when_it_is_written():
    from mint_plus_b200 import ops
    t = torch.zeros(6, 2, 8)
    q8 = torch.zeros(12, 8, dtype=torch.uint8)
    ops.attach_e4m3(t, q8, 0.5)
    assert ops.e4m3_of(t, 0.5).data_ptr() == q8.data_ptr() and tuple(ops.e4m3_of(t, 0.5).shape) == (12, 8)
    with pytest.raises(RuntimeError):           # another scale: a cast pass is needed, and that runs on CUDA tensors only
        ops.e4m3_of(t, 1.0)
    t.add_(1.0)                                 # written since: the copy no longer describes it
    with pytest.raises(RuntimeError):
        ops.e4m3_of(t, 0.5)


def test_gelu_polynomial_of_the_gemm_epilogue_matches_erf_gelu():
    """The projection epilogue computes erf-GELU as max(x, 0) - a 2^s(a), a = min(|x|, 5.75), with a degree-6 polynomial s.
    The coefficients are read from the CUDA source and the formula is evaluated here in fp32 steps (Horner form, as the
    kernel does) against x/2 (1 + erf(x / sqrt 2)) in fp64: the absolute error stays below 1e-6 everywhere, which is the
    accuracy the formula it replaced had (gelu_erf of mint_plus/models/modules.py:16-23 is the function approximated)."""
    import os
    import re
    src = open(os.path.join(os.path.dirname(os.path.abspath(M.__file__)), "csrc", "gemm_tc.cu")).read()
    body = src[src.index("void gelu_erf2("):]
    body = body[:body.index("ex2.approx")]
    coef = [float(c) for c in re.findall(r"pack2\((-?[0-9.]+e[-+][0-9]+)f,", body)]
    assert len(coef) == 7, coef                     # c6 first, then c5 ... c0 (Horner order)
    clamp = float(re.search(r"fminf\(fabsf\(x0\), ([0-9.]+)f\)", body).group(1))
    x = torch.cat([torch.linspace(-12, 12, 200001, dtype=torch.float64), torch.randn(200000, dtype=torch.float64) * 1.5])
    xf = x.float()
    a = xf.abs().clamp(max=clamp)
    s = torch.full_like(a, coef[0])
    for c in coef[1:]:
        s = s * a + torch.tensor(c, dtype=torch.float32)   # one rounding per step (the kernel's FMA rounds once as well)
    got = (torch.clamp(xf, min=0) - a * torch.exp2(s.double()).float()).double()
    want = 0.5 * x * (1.0 + torch.erf(x / 2.0 ** 0.5))
    err = (got - want).abs()
    assert err.max().item() < 1e-6, err.max().item()
    big = want.abs() >= 1e-3
    assert (err[big] / want[big].abs()).max().item() < 1e-4
