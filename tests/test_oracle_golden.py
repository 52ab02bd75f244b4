"""The CPU oracle against the vectors produced by the reference's own PyTorch modules."""
import pytest
import torch

from conftest import golden_cases, load_golden
from oracle import multimer_attention as O


@pytest.mark.parametrize("name", golden_cases())
def test_oracle_matches_reference_vectors(name):
    g = load_golden(name)
    mask = O.chain_mask_from_ids(g["chain_ids"])
    out, grads = O.multimer_attention_fwd_bwd(
        g["q_s"], g["k_s"], g["v_s"], g["q_c"], g["k_c"], g["v_c"], mask, g["grad_out"],
        key_pad=g["key_pad"], rope=True, sqrt_softmax=bool(g["sqrt_softmax"]))
    # fp32 on both sides, same operation order up to the reference's (T,B,E) layout: 1e-5 relative
    torch.testing.assert_close(out, g["out"], rtol=1e-5, atol=1e-6)
    for got, key in zip(grads, ("dq_s", "dk_s", "dv_s", "dq_c", "dk_c", "dv_c")):
        torch.testing.assert_close(got, g[key], rtol=1e-4, atol=2e-6, msg=lambda m: f"{key}: {m}")


def test_projection_matches_reference_vectors():
    g = load_golden("attn_d32_two_chain")
    H = g["q_c"].shape[1]
    q, k, v = O.project_qkv_4d(g["x"], g["w_qkv_c"], g["b_qkv_c"], H)
    torch.testing.assert_close(q, g["q_c"], rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(k, g["k_c"], rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(v, g["v_c"], rtol=1e-5, atol=1e-5)


def test_padded_keys_get_zero_probability_and_pad_queries_are_ordinary_rows():
    (qs, ks, vs, qc, kc, vc), cid, pad, _ = O.make_op_inputs(2, 2, 64, 16, seed=5, max_pad=8)
    pad[0, -5:] = True
    mask = O.chain_mask_from_ids(cid)
    out = O.multimer_attention(qs, ks, vs, qc, kc, vc, mask, pad)
    vs2, vc2 = vs.clone(), vc.clone()
    vs2[0, :, -5:] = 1e6
    vc2[0, :, -5:] = 1e6
    out2 = O.multimer_attention(qs, ks, vs2, qc, kc, vc2, mask, pad)
    assert torch.equal(out, out2)                     # padded keys never contribute, bit-exactly
    assert torch.isfinite(out[0, :, -5:]).all()       # padded query rows still attend to real keys


def test_combine_from_logits_equals_fused_path():
    (qs, ks, vs, qc, kc, vc), cid, pad, _ = O.make_op_inputs(1, 2, 48, 16, seed=6, max_pad=4)
    mask = O.chain_mask_from_ids(cid)
    D = qs.shape[-1]
    intra = torch.matmul(O.apply_rope(qs * D ** -0.5), O.apply_rope(ks).transpose(-1, -2))
    inter = torch.matmul(qc * D ** -0.5, kc.transpose(-1, -2))
    intra = intra.masked_fill(pad[:, None, None, :], float("-inf"))
    inter = inter.masked_fill(pad[:, None, None, :], float("-inf"))
    a = O.combine_from_logits(intra, inter, mask, vs, vc)
    b = O.multimer_attention(qs, ks, vs, qc, kc, vc, mask, pad)
    torch.testing.assert_close(a, b, rtol=1e-6, atol=1e-7)
