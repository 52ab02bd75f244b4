"""Generate the golden vectors under tests/golden/ from the reference's own PyTorch modules.

Run in a container where the reference checkout is importable:

    python tests/golden/make_golden.py --reference <path to the mint_plus checkout>

It instantiates the reference's `TransformerLayer_MINT_mu` (whose `_multimer_attention` is the
fp32-softmax statement of the combined-softmax attention, mint_plus/models/mu_scaling/layer.py:126-179),
replaces `self_attn.out_proj` by the identity so the attention output itself is returned, captures the
q/k/v projection outputs with forward hooks (so gradients w.r.t. them come from torch.autograd through
the reference code), and stores inputs, outputs and gradients as small .npz files.  A second family of
cases runs the reference's `MultimerAttention` (fused QKV) for the cross pathway, as `_plus` models do
(mint_plus/models/attention.py:263-371).  The test-suite only reads the .npz files.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _masks(kind, B, T, g):
    chain_ids = torch.zeros(B, T, dtype=torch.int32)
    pad = torch.zeros(B, T, dtype=torch.bool)
    if kind == "two_chain_tail_pad":
        for b in range(B):
            s = int(torch.randint(T // 4, 3 * T // 4, (1,), generator=g))
            chain_ids[b, s:] = 1
            p = int(torch.randint(0, T // 6 + 1, (1,), generator=g))
            if p:
                pad[b, T - p:] = True
    elif kind == "mid_pad":            # pads between the chains, as the reference CollateFn produces
        for b in range(B):
            s = T // 2
            chain_ids[b, s:] = 1
            p1 = int(torch.randint(1, T // 8 + 1, (1,), generator=g))
            p2 = int(torch.randint(1, T // 8 + 1, (1,), generator=g))
            pad[b, s - p1:s] = True
            pad[b, T - p2:] = True
    elif kind == "single_chain":
        pass
    elif kind == "two_chain_no_pad":   # sqrt-softmax: the reference's autograd gives NaN grads once a key has p = 0
        for b in range(B):
            chain_ids[b, int(torch.randint(T // 4, 3 * T // 4, (1,), generator=g)):] = 1
    elif kind == "three_chain":
        chain_ids[:, T // 3:] = 1
        chain_ids[:, 2 * T // 3:] = 2
        pad[:, T - 3:] = True
    elif kind == "alternating":        # every key tile is mixed
        chain_ids[:, 1::2] = 1
    else:
        raise ValueError(kind)
    return chain_ids, pad


def run_case(name, B, H, T, D, mask_kind, sqrt_softmax, plus, seed):
    from mint_plus.models.mu_scaling.layer import TransformerLayer_MINT_mu
    from mint_plus.models.attention import MultimerAttention

    torch.manual_seed(seed)
    g = torch.Generator().manual_seed(seed + 1)
    E = H * D
    layer = TransformerLayer_MINT_mu(E, 4 * E, H, use_rotary_embeddings=True, use_multimer=True,
                                     use_erf_gelu=True, num_layers=6, use_sqrt_softmax=sqrt_softmax)
    if plus:
        layer.multimer_attn = MultimerAttention(E, H)
    layer = layer.float().eval()
    layer.self_attn.out_proj = torch.nn.Identity()
    # biases are zero-initialised by the reference; make them matter
    for p_name, p in layer.named_parameters():
        if p_name.endswith("bias") and ("self_attn" in p_name or "multimer_attn" in p_name):
            p.data = 0.1 * torch.randn(p.shape, generator=g)

    captured = {}

    def hook(key):
        def fn(_mod, _inp, out):
            out.retain_grad()
            captured[key] = out
        return fn

    sa, ma = layer.self_attn, layer.multimer_attn
    sa.q_proj.register_forward_hook(hook("q_s"))
    sa.k_proj.register_forward_hook(hook("k_s"))
    sa.v_proj.register_forward_hook(hook("v_s"))
    if plus:
        ma.fused_qkv.register_forward_hook(hook("qkv_c"))
    else:
        ma.q_proj.register_forward_hook(hook("q_c"))
        ma.k_proj.register_forward_hook(hook("k_c"))
        ma.v_proj.register_forward_hook(hook("v_c"))

    x = (2.0 * torch.randn(T, B, E, generator=g)).requires_grad_(True)
    chain_ids, pad = _masks(mask_kind, B, T, g)
    chain_mask = ~torch.eq(chain_ids.unsqueeze(-1), chain_ids.unsqueeze(-2))

    out_tbe, _ = layer._multimer_attention(x, chain_mask, pad)          # (T, B, E) through identity out_proj
    grad_tbe = torch.randn(T, B, E, generator=g)
    out_tbe.backward(grad_tbe)

    def to4d(t):                                                          # (T,B,E) -> (B,H,T,D)
        return t.detach().reshape(T, B, H, D).permute(1, 2, 0, 3).contiguous()

    if plus:
        qkv, dqkv = captured["qkv_c"], captured["qkv_c"].grad
        for i, k in enumerate(("q_c", "k_c", "v_c")):
            captured[k] = qkv[..., i * E:(i + 1) * E]
            captured["d" + k] = dqkv[..., i * E:(i + 1) * E]
    arrays = {}
    for k in ("q_s", "k_s", "v_s", "q_c", "k_c", "v_c"):
        arrays[k] = to4d(captured[k]).numpy()
        gk = captured.get("d" + k)
        arrays["d" + k] = to4d(gk if gk is not None else captured[k].grad).numpy()
    arrays["out"] = to4d(out_tbe).numpy()
    arrays["grad_out"] = to4d(grad_tbe).numpy()
    arrays["chain_ids"] = chain_ids.numpy()
    arrays["key_pad"] = pad.numpy()
    arrays["sqrt_softmax"] = np.array(int(sqrt_softmax))
    # keep a projection-level record too: x and the fused cross-pathway weights
    if plus:
        arrays["x"] = x.detach().numpy()
        arrays["w_qkv_c"] = ma.fused_qkv.weight.detach().numpy()
        arrays["b_qkv_c"] = ma.fused_qkv.bias.detach().numpy()
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **{k: (v.astype(np.float32) if v.dtype == np.float64 else v) for k, v in arrays.items()})
    print(f"{name}: B{B} H{H} T{T} D{D} {mask_kind} sqrt={sqrt_softmax} plus={plus} -> {os.path.getsize(path)/1024:.0f} KiB")


CASES = [
    # name,                 B, H, T,   D,  masks,                 sqrt,  plus, seed
    ("attn_d16_two_chain",   2, 2, 72,  16, "two_chain_tail_pad",  False, False, 11),
    ("attn_d32_two_chain",   2, 2, 100, 32, "two_chain_tail_pad",  False, True,  12),
    ("attn_d64_mid_pad",     1, 2, 96,  64, "mid_pad",             False, True,  13),
    ("attn_d32_single",      1, 2, 64,  32, "single_chain",        False, False, 14),
    ("attn_d16_three_chain", 1, 3, 45,  16, "three_chain",         False, False, 15),
    ("attn_d32_alternating", 1, 2, 130, 32, "alternating",         False, True,  16),
    ("attn_d32_sqrt",        2, 2, 64,  32, "two_chain_no_pad",    True,  False, 17),
]


def _fp32_softmax_attention(self, x, chain_mask, padding_mask, chain_ids=None):
    """The base layer's PyTorch attention (mint_plus/models/modules.py:94-154) with the softmax in float32 followed by a
    cast back, as the reference's own muS layer does it (mu_scaling/layer.py:159-165).  The base layer hard-codes a bfloat16
    softmax that cannot run on float32 tensors, and its default path launches Triton kernels, which need a GPU."""
    import torch.nn.functional as F
    intra_logits, intra_values = self.self_attn(x=x, key_padding_mask=padding_mask, before_softmax=True)
    inter_logits, inter_values = self.multimer_attn(x=x, key_padding_mask=padding_mask, before_softmax=True)
    m = chain_mask.unsqueeze(1)
    probs = F.softmax(torch.where(m, inter_logits, intra_logits), dim=-1, dtype=torch.float32).type_as(intra_values)
    out = torch.matmul(probs.masked_fill(m, 0.0), intra_values) + torch.matmul(probs.masked_fill(~m, 0.0), inter_values)
    out = out.transpose(1, 2).contiguous()
    out = out.view(*out.shape[:2], -1)
    return self.self_attn.out_proj(out).transpose(0, 1).contiguous(), None


def run_model_case(name, kind, seed, batch_seed, B, T, lo, hi, sqrt_softmax=False):
    """Whole-model forward of the reference MINT-8M (6 layers, d=320, 20 heads, fp32, eval) on a seeded batch; the weights
    are the name-keyed values of oracle/seeded_weights.py, so only tokens, chain ids and outputs are stored."""
    sys.path.insert(0, os.path.join(HERE, "..", ".."))
    from oracle.seeded_weights import c1_batch, fill_state_dict_
    from mint_plus.models.esm2 import MINT
    from mint_plus.models.modules import TransformerLayer_MINT
    if kind == "base":
        TransformerLayer_MINT._multimer_attention_plus = _fp32_softmax_attention
        model = MINT(num_layers=6, embed_dim=320, attention_heads=20, use_multimer=True, use_erf_gelu=True)
    else:
        from mint_plus.models.mu_scaling import build_mint_mu
        model = build_mint_mu("8M", use_sqrt_softmax=sqrt_softmax)
    fill_state_dict_(model, seed)
    model.eval()
    tokens, chain_ids = c1_batch(batch_seed, B, T, lo, hi)
    with torch.no_grad():
        res = model(tokens, chain_ids, repr_layers=[3, 6])
    np.savez_compressed(os.path.join(HERE, name + ".npz"), tokens=tokens.numpy().astype(np.int16),
                        chain_ids=chain_ids.numpy().astype(np.int8), logits=res["logits"].numpy(),
                        repr3=res["representations"][3][:, ::8].contiguous().numpy(),
                        repr6=res["representations"][6][:, ::8].contiguous().numpy(),
                        meta=np.array([seed, batch_seed, B, T, lo, hi, int(sqrt_softmax)]),
                        keys=np.array(sorted(model.state_dict().keys())))
    print(name, "logits", tuple(res["logits"].shape), "abs max", float(res["logits"].abs().max()))


MODEL_CASES = [
    # name                kind    weight seed  batch seed  B  T    lo  hi   sqrt
    ("mint8m_c1",          "base", 1234,        1001,       4, 512, 64, 200, False),   # the reference's CPU-runnable 8M configuration
    ("mint8m_small",       "base", 1235,        1002,       2, 96,  10, 40,  False),
    ("mint8m_mu",          "mu",   1236,        1003,       2, 160, 20, 70,  False),
    ("mint8m_mu_sqrt",     "mu",   1237,        1004,       2, 160, 20, 70,  True),
]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path to the mint_plus checkout")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    torch.set_grad_enabled(True)
    for c in CASES:
        run_case(*c)
    for c in MODEL_CASES:
        run_model_case(*c)


if __name__ == "__main__":
    main()
