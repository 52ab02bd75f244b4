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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path to the mint_plus checkout")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    torch.set_grad_enabled(True)
    for c in CASES:
        run_case(*c)


if __name__ == "__main__":
    main()
