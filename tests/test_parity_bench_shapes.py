"""Parity at the configurations the benchmarks run: the CUDA path (through the C ABI) against the CPU oracle on the exact
isolated-op batch (B8 H20 T1024 D32), on the MINT-650M attention shape (H20 T2048 D64, chains of 100..900 residues padded
to 2048, plain and square-root softmax), on a pair with skewed chain lengths at T2048, and one E=1280 / H=20 / T=2048 muS
layer in bf16 and in e4m3 against the CPU restatement of the same quantised layer (oracle/layer.py).

Tolerances: attention outputs <= 2e-2 max-abs against the fp32 oracle on the same bf16-rounded inputs, gradients within 2 % of
their scale (as tests/test_attn_gpu.py); layer outputs and gradients within a few bf16 steps of the restated layer.  The
e4m3 arithmetic itself is parity-unpinned: transformer_engine 2.16.0, which the reference calls for it, is not available;
the check is against the formula restated from mint_plus/models/alt/munit_scaling.py:22-55."""
import copy
import math

import pytest
import torch

from oracle import layer as OL
from oracle import multimer_attention as O

pytestmark = pytest.mark.gpu

import mint_plus_b200 as M  # noqa: E402
from mint_plus_b200 import ops  # noqa: E402

DEV = "cuda"
BF16_OUT_ATOL = 2e-2
BF16_GRAD_REL = 2e-2
NAMES = ("dq_s", "dk_s", "dv_s", "dq_c", "dk_c", "dv_c")


def make_pair_inputs(B, H, T, D, seed, len_a, len_b):
    """Seeded op inputs for pairs of chains: chain A of len_a = (lo, hi) residues, chain B of len_b, padded to T."""
    g = torch.Generator().manual_seed(seed)
    ts = [(torch.randn(B, H, T, D, generator=g) / math.sqrt(D)) for _ in range(6)]
    la = torch.randint(len_a[0], len_a[1] + 1, (B,), generator=g)
    lb = torch.randint(len_b[0], len_b[1] + 1, (B,), generator=g)
    cid = torch.zeros(B, T, dtype=torch.int32)
    pad = torch.zeros(B, T, dtype=torch.bool)
    for b in range(B):
        cid[b, int(la[b]):] = 1
        pad[b, min(T, int(la[b]) + int(lb[b])):] = True
    grad = torch.randn(B, H, T, D, generator=g)
    return ts, cid, pad, grad


def _check_against_oracle(ts, cid, pad, grad, sqrt_softmax=False):
    ts = [t.bfloat16().float() for t in ts]
    grad = grad.bfloat16().float()
    want, wgrads = O.multimer_attention_fwd_bwd(*ts, O.chain_mask_from_ids(cid), grad, key_pad=pad, sqrt_softmax=sqrt_softmax)
    leaves = [t.to(DEV, torch.bfloat16).requires_grad_(True) for t in ts]
    out = M.multimer_attention(*leaves, chain_ids=cid.to(DEV), key_padding_mask=pad.to(DEV), sqrt_softmax=sqrt_softmax)
    grads = torch.autograd.grad(out, leaves, grad.to(DEV, torch.bfloat16))
    ops.check_device_status()
    tol = BF16_OUT_ATOL * (max(1.0, want.abs().max().item()) if sqrt_softmax else 1.0)
    err = (out.float().cpu() - want).abs().max().item()
    assert err <= tol, f"out: max err {err:.4g} > {tol:.4g}"
    for g, w, n in zip(grads, wgrads, NAMES):
        scale = w.abs().max().item()
        e = (g.float().cpu() - w).abs().max().item()
        assert e <= BF16_GRAD_REL * scale + 1e-5, f"{n}: max err {e:.4g} vs scale {scale:.4g}"


def test_isolated_op_benchmark_batch_against_oracle():
    """The very batch bench.py times (seed 2002): forward and the six gradients."""
    ts, cid, pad, grad = O.make_op_inputs(8, 20, 1024, 32, seed=2002)
    _check_against_oracle(ts, cid, pad, grad)


@pytest.mark.parametrize("sqrt_softmax", [False, True])
def test_mint650m_attention_shape_against_oracle(sqrt_softmax):
    """H=20, D=64, T=2048, chain lengths uniform in [100, 900] padded to 2048 (16 query tiles, fully padded key tiles)."""
    ts, cid, pad, grad = make_pair_inputs(2, 20, 2048, 64, seed=4004, len_a=(100, 900), len_b=(100, 900))
    _check_against_oracle(ts, cid, pad, grad, sqrt_softmax)


def test_skewed_pair_at_2048_against_oracle():
    """One chain of 30..80 residues against a partner of 800..1900 (the inference configuration's length distribution)."""
    ts, cid, pad, grad = make_pair_inputs(2, 8, 2048, 64, seed=5005, len_a=(30, 80), len_b=(800, 1900))
    _check_against_oracle(ts, cid, pad, grad)


def _bf16_representable_(module):
    for p in module.parameters():
        p.data = p.data.bfloat16().float()


@pytest.mark.parametrize("mode", ["bf16", "fp8", "fp8_unit_sqrt"])
def test_mus_layer_1280_wide_against_restated_layer(mode):
    """E=1280, H=20 (D=64), T=2048, one pair: the muS layer of the MINT-650M FP8 workload on the GPU against the CPU
    restatement with the same rounding points.  `fp8`: e4m3 projections with default initialisation; `fp8_unit_sqrt`:
    unit-variance weights, the static 1/sqrt(fan_in) output multipliers and the square-root softmax (the benchmark's set-up)."""
    from mint_plus_b200.mu_scaling import TransformerLayer_MINT_mu, set_unit_output_scales, unit_variance_init_
    torch.manual_seed(1280)
    E, H, T, B = 1280, 20, 2048, 1
    tau = 0.5 / math.sqrt(33)
    sqrt_sm = mode == "fp8_unit_sqrt"
    layer = TransformerLayer_MINT_mu(E, 4 * E, H, use_rotary_embeddings=True, use_multimer=True, use_erf_gelu=True, tau=tau,
                                     num_layers=33, use_sqrt_softmax=sqrt_sm).float()
    if mode == "fp8_unit_sqrt":
        unit_variance_init_(layer)
    else:
        with torch.no_grad():
            for name, p in layer.named_parameters():
                if name.endswith("bias"):
                    p.normal_(0, 0.05)
    _bf16_representable_(layer)
    x = torch.randn(T, B, E).bfloat16().float()
    gy = torch.randn(T, B, E).bfloat16().float()
    g = torch.Generator().manual_seed(650)
    la, lb = (int(torch.randint(100, 901, (1,), generator=g)) for _ in range(2))
    cid = torch.zeros(B, T, dtype=torch.int32); cid[:, la:] = 1
    pad = torch.zeros(B, T, dtype=torch.bool); pad[:, la + lb:] = True
    mask = O.chain_mask_from_ids(cid)

    # GPU layer first: its 8-bit backward measures the static e5m2 gradient scales that the restatement then takes over
    glayer = copy.deepcopy(layer).to(DEV).to(torch.bfloat16)
    if mode != "bf16":
        holder = torch.nn.Module()
        holder.layers = torch.nn.ModuleList([glayer])
        M.apply_fp8_to_model(holder)
        if mode == "fp8_unit_sqrt":
            set_unit_output_scales(holder)
    xg = x.to(DEV, torch.bfloat16).requires_grad_(True)
    out, _ = glayer(xg, self_attn_padding_mask=pad.to(DEV), chain_ids=cid.to(DEV))
    out.backward(gy.to(DEV, torch.bfloat16))
    ops.check_device_status()

    fp8 = None
    if mode != "bf16":
        sa, ma, ff = glayer.self_attn, glayer.multimer_attn, glayer.feed_forward
        os_e, os_4e = (E ** -0.5, (4 * E) ** -0.5) if mode == "fp8_unit_sqrt" else (1.0, 1.0)
        ws_s = OL.weight_scale(layer.self_attn.q_proj.weight, layer.self_attn.k_proj.weight, layer.self_attn.v_proj.weight)
        ws_c = OL.weight_scale(layer.multimer_attn.q_proj.weight, layer.multimer_attn.k_proj.weight, layer.multimer_attn.v_proj.weight)
        gs_s = sa._fp8_qkv_grad_scale.scale
        assert gs_s is not None and sa.out_proj.grad_scale.scale is not None and ff.fc1.grad_scale.scale is not None
        fp8 = {"x_scale": 1.0, "out_scale": os_e, "per": {
            "sa_qkv": {"g_scale": gs_s}, "ma_qkv": {"g_scale": gs_s * ws_s / ws_c},     # one multiplier for both dgrad pairs
            "out": {"g_scale": sa.out_proj.grad_scale.scale}, "fc1": {"g_scale": ff.fc1.grad_scale.scale},
            "fc2": {"g_scale": ff.fc2.grad_scale.scale, "out_scale": os_4e}}}
    # CPU restatement (fp32 arithmetic on bf16-representable values)
    xc = x.clone().requires_grad_(True)
    want = OL.mu_layer(layer, xc, mask, pad, tau, fp8=fp8, sqrt_softmax=sqrt_sm)
    want.backward(gy)
    wgx = xc.grad.clone()
    wg_fc1 = layer.feed_forward.fc1.weight.grad.clone()
    wg_q = layer.self_attn.q_proj.weight.grad.clone()
    layer.zero_grad()

    def rel(got, ref):
        return (got.float().cpu() - ref).abs().max().item() / ref.abs().max().item()

    def fro(got, ref):
        return ((got.float().cpu() - ref).norm() / ref.norm()).item()

    pairs = {"out": (out.detach(), want.detach()), "dx": (xg.grad, wgx), "dW_fc1": (glayer.feed_forward.fc1.weight.grad, wg_fc1),
             "dW_q": (glayer.self_attn.q_proj.weight.grad, wg_q)}
    errs = {k: rel(*v) for k, v in pairs.items()}
    frob = {k: fro(*v) for k, v in pairs.items()}
    print(f"mus layer {mode}: max/scale " + ", ".join(f"{k} {v:.3g}" for k, v in errs.items())
          + " | frobenius " + ", ".join(f"{k} {v:.3g}" for k, v in frob.items()))
    # the layer's output is a LayerNorm result (values of a few units): a bf16 step there is 1.6e-2 relative to the largest
    assert errs["out"] <= 3e-2, errs
    # Gradients.  bf16 products: a few bf16 steps.  8-bit products: an e5m2 number has two mantissa bits, and a gradient
    # element that differs by one bf16 step between the two sides can round to e5m2 neighbours 12.5 - 25 % apart, so single
    # elements of a weight gradient move by more than the bulk does; the bulk is held by the relative Frobenius error.
    grad_tol = 4e-2 if mode == "bf16" else 1e-1
    assert max(errs["dx"], errs["dW_fc1"], errs["dW_q"]) <= grad_tol, errs
    assert max(frob.values()) <= (2e-2 if mode == "bf16" else 8e-2), frob
