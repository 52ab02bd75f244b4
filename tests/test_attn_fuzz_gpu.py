"""Seeded random cases of the attention path against the CPU oracle: shapes off every tile boundary, one to five chains per
sample, padded positions at the end of chains (so pads sit between chains as well as at the end, as the reference's collate
function leaves them, data/data.py:69-74,113-127), both softmax modes, with and without RoPE, fp32 and bf16."""
import math
import random

import pytest
import torch

from oracle import multimer_attention as O

pytestmark = pytest.mark.gpu

import mint_plus_b200 as M  # noqa: E402
from mint_plus_b200 import ops  # noqa: E402

DEV = "cuda"


def _case(seed):
    rng = random.Random(1000 + seed)
    D = rng.choice([16, 32, 64])
    B, H = rng.randint(1, 3), rng.randint(1, 4)
    T = rng.choice([rng.randint(1, 130), rng.randint(120, 400), rng.randint(380, 700), 128, 256, 384, 512])
    if rng.random() < 0.15:
        T = rng.randint(700, 1300)
    sq, rope, f32 = rng.random() < 0.3, rng.random() < 0.7, rng.random() < 0.3
    g = torch.Generator().manual_seed(rng.randint(0, 1 << 30))
    rnd = (lambda t: t) if f32 else (lambda t: t.bfloat16().float())
    ts = [rnd(torch.randn(B, H, T, D, generator=g) / math.sqrt(D)) for _ in range(6)]
    grad = rnd(torch.randn(B, H, T, D, generator=g))
    cid = torch.zeros(B, T, dtype=torch.int32)
    pad = torch.zeros(B, T, dtype=torch.bool)
    for b in range(B):
        n_ch = rng.randint(1, 5)
        cuts = sorted(rng.sample(range(1, T), min(n_ch - 1, T - 1))) if T > 1 else []
        bounds = [0] + cuts + [T]
        for c in range(len(bounds) - 1):
            cid[b, bounds[c]:bounds[c + 1]] = c
            seg = bounds[c + 1] - bounds[c]
            if seg > 2 and rng.random() < 0.5:
                npad = rng.randint(1, max(1, seg // 3))
                pad[b, bounds[c + 1] - npad:bounds[c + 1]] = True
        if pad[b].all():
            pad[b, 0] = False
    return ts, grad, cid, pad, sq, rope, f32


@pytest.mark.parametrize("seed", range(32))
def test_random_case_against_oracle(seed):
    ts, grad, cid, pad, sq, rope, f32 = _case(seed)
    want, wgrads = O.multimer_attention_fwd_bwd(*ts, O.chain_mask_from_ids(cid), grad, key_pad=pad, sqrt_softmax=sq, rope=rope)
    dt = torch.float32 if f32 else torch.bfloat16
    leaves = [t.to(DEV, dt).requires_grad_(True) for t in ts]
    out = M.multimer_attention(*leaves, chain_ids=cid.to(DEV), key_padding_mask=pad.to(DEV), rope=rope, sqrt_softmax=sq)
    grads = torch.autograd.grad(out, leaves, grad.to(DEV, dt))
    ops.check_device_status()
    out = out.float().cpu()
    # fp32: 1e-5 relative (floor 2e-6); bf16: 2e-2 max-abs, relative to the largest output for the square-root softmax,
    # whose rows sum to more than one
    big = max(1.0, want.abs().max().item())
    tol = (1e-5 * big + 2e-6) if f32 else 2e-2 * (big if sq else 1.0)
    assert torch.isfinite(want).all()
    assert (out - want).abs().max().item() <= tol
    for name, g, w in zip(("dq_s", "dk_s", "dv_s", "dq_c", "dk_c", "dv_c"), grads, wgrads):
        g = g.float().cpu()
        scale = w.abs().max().item()
        assert torch.isfinite(g).all(), name
        assert (g - w).abs().max().item() <= (1e-4 if f32 else 2e-2) * scale + 1e-5, name
