"""Seeded random shapes of the projection GEMMs (forward with its epilogues, dgrad, wgrad) against fp32 tensor expressions
on the same bf16 operands: rows, columns and reduction lengths off every tile and slab boundary, wgrad reductions that
exercise the large-unit / short-piece plan with ragged last pieces."""
import random

import pytest
import torch

from oracle import multimer_attention as O

pytestmark = pytest.mark.gpu

from mint_plus_b200 import ops  # noqa: E402

DEV = "cuda"


def _dims(seed):
    rng = random.Random(500 + seed)
    Mr = rng.choice([rng.randint(1, 140), rng.randint(120, 700), rng.randint(600, 3000)])
    N = 8 * rng.choice([rng.randint(1, 40), rng.randint(30, 120), rng.randint(100, 400)])
    K = 8 * rng.choice([rng.randint(1, 20), rng.randint(8, 90), rng.randint(80, 330)])
    return rng, Mr, N, K


@pytest.mark.parametrize("seed", range(16))
def test_forward_epilogues(seed):
    rng, Mr, N, K = _dims(seed)
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(Mr, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) / K ** 0.5).bfloat16()
    b = torch.randn(N, generator=g) if rng.random() < 0.8 else None
    gelu = rng.random() < 0.5
    z = x.float() @ w.float().t() + (b if b is not None else 0.0)
    want = O.gelu_erf(z) if gelu else z
    bd = None if b is None else b.to(DEV)
    if gelu and rng.random() < 0.5:
        got, pre = ops.gemm_bf16(x.to(DEV), w.to(DEV), bd, True, True)
        torch.testing.assert_close(pre.float().cpu(), z, rtol=1e-2, atol=1e-2)
    else:
        got = ops.gemm_bf16(x.to(DEV), w.to(DEV), bd, gelu)
    ops.check_device_status()
    torch.testing.assert_close(got.float().cpu(), want, rtol=1e-2, atol=1e-2)
    # the residual sum of the layer formed in the epilogue
    r = torch.randn(Mr, N, generator=g).bfloat16()
    a_, b_ = rng.uniform(0.5, 1.0), rng.uniform(0.2, 1.0)
    s, _ = ops.gemm_res(x.to(DEV), w.to(DEV), 1.0, bd, r.to(DEV), a_, b_)
    ops.check_device_status()
    torch.testing.assert_close(s.float().cpu(), a_ * r.float() + b_ * z, rtol=1e-2, atol=2e-2)


@pytest.mark.parametrize("seed", range(16))
def test_backward_products(seed):
    rng, Mr, N, K = _dims(100 + seed)
    g = torch.Generator().manual_seed(seed)
    dz = torch.randn(Mr, N, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) / N ** 0.5).bfloat16()
    x = torch.randn(Mr, K, generator=g).bfloat16()
    dx = ops.gemm_dgrad(dz.to(DEV), w.to(DEV)).float().cpu()
    want_dx = dz.float() @ w.float()
    torch.testing.assert_close(dx, want_dx, rtol=1e-2, atol=1e-2 * max(1.0, want_dx.abs().max().item()) / 4)
    want_dw = dz.float().t() @ x.float()
    for odt in (torch.float32, torch.bfloat16):
        dw = ops.gemm_wgrad(dz.to(DEV), x.to(DEV), out_dtype=odt).float().cpu()
        tol = (2e-5 if odt == torch.float32 else 1e-2) * max(1.0, want_dw.abs().max().item())
        assert (dw - want_dw).abs().max().item() <= tol
    ops.check_device_status()
