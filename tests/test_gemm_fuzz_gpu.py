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


@pytest.mark.parametrize("seed", range(12))
def test_eight_bit_products(seed):
    """e4m3 x e4m3 forward (bf16 result; e4m3 result with the bf16 pre-activation beside it, the fc1 configuration) and
    e5m2 x e4m3 backward products on random shapes, against fp32 products of the SAME 8-bit values: only the order of the
    fp32 additions and the final rounding differ."""
    rng = random.Random(900 + seed)
    Mr = 16 * rng.choice([rng.randint(1, 9), rng.randint(8, 60), rng.randint(40, 200)])
    N = 16 * rng.choice([rng.randint(1, 20), rng.randint(16, 100)])
    K = 16 * rng.choice([rng.randint(1, 12), rng.randint(8, 90)])
    g = torch.Generator().manual_seed(seed)
    x8 = (torch.randn(Mr, K, generator=g) * 2).to(torch.float8_e4m3fn)
    w8 = (torch.randn(N, K, generator=g) * 2).to(torch.float8_e4m3fn)
    b = torch.randn(N, generator=g)
    alpha = 1.0 / (4.0 * K ** 0.5)
    z = alpha * (x8.float() @ w8.float().t()) + b
    got = ops.gemm_e4m3(x8.to(DEV), w8.to(DEV), alpha, b.to(DEV)).float().cpu()
    torch.testing.assert_close(got, z, rtol=1e-2, atol=1e-2)
    # GELU, e4m3 result and bf16 pre-activation from one launch
    out_scale = max(float(O.gelu_erf(z).abs().max()), 1e-3) / 448.0
    q, pre = ops.gemm_e4m3(x8.to(DEV), w8.to(DEV), alpha, b.to(DEV), gelu=True, out_e4m3_scale=out_scale, save_preact=True)
    ops.check_device_status()
    torch.testing.assert_close(pre.float().cpu(), z, rtol=1e-2, atol=1e-2)
    want_q = O.gelu_erf(z)
    assert (q.float().cpu() * out_scale - want_q).abs().max().item() <= 0.07 * max(float(want_q.abs().max()), 1e-3)   # 3 mantissa bits
    # backward products: e5m2 gradient against the e4m3 operands
    g8 = (torch.randn(Mr, N, generator=g) * 4).to(torch.float8_e5m2)
    dx = ops.gemm_dgrad(g8.to(DEV), w8.to(DEV)).float().cpu()
    want_dx = g8.float() @ w8.float()
    assert (dx - want_dx).abs().max().item() <= 1e-2 * max(1.0, want_dx.abs().max().item())
    dw = ops.gemm_wgrad(g8.to(DEV), x8.to(DEV), out_dtype=torch.float32).float().cpu()
    want_dw = g8.float().t() @ x8.float()
    assert (dw - want_dw).abs().max().item() <= 2e-5 * max(1.0, want_dw.abs().max().item())
    ops.check_device_status()
