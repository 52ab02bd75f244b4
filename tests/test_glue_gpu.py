"""The HBM-bound glue kernels (fused residual + LayerNorm, GELU backward + bias gradient, QKV gradient pack) against plain
PyTorch fp32 statements of the same arithmetic, through the C ABI."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from mint_plus_b200 import ops  # noqa: E402

DEV = "cuda"


def _bf(t):
    return t.to(torch.bfloat16)


@pytest.mark.parametrize("E", [320, 640, 1280, 2560, 72])
@pytest.mark.parametrize("mode", ["ln_only", "add_ln", "add_ln_keep_s", "add_only"])
def test_add_layernorm_forward_and_backward(E, mode):
    torch.manual_seed(E)
    rows_shape = (37, 3)                         # ragged number of rows: 111
    x = _bf(torch.randn(*rows_shape, E, device=DEV)).requires_grad_(True)
    r = _bf(torch.randn(*rows_shape, E, device=DEV)).requires_grad_(True) if mode != "ln_only" else None
    a, b = (1.0, 0.0) if mode == "ln_only" else (math.sqrt(0.9), math.sqrt(0.1))
    norm = None
    if mode != "add_only":
        norm = torch.nn.LayerNorm(E).to(DEV, torch.bfloat16)
        with torch.no_grad():
            norm.weight.copy_(1 + 0.1 * torch.randn(E))
            norm.bias.copy_(0.1 * torch.randn(E))
    need_s = mode in ("add_ln_keep_s", "add_only")
    s, y = ops.add_layernorm(x, r, a, b, norm, need_s=need_s)

    xf = x.detach().float().requires_grad_(True)
    rf = r.detach().float().requires_grad_(True) if r is not None else None
    sf = a * xf + (b * rf if rf is not None else 0.0)
    gs = torch.randn_like(sf)
    gy = torch.randn_like(sf)
    loss_ref = 0.0
    loss = 0.0
    if need_s:
        torch.testing.assert_close(s.float(), sf, rtol=1e-2, atol=1e-2)
        loss = loss + (s.float() * gs).sum()
        loss_ref = loss_ref + (sf * gs).sum()
    else:
        assert s is None
    if norm is not None:
        w32, b32 = norm.weight.detach().float().requires_grad_(True), norm.bias.detach().float().requires_grad_(True)
        yf = torch.nn.functional.layer_norm(sf, (E,), w32, b32, norm.eps)
        torch.testing.assert_close(y.float(), yf, rtol=2e-2, atol=2e-2)
        loss = loss + (y.float() * gy).sum()
        loss_ref = loss_ref + (yf * gy).sum()
    loss.backward()
    loss_ref.backward()
    scale = xf.grad.abs().max().item()
    assert (x.grad.float() - xf.grad).abs().max().item() <= 2e-2 * scale + 1e-3
    if r is not None:
        assert (r.grad.float() - rf.grad).abs().max().item() <= 2e-2 * rf.grad.abs().max().item() + 1e-3
    if norm is not None:
        assert (norm.weight.grad.float() - w32.grad).abs().max().item() <= 2e-2 * w32.grad.abs().max().item() + 1e-2
        assert (norm.bias.grad.float() - b32.grad).abs().max().item() <= 2e-2 * b32.grad.abs().max().item() + 1e-2


@pytest.mark.parametrize("E", [320, 1280, 2560])
def test_add_layernorm_backward_walks_many_rows(E):
    """More rows than one sweep of the backward grid holds (a CTA takes several batches of rows, the last one ragged)."""
    torch.manual_seed(7)
    rows = 10007
    x = _bf(torch.randn(rows, E, device=DEV)).requires_grad_(True)
    r = _bf(torch.randn(rows, E, device=DEV)).requires_grad_(True)
    a, b = math.sqrt(0.7), math.sqrt(0.3)
    norm = torch.nn.LayerNorm(E).to(DEV, torch.bfloat16)
    with torch.no_grad():
        norm.weight.copy_(1 + 0.1 * torch.randn(E))
    s, y = ops.add_layernorm(x, r, a, b, norm, need_s=True)
    gs, gy = torch.randn(rows, E, device=DEV), torch.randn(rows, E, device=DEV)
    ((s.float() * gs).sum() + (y.float() * gy).sum()).backward()
    xf, rf = x.detach().float().requires_grad_(True), r.detach().float().requires_grad_(True)
    w32, b32 = norm.weight.detach().float().requires_grad_(True), norm.bias.detach().float().requires_grad_(True)
    sf = a * xf + b * rf
    yf = torch.nn.functional.layer_norm(sf, (E,), w32, b32, norm.eps)
    # the kernel receives the upstream gradients rounded to bf16
    ((sf * _bf(gs).float()).sum() + (yf * _bf(gy).float()).sum()).backward()
    for got, want in ((x.grad, xf.grad), (r.grad, rf.grad)):
        assert (got.float() - want).abs().max().item() <= 2e-2 * want.abs().max().item() + 1e-3
    for got, want in ((norm.weight.grad, w32.grad), (norm.bias.grad, b32.grad)):
        assert (got.float() - want).abs().max().item() <= 2e-2 * want.abs().max().item() + 5e-2
    # fixed order of every sum: a second run gives the same bits
    x2, r2 = x.detach().clone().requires_grad_(True), r.detach().clone().requires_grad_(True)
    norm.weight.grad = None
    norm.bias.grad = None
    s2, y2 = ops.add_layernorm(x2, r2, a, b, norm, need_s=True)
    ((s2.float() * gs).sum() + (y2.float() * gy).sum()).backward()
    assert torch.equal(x2.grad, x.grad) and torch.equal(r2.grad, r.grad)


def test_add_layernorm_rejects_unsupported_width():
    x = _bf(torch.randn(4, 4096, device=DEV))
    with pytest.raises(NotImplementedError):
        ops.add_layernorm(x, None, 1.0, 0.0, torch.nn.LayerNorm(4096).to(DEV, torch.bfloat16))
    with pytest.raises((ValueError, NotImplementedError)):
        ops.add_layernorm(_bf(torch.randn(4, 36, device=DEV)), None, 1.0, 0.0, None)


@pytest.mark.parametrize("shape", [(300, 1280), (513, 72), (64, 5120)])
@pytest.mark.parametrize("with_z", [True, False])
def test_gelu_backward_and_bias_gradient(shape, with_z):
    torch.manual_seed(1)
    M, N = shape
    dy = _bf(torch.randn(M, N, device=DEV))
    z = _bf(2 * torch.randn(M, N, device=DEV)) if with_z else None
    dz, db = ops.gelu_bwd_colsum(dy, z)
    if with_z:
        zf = z.float().requires_grad_(True)
        torch.nn.functional.gelu(zf).backward(dy.float())
        want = zf.grad
        assert (dz.float() - want).abs().max().item() <= 1e-2 * want.abs().max().item() + 1e-3
    else:
        assert dz is dy or torch.equal(dz, dy)
    want_db = dz.float().sum(0)
    assert (db - want_db).abs().max().item() <= 1e-3 * want_db.abs().max().item() + 1e-3


@pytest.mark.parametrize("shape", [(300, 1280), (513, 72)])
@pytest.mark.parametrize("with_z", [True, False])
def test_e5m2_gradient_copy_and_its_bias_gradient(shape, with_z):
    """mintb_gelu_bwd_colsum_f8: dz = dy gelu'(z) (dy without z) leaves the pass as e5m2 numbers saturate(dz / scale) - the
    operand of the 8-bit dgrad / wgrad products - and db sums those very numbers times the scale
    (mint_plus/models/alt/munit_scaling.py:41-55 of the reference)."""
    torch.manual_seed(4)
    M, N = shape
    dy = _bf(torch.randn(M, N, device=DEV))
    dy[0, :8] = _bf(torch.tensor([1e4, -1e4, 3e-7, 0.0, 1.0, -1.0, 2.5, 1e-3], device=DEV))
    z = _bf(2 * torch.randn(M, N, device=DEV)) if with_z else None
    scale = 0.01                                          # 1e4 / 0.01 = 1e6 saturates at 57344
    dz8, db, dz = ops.grad_colsum_f8(dy, z, True, scale, want_dz=True)
    want = dy.float()
    if with_z:
        zf = z.float().requires_grad_(True)
        torch.nn.functional.gelu(zf).backward(dy.float())
        want = zf.grad
        assert (dz.float() - want).abs().max().item() <= 1e-2 * want.abs().max().item() + 1e-3
    deq = dz8.float() * scale
    ref = (want / scale).clamp(-57344.0, 57344.0).to(torch.float8_e5m2).float() * scale
    # e5m2 has two mantissa bits: the kernel's fp32 value and the reference's may round to neighbours (one step = 25 %)
    close = (deq - ref).abs() <= 0.26 * ref.abs() + 1.01 * 2.0 ** -16 * scale       # (or by one subnormal step near zero)
    assert close.all() and (deq == ref).float().mean().item() > 0.98
    assert deq.abs().max().item() == pytest.approx(57344.0 * scale, rel=1e-6)     # saturated, finite
    want_db = deq.sum(0)
    assert (db - want_db).abs().max().item() <= 1e-3 * want_db.abs().max().item() + 1e-4


@pytest.mark.parametrize("D", [16, 32, 64])
@pytest.mark.parametrize("rope", [True, False])
def test_qkv_gradient_pack(D, rope):
    torch.manual_seed(D)
    T, B, H = 45, 3, 4
    E = H * D
    dq, dk, dv = (_bf(torch.randn(B, H, T, D, device=DEV)) for _ in range(3))
    cos = sin = None
    if rope:
        cos, sin, _ = ops.rope_tables(T, D, torch.device(DEV))
    q_scale = 0.25
    g = torch.empty(T * B, 3 * E, dtype=torch.bfloat16, device=DEV)
    from mint_plus_b200 import _lib as L
    db = torch.empty(3 * E, dtype=torch.float32, device=DEV)
    rc = L.lib().mintb_qkv_grad_pack(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), g.data_ptr(), db.data_ptr(),
                                     cos.data_ptr() if rope else None, sin.data_ptr() if rope else None, None, 0, T, B, H, D,
                                     q_scale, torch.cuda.current_stream().cuda_stream)
    L.check(rc, "mintb_qkv_grad_pack")
    torch.cuda.synchronize()
    a, b = dq.float(), dk.float()
    if rope:
        a, b = ops._rope_rotate_torch(a, cos, sin, True).float(), ops._rope_rotate_torch(b, cos, sin, True).float()
    a = a * q_scale
    want = torch.cat([t.permute(2, 0, 1, 3).reshape(T * B, E) for t in (a, b, dv.float())], dim=1)
    torch.testing.assert_close(g.float(), want, rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(db, g.float().sum(0), rtol=1e-3, atol=1e-3)
    # packed rows: only the listed (t, b) positions, in the listed order
    rows = torch.tensor([5, 0, 7, 44, T * B - 1, 17, 18, 19, 60], dtype=torch.int32, device=DEV)
    gp = torch.empty(rows.numel(), 3 * E, dtype=torch.bfloat16, device=DEV)
    rc = L.lib().mintb_qkv_grad_pack(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), gp.data_ptr(), db.data_ptr(),
                                     cos.data_ptr() if rope else None, sin.data_ptr() if rope else None, rows.data_ptr(),
                                     rows.numel(), T, B, H, D, q_scale, torch.cuda.current_stream().cuda_stream)
    L.check(rc, "mintb_qkv_grad_pack")
    torch.cuda.synchronize()
    assert torch.equal(gp, g[rows.long()])
    torch.testing.assert_close(db, gp.float().sum(0), rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("with_norm", [True, False])
def test_add_layernorm_writes_the_e4m3_operand_of_the_next_projection(with_norm):
    """quant_scale: the pass also leaves sat(result / scale) in e4m3 — the very bytes quantize_e4m3 gives — where the next
    FP8 projection looks for it (attached to the returned tensor)."""
    torch.manual_seed(2)
    x, r = _bf(3 * torch.randn(70, 2, 640, device=DEV)), _bf(3 * torch.randn(70, 2, 640, device=DEV))
    norm = torch.nn.LayerNorm(640).to(DEV, torch.bfloat16) if with_norm else None
    scale = 0.004                                     # small enough that some values saturate at 448
    s, y = ops.add_layernorm(x, r, 0.8, 0.6, norm, need_s=not with_norm, quant_scale=scale)
    main = y if with_norm else s
    assert main._mintb_e4m3[1] == scale                # the copy rides on the tensor the pass returned
    got = ops.e4m3_of(main, scale)
    assert got.data_ptr() == main._mintb_e4m3[0].data_ptr() and tuple(got.shape) == (140, 640)
    want = ops.quantize_e4m3(main.reshape(-1, 640).contiguous(), scale)
    assert torch.equal(got.view(torch.uint8), want.view(torch.uint8))
    assert (want.float().abs() == 448).any()


def test_add_layernorm_backward_with_frozen_norm_parameters():
    """Frozen gamma / beta (LoRA fine-tuning): the parameter-gradient sums and their second pass are skipped, the input
    gradients are the same bits."""
    torch.manual_seed(3)
    x0, r0 = _bf(torch.randn(500, 640, device=DEV)), _bf(torch.randn(500, 640, device=DEV))
    gy = _bf(torch.randn(500, 640, device=DEV))
    norm = torch.nn.LayerNorm(640).to(DEV, torch.bfloat16)
    grads = []
    for frozen in (False, True):
        for p in norm.parameters():
            p.requires_grad_(not frozen)
            p.grad = None
        x, r = x0.clone().requires_grad_(True), r0.clone().requires_grad_(True)
        _, y = ops.add_layernorm(x, r, 0.9, 0.4, norm, need_s=False)
        y.backward(gy)
        grads.append((x.grad, r.grad))
        assert (norm.weight.grad is None) == frozen
    assert torch.equal(grads[0][0], grads[1][0]) and torch.equal(grads[0][1], grads[1][1])
