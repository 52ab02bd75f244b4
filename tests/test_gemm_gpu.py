"""The tcgen05 projection GEMMs (bf16 and e4m3, fused epilogues), called through the C ABI, against CPU restatements."""
import pytest
import torch

from oracle import multimer_attention as O

pytestmark = pytest.mark.gpu

import mint_plus_b200 as M  # noqa: E402
from mint_plus_b200 import ops  # noqa: E402

DEV = "cuda"


def _ref_linear(x, w, b, gelu):
    y = x.float() @ w.float().t()
    if b is not None:
        y = y + b.float()
    return O.gelu_erf(y) if gelu else y


# (M, N, K): multiples of the 128 x 256 tile, ragged edges in every dimension, K shorter and longer than one 64-element slab
SHAPES = [(128, 256, 64), (300, 320, 320), (130, 264, 200), (1024, 3840, 1280), (77, 8, 8), (512, 1280, 5120)]


@pytest.mark.parametrize("gelu", [False, True])
@pytest.mark.parametrize("shape", SHAPES)
def test_bf16_linear_matches_fp32_reference(shape, gelu):
    Mr, N, K = shape
    g = torch.Generator().manual_seed(Mr + N + K)
    x = torch.randn(Mr, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) / K ** 0.5).bfloat16()
    b = torch.randn(N, generator=g)
    want = _ref_linear(x, w, b, gelu)
    got = ops.gemm_bf16(x.to(DEV), w.to(DEV), b.to(DEV), gelu).float().cpu()
    ops.check_device_status()
    # fp32 accumulation of bf16 products, result rounded to bf16: relative error ~2^-9 of the magnitude
    torch.testing.assert_close(got, want, rtol=1e-2, atol=1e-2)
    got_nb = ops.gemm_bf16(x.to(DEV), w.to(DEV), None, gelu).float().cpu()
    torch.testing.assert_close(got_nb, _ref_linear(x, w, None, gelu), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("shape", [(256, 512, 256), (300, 320, 320), (1024, 1280, 1280), (100, 72, 144)])
def test_e4m3_linear_matches_cpu_restatement(shape):
    Mr, N, K = shape
    g = torch.Generator().manual_seed(7 * Mr + N)
    x = torch.randn(Mr, K, generator=g).bfloat16()
    w = torch.randn(N, K, generator=g).bfloat16()
    b = torch.randn(N, generator=g)
    xs, ws = 1.0, float(w.float().abs().amax()) / 448.0
    # CPU restatement on the scaled tensors (alt/munit_scaling.py:22-34): clamp, e4m3 cast, fp32 matmul, scale back, bias
    want = O.fp8_e4m3_linear(x.float() / xs, w.float() / ws, None, out_scale=xs * ws) + b
    xq = ops.quantize_e4m3(x.to(DEV), xs)
    wq = ops.quantize_e4m3(w.to(DEV), ws)
    # the casts themselves are exact restatements
    assert torch.equal(xq.float().cpu(), (x.float() / xs).clamp(-448, 448).to(torch.float8_e4m3fn).float())
    assert torch.equal(wq.float().cpu(), (w.float() / ws).clamp(-448, 448).to(torch.float8_e4m3fn).float())
    got = ops.gemm_e4m3(xq, wq, xs * ws, b.to(DEV)).float().cpu()
    ops.check_device_status()
    # equal up to fp32 summation order and the final bf16 rounding
    torch.testing.assert_close(got, want, rtol=8e-3, atol=8e-3 * float(want.abs().max()) / 16)
    # e4m3 output with its own scale (the cast a following FP8 GEMM would consume)
    out_scale = float(want.abs().amax()) / 448.0
    got8 = ops.gemm_e4m3(xq, wq, xs * ws, b.to(DEV), out_e4m3_scale=out_scale).float().cpu() * out_scale
    assert (got8 - want).abs().max().item() <= 0.07 * float(want.abs().max())     # e4m3 has 3 mantissa bits


@pytest.mark.parametrize("rope", [False, True])
@pytest.mark.parametrize("dims", [(50, 3, 20, 16), (96, 2, 20, 32), (130, 2, 4, 64), (33, 1, 10, 32)])
def test_qkv_projection_head_major_with_rope(dims, rope):
    T, B, H, D = dims
    E = H * D
    g = torch.Generator().manual_seed(T + D)
    x = torch.randn(T, B, E, generator=g).bfloat16()
    w = (torch.randn(3 * E, E, generator=g) / E ** 0.5).bfloat16()
    b = (0.1 * torch.randn(3 * E, generator=g))
    q, k, v = O.project_qkv_4d(x.float(), w.float(), b, H)
    if rope:
        q, k = O.apply_rope(q), O.apply_rope(k)
    tabs = ops.rope_tables(T, D, torch.device(DEV))[:2] if rope else None
    gq, gk, gv = ops.qkv_project(x.to(DEV), w.to(DEV), b.to(DEV), H, rope=tabs)
    ops.check_device_status()
    for got, want in ((gq, q), (gk, k), (gv, v)):
        assert got.shape == (B, H, T, D) and got.is_contiguous()
        torch.testing.assert_close(got.float().cpu(), want, rtol=1e-2, atol=2e-2)


@pytest.mark.parametrize("dims", [(70, 3, 4, 32), (130, 2, 5, 64), (40, 2, 6, 16)])
@pytest.mark.parametrize("fp8", [False, True])
def test_two_pathway_qkv_product_equals_the_two_single_products(dims, fp8):
    """mintb_qkv2_fwd: both pathways' projections as one product on the [6E][E] operand give the very bits of the two
    3E-wide products (same tiles, same accumulation order): six head-major tensors, RoPE on the first pathway only,
    separate multipliers for the two pathways' e4m3 weights."""
    from mint_plus_b200 import _lib as L
    T, B, H, D = dims
    E = H * D
    g = torch.Generator().manual_seed(T * 7 + D)
    x = torch.randn(T, B, E, generator=g).bfloat16().to(DEV)
    w1, w2 = ((torch.randn(3 * E, E, generator=g) * s).bfloat16().to(DEV) for s in (E ** -0.5, 2 * E ** -0.5))
    b1, b2 = ((0.1 * torch.randn(3 * E, generator=g)).to(DEV) for _ in range(2))
    tabs = ops.rope_tables(T, D, torch.device(DEV))[:2]
    if fp8:
        s1, s2 = float(w1.float().abs().max()) / 448, float(w2.float().abs().max()) / 448
        f1, f2 = (ops.quantize_e4m3(w1, s1), s1, 1.0, 1.0), (ops.quantize_e4m3(w2, s2), s2, 1.0, 1.0)
        w6 = torch.cat([f1[0].view(torch.uint8), f2[0].view(torch.uint8)]).view(torch.float8_e4m3fn)
        xin, in_dt, al = ops.quantize_e4m3(x.reshape(-1, E), 1.0), L.E4M3, (s1, s2)
    else:
        f1 = f2 = None
        w6, xin, in_dt, al = torch.cat([w1, w2]), x.reshape(-1, E), L.BF16, (1.0, 1.0)
    want = list(ops.qkv_project(x, w1, b1, H, rope=tabs, fp8=f1)) + list(ops.qkv_project(x, w2, b2, H, fp8=f2))
    b6 = torch.cat([b1, b2])
    outs = [torch.empty(B, H, T, D, dtype=torch.bfloat16, device=DEV) for _ in range(6)]
    rc = L.lib().mintb_qkv2_fwd(xin.data_ptr(), w6.data_ptr(), b6.data_ptr(), *[t.data_ptr() for t in outs], T, B, H, D, in_dt, L.F32,
                                al[0], al[1], 1.0, tabs[0].data_ptr(), tabs[1].data_ptr(), None, T * B,
                                torch.cuda.current_stream().cuda_stream, ops._dev_status(torch.device(DEV, 0)).data_ptr())
    L.check(rc, "mintb_qkv2_fwd")
    ops.check_device_status()
    for got, ref in zip(outs, want):
        assert torch.equal(got, ref)


@pytest.mark.parametrize("shape", [(300, 256, 128), (77, 136, 64), (2048, 1280, 1280)])
@pytest.mark.parametrize("quant", [False, True])
def test_residual_sum_in_the_projection_epilogue(shape, quant):
    """mintb_linear_res_fwd: a r + b (x W^T + bias) in one pass, and with an e4m3 result the bf16 copy beside it, the e4m3
    numbers cast from the bf16 values."""
    M_, N, K = shape
    g = torch.Generator().manual_seed(N)
    x = torch.randn(M_, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) / K ** 0.5).bfloat16()
    bias = 0.1 * torch.randn(N, generator=g)
    r = torch.randn(M_, N, generator=g).bfloat16()
    a, b = 0.9, 0.4
    want = a * r.float() + b * (x.float() @ w.float().t() + bias)
    out, q8 = ops.gemm_res(x.to(DEV), w.to(DEV), 1.0, bias.to(DEV), r.to(DEV), a, b, quant_scale=0.02 if quant else None)
    ops.check_device_status()
    assert (out.float().cpu() - want).abs().max().item() <= 1e-2 * want.abs().max().item() + 1e-3
    if quant:
        ref8 = ops.quantize_e4m3(out, 0.02)
        assert torch.equal(q8.view(torch.uint8), ref8.view(torch.uint8))
    # and differentiable: gradients of x, W, bias and the residual
    xd, wd, bd, rd = (t.to(DEV).requires_grad_(True) for t in (x, w, bias, r))
    gy = torch.randn(M_, N, generator=g).bfloat16()
    ops.linear_res(xd, wd, bd, rd, a, b).backward(gy.to(DEV))
    xr, wr, br, rr = (t.float().requires_grad_(True) for t in (x, w, bias, r))
    (a * rr + b * (xr @ wr.t() + br)).backward(gy.float())
    for got, ref in ((xd.grad, xr.grad), (wd.grad, wr.grad), (bd.grad, br.grad), (rd.grad, rr.grad)):
        assert (got.float().cpu() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-3


def test_linear_and_qkv_gradients_match_autograd():
    g = torch.Generator().manual_seed(3)
    T, B, H, D = 40, 2, 4, 32
    E = H * D
    x = torch.randn(T, B, E, generator=g).bfloat16()
    w = (torch.randn(3 * E, E, generator=g) / E ** 0.5).bfloat16()
    b = 0.1 * torch.randn(3 * E, generator=g)
    go = [torch.randn(B, H, T, D, generator=g).bfloat16() for _ in range(3)]
    # reference through the oracle projection + rope in fp32
    xr, wr, br = x.float().requires_grad_(True), w.float().requires_grad_(True), b.clone().requires_grad_(True)
    q, k, v = O.project_qkv_4d(xr, wr, br, H)
    q, k = O.apply_rope(q), O.apply_rope(k)
    torch.autograd.backward([q, k, v], [t.float() for t in go])
    xd, wd, bd = x.to(DEV).requires_grad_(True), w.to(DEV).requires_grad_(True), b.to(DEV).requires_grad_(True)
    tabs = ops.rope_tables(T, D, torch.device(DEV))[:2]
    outs = ops.qkv_project(xd, wd, bd, H, rope=tabs)
    torch.autograd.backward(list(outs), [t.to(DEV) for t in go])
    for got, want in ((xd.grad, xr.grad), (wd.grad, wr.grad), (bd.grad, br.grad)):
        err = (got.float().cpu() - want).abs().max().item()
        assert err <= 3e-2 * want.abs().max().item() + 1e-3
    # linear + GELU
    xl = torch.randn(70, E, generator=g).bfloat16()
    wl = (torch.randn(2 * E, E, generator=g) / E ** 0.5).bfloat16()
    bl = 0.1 * torch.randn(2 * E, generator=g)
    gy = torch.randn(70, 2 * E, generator=g).bfloat16()
    xr, wr, br = xl.float().requires_grad_(True), wl.float().requires_grad_(True), bl.clone().requires_grad_(True)
    _ref_linear(xr, wr, br, True).backward(gy.float())
    xd, wd, bd = xl.to(DEV).requires_grad_(True), wl.to(DEV).requires_grad_(True), bl.to(DEV).requires_grad_(True)
    ops.linear(xd, wd, bd, gelu=True).backward(gy.to(DEV))
    for got, want in ((xd.grad, xr.grad), (wd.grad, wr.grad), (bd.grad, br.grad)):
        err = (got.float().cpu() - want).abs().max().item()
        assert err <= 3e-2 * want.abs().max().item() + 1e-3


@pytest.mark.parametrize("fp8", [False, True])
def test_bf16_layer_forward_backward_against_restated_layer(fp8):
    """TransformerLayer_MINT_plus in bf16 on the GPU (GEMM epilogues + fused attention; e4m3 projections with 8-bit backward
    products when `fp8`) against the CPU restatement of the same layer with the same rounding and quantisation points
    (oracle/layer.py), at a tolerance of a few bf16 steps.  The e4m3 / e5m2 arithmetic is parity-unpinned (transformer_engine,
    which the reference calls for it, is not available): the check is against the formulas restated from
    mint_plus/models/alt/munit_scaling.py:22-55."""
    import copy
    from oracle import layer as OL
    torch.manual_seed(11)
    E, H, T, B = 128, 4, 150, 2
    layer = M.TransformerLayer_MINT_plus(E, 4 * E, H, use_multimer=True, use_erf_gelu=True).float()
    with torch.no_grad():
        for name, p in layer.named_parameters():
            if name.endswith("bias"):
                p.normal_(0, 0.05)
    for p in layer.parameters():                      # bf16-representable weights so both sides see the same numbers
        p.data = p.data.bfloat16().float()
    x = torch.randn(T, B, E).bfloat16().float()
    gy = torch.randn(T, B, E).bfloat16().float()
    cid = torch.zeros(B, T, dtype=torch.int32); cid[:, 70:] = 1
    pad = torch.zeros(B, T, dtype=torch.bool); pad[1, -13:] = True
    mask = O.chain_mask_from_ids(cid)

    glayer = copy.deepcopy(layer).to(DEV).to(torch.bfloat16)
    if fp8:
        holder = torch.nn.Module()
        holder.layers = torch.nn.ModuleList([glayer])
        M.apply_fp8_to_model(holder)
        assert isinstance(glayer.feed_forward.fc1, M.Fp8Linear) and isinstance(glayer.self_attn.fused_qkv, M.Fp8Linear)
        assert holder._fp8_config == {"enabled": True, "static_scale": True}
    xg = x.to(DEV, torch.bfloat16).requires_grad_(True)
    out, _ = glayer(xg, self_attn_mask=mask.to(DEV), self_attn_padding_mask=pad.to(DEV))
    out.backward(gy.to(DEV, torch.bfloat16))
    ops.check_device_status()

    cfg = None
    if fp8:      # the static e5m2 gradient scales the GPU layer measured on this (its first) backward pass
        sa, ma, ff = glayer.self_attn, glayer.multimer_attn, glayer.feed_forward
        gs = sa.fused_qkv.grad_scale.scale
        ratio = OL.weight_scale(layer.self_attn.fused_qkv.weight) / OL.weight_scale(layer.multimer_attn.fused_qkv.weight)
        cfg = {"x_scale": 1.0, "out_scale": 1.0, "per": {
            "sa_qkv": {"g_scale": gs}, "ma_qkv": {"g_scale": gs * ratio}, "out": {"g_scale": sa.out_proj.grad_scale.scale},
            "fc1": {"g_scale": ff.fc1.grad_scale.scale}, "fc2": {"g_scale": ff.fc2.grad_scale.scale}}}
    xc = x.clone().requires_grad_(True)
    want = OL.pre_ln_layer(layer, xc, mask, pad, fp8=cfg)
    want.backward(gy)

    def rel(got, ref):
        return (got.float().cpu() - ref).abs().max().item() / ref.abs().max().item()

    errs = {"out": rel(out.detach(), want.detach()), "dx": rel(xg.grad, xc.grad),
            "dW_fc2": rel(glayer.feed_forward.fc2.weight.grad, layer.feed_forward.fc2.weight.grad),
            "dW_qkv_cross": rel(glayer.multimer_attn.fused_qkv.weight.grad, layer.multimer_attn.fused_qkv.weight.grad),
            "db_out": rel(glayer.self_attn.out_proj.bias.grad, layer.self_attn.out_proj.bias.grad)}
    print(f"pre-LN layer fp8={fp8}: " + ", ".join(f"{k} {v:.3g}" for k, v in errs.items()))
    assert errs["out"] <= 3e-2, errs
    # (e5m2 gradients: elements that differ by one bf16 step between the two sides can round to e5m2 neighbours 12.5 - 25 % apart)
    assert max(errs["dx"], errs["dW_fc2"], errs["dW_qkv_cross"], errs["db_out"]) <= (8e-2 if fp8 else 3e-2), errs


def test_lora_linear_on_the_merged_weight_matches_the_formula():
    """y = x W^T + b + s (x A^T) B^T (lora.py / peft's LoRA) as one product on W + s B A, adapter gradients through thin
    products: values and gradients against the fp32 formula."""
    torch.manual_seed(4)
    M_, K, N, r, s = 300, 320, 192, 8, 2.0
    x = torch.randn(M_, K, device="cuda").to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(N, K, device="cuda") / K ** 0.5).to(torch.bfloat16)
    b = (0.1 * torch.randn(N, device="cuda")).to(torch.bfloat16)
    A = (torch.randn(r, K, device="cuda") / K ** 0.5).to(torch.bfloat16).requires_grad_(True)
    B = (0.3 * torch.randn(N, r, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    y = ops.lora_linear(x, w, b, A, B, s)
    gy = torch.randn(M_, N, device="cuda").to(torch.bfloat16)
    gx, gA, gB = torch.autograd.grad(y, (x, A, B), gy)
    xf, Af, Bf = (t.detach().float().requires_grad_(True) for t in (x, A, B))
    yf = xf @ w.float().t() + b.float() + (xf @ Af.t()) @ Bf.t() * s
    wx, wA, wB = torch.autograd.grad(yf, (xf, Af, Bf), gy.float())
    assert (y.float() - yf).abs().max().item() <= 2e-2 * yf.abs().max().item()
    for got, want in ((gx, wx), (gA, wA), (gB, wB)):
        assert (got.float() - want).abs().max().item() <= 2e-2 * want.abs().max().item() + 1e-3


def test_fp8_ffn_as_one_step_matches_the_two_projection_path():
    """fc1 handing gelu(.) to fc2 as e4m3 (no bf16 copy, gelu(z) rebuilt in the backward pass) against the two separate
    Fp8Linear calls: same arithmetic up to the rounding of the activation before its e4m3 cast."""
    from mint_plus_b200.mu_scaling import Fp8Linear, fp8_ffn
    torch.manual_seed(6)
    E, F_, M_ = 256, 1024, 300
    fc1, fc2 = Fp8Linear(E, F_).cuda().to(torch.bfloat16), Fp8Linear(F_, E).cuda().to(torch.bfloat16)
    with torch.no_grad():
        fc1.weight.normal_(0, 1); fc2.weight.normal_(0, 1)
        fc1.bias.normal_(0, 0.1); fc2.bias.normal_(0, 0.1)
    fc1.out_scale, fc2.out_scale = E ** -0.5, F_ ** -0.5
    x = torch.randn(M_, 1, E, device="cuda").to(torch.bfloat16)
    gy = torch.randn(M_, 1, E, device="cuda").to(torch.bfloat16)
    res = []
    for fused in (False, True):
        xi = x.clone().requires_grad_(True)
        for p in list(fc1.parameters()) + list(fc2.parameters()):
            p.grad = None
        y = fp8_ffn(fc1, fc2, xi) if fused else fc2(fc1(xi, gelu=True))
        y.backward(gy)
        res.append([y.detach().float(), xi.grad.float()] + [p.grad.float() for p in (fc1.weight, fc1.bias, fc2.weight, fc2.bias)])
    ops.check_device_status()
    for a, b, n in zip(res[1], res[0], ("y", "dx", "dW1", "db1", "dW2", "db2")):
        err, scale = (a - b).abs().max().item(), b.abs().max().item()
        assert err <= 3e-2 * scale + 1e-3, f"{n}: {err:.4g} vs scale {scale:.4g}"


def test_e4m3_cast_saturates_finite_values_and_keeps_nan():
    """A diverged run must stay visible: NaN activations stay NaN through the e4m3 cast (a clamp would turn them into -448)."""
    x = torch.tensor([0.5, -3.0, 1e6, -1e6, float("nan"), float("inf"), 448.0, 20.0] * 4, dtype=torch.bfloat16, device=DEV)
    q = ops.quantize_e4m3(x, 1.0).float().cpu()
    want = torch.tensor([0.5, -3.0, 448.0, -448.0, float("nan"), 448.0, 448.0, 20.0] * 4)
    assert torch.equal(torch.isnan(q), torch.isnan(want))
    assert torch.equal(q[~torch.isnan(q)], want[~torch.isnan(want)])
    # and through a projection: one NaN in x poisons its output row, the other rows stay finite
    xm = torch.randn(64, 128, device=DEV).to(torch.bfloat16)
    xm[3, 5] = float("nan")
    w = ops.quantize_e4m3(torch.randn(64, 128, device=DEV).to(torch.bfloat16), 1.0)
    y = ops.gemm_e4m3(ops.quantize_e4m3(xm, 1.0), w, 1.0).float()
    assert torch.isnan(y[3]).all() and torch.isfinite(y[:3]).all() and torch.isfinite(y[4:]).all()


def test_fp8_weight_cache_follows_in_place_updates_and_refresh():
    from mint_plus_b200.mu_scaling import Fp8Linear, refresh_fp8_weights
    torch.manual_seed(2)
    lin = Fp8Linear(128, 64).cuda().to(torch.bfloat16)
    with torch.no_grad():
        lin.weight.normal_(0, 1)
    x = torch.randn(32, 128, device=DEV).to(torch.bfloat16)
    y0 = lin(x).float()
    with torch.no_grad():
        lin.weight.mul_(2.0)                        # in place on the Parameter: the version counter moves, the cache follows
    y1 = lin(x).float()
    assert (y1 - 2 * y0).abs().max().item() <= 2e-2 * y1.abs().max().item()
    lin.weight.data.mul_(0.5)                       # an in-place write through .data is invisible to the cache ...
    assert torch.equal(lin(x).float(), y1)
    refresh_fp8_weights(lin)                        # ... until it is dropped
    y2 = lin(x).float()
    assert (y2 - y0).abs().max().item() <= 2e-2 * y0.abs().max().item()


@pytest.mark.gpu
def test_fp8_weight_scaler_uses_the_maxima_of_the_refresh_before():
    """Fp8WeightScaler.refresh(): the first refresh reads its maxima back, every later one casts with the maxima the
    refresh before it measured (no host read in the step), and the forward pass then finds fresh copies."""
    import mint_plus_b200 as M
    from mint_plus_b200 import mu_scaling as MU
    torch.manual_seed(5)
    model = torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.Linear(128, 64)).cuda().bfloat16()
    model[0] = M.Fp8Linear.from_linear(model[0])
    model[1] = M.Fp8Linear.from_linear(model[1])
    sc = M.Fp8WeightScaler(model)
    sc.refresh()
    a0 = [float(m.weight.abs().amax()) for m in model]
    for m, a in zip(model, a0):
        assert m._w_scale == pytest.approx(a / 448.0)
        assert m._wq_key == (m.weight.data_ptr(), m.weight._version, m.weight.device)      # the forward pass will not re-cast
    with torch.no_grad():
        for m in model:
            m.weight.mul_(2.0)
    sc.refresh()                                      # weights doubled, scales still from the maxima before
    for m, a in zip(model, a0):
        assert m._w_scale == pytest.approx(a / 448.0)
        want = (m.weight.float() / m._w_scale).clamp(-448, 448).to(torch.float8_e4m3fn)
        assert torch.equal(m._wq.view(torch.uint8), want.view(torch.uint8))
    sc.refresh()                                      # now the doubled maxima have arrived
    for m, a in zip(model, a0):
        assert m._w_scale == pytest.approx(2.0 * a / 448.0)
    x = torch.randn(32, 64, device="cuda").bfloat16()
    y = model(x)
    ref = torch.nn.functional.linear(torch.nn.functional.linear(x.float(), model[0].weight.float(), model[0].bias.float()),
                                     model[1].weight.float(), model[1].bias.float())
    assert (y.float() - ref).abs().max() <= 0.08 * ref.abs().max()
