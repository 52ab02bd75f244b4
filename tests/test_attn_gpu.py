"""Parity of the CUDA attention path (called through the C ABI) with the CPU oracle and the golden vectors."""
import math

import pytest
import torch

from conftest import golden_cases, load_golden
from oracle import multimer_attention as O

pytestmark = pytest.mark.gpu

import mint_plus_b200 as M  # noqa: E402
from mint_plus_b200 import ops  # noqa: E402

DEV = "cuda"
# Tolerances.  fp32 kernels vs fp32 oracle: 1e-5 relative (plus a small absolute floor for values near zero).
# bf16 kernels vs the fp32 oracle evaluated on the same bf16-rounded inputs: 2e-2 max-abs on attention outputs;
# gradients carry the same bf16 rounding of P, dS and of the stored result, checked relative to their scale.
F32_RTOL, F32_ATOL = 1e-5, 2e-6
BF16_OUT_ATOL = 2e-2
BF16_GRAD_REL = 2e-2


def _run(ts, grad, dtype, **kw):
    leaves = [t.to(DEV, dtype).requires_grad_(True) for t in ts]
    out = M.multimer_attention(*leaves, **kw)
    grads = torch.autograd.grad(out, leaves, grad.to(DEV, dtype))
    ops.check_device_status()
    return out.detach().float().cpu(), [g.float().cpu() for g in grads]


def _assert_grads(got, want, dtype, names=("dq_s", "dk_s", "dv_s", "dq_c", "dk_c", "dv_c")):
    for g, w, n in zip(got, want, names):
        if dtype == torch.float32:
            torch.testing.assert_close(g, w, rtol=1e-4, atol=5e-6, msg=lambda m: f"{n}: {m}")
        else:
            scale = w.abs().max().item()
            err = (g - w).abs().max().item()
            # relative to the gradient's scale, with an absolute floor for gradients that are exactly zero
            assert err <= BF16_GRAD_REL * scale + 1e-5, f"{n}: max err {err:.4g} vs scale {scale:.4g}"


@pytest.mark.parametrize("force_simt", [True, False])
@pytest.mark.parametrize("name", golden_cases())
def test_golden_fp32(name, force_simt):
    g = load_golden(name)
    ts = [g[k] for k in ("q_s", "k_s", "v_s", "q_c", "k_c", "v_c")]
    out, grads = _run(ts, g["grad_out"], torch.float32, chain_ids=g["chain_ids"].to(DEV),
                      key_padding_mask=g["key_pad"].to(DEV), rope=True, force_simt=force_simt,
                      sqrt_softmax=bool(g["sqrt_softmax"]))
    torch.testing.assert_close(out, g["out"], rtol=F32_RTOL, atol=F32_ATOL)
    _assert_grads(grads, [g[k] for k in ("dq_s", "dk_s", "dv_s", "dq_c", "dk_c", "dv_c")], torch.float32)


@pytest.mark.parametrize("force_simt", [True, False])
@pytest.mark.parametrize("name", golden_cases())
def test_golden_bf16(name, force_simt):
    g = load_golden(name)
    sq = bool(g["sqrt_softmax"])
    ts = [g[k].bfloat16().float() for k in ("q_s", "k_s", "v_s", "q_c", "k_c", "v_c")]
    go = g["grad_out"].bfloat16().float()
    mask = O.chain_mask_from_ids(g["chain_ids"])
    want, wgrads = O.multimer_attention_fwd_bwd(*ts, mask, go, key_pad=g["key_pad"], sqrt_softmax=sq)
    out, grads = _run(ts, go, torch.bfloat16, chain_ids=g["chain_ids"].to(DEV),
                      key_padding_mask=g["key_pad"].to(DEV), rope=True, force_simt=force_simt, sqrt_softmax=sq)
    # sqrt(p) sums to more than one, so those outputs are several units large and one bf16 step of the result alone is
    # 1.6e-2 at 3; the 2e-2 bound is therefore taken relative to the largest output there
    tol = BF16_OUT_ATOL * (max(1.0, want.abs().max().item()) if sq else 1.0)
    assert (out - want).abs().max().item() <= tol
    # and against the reference's own vectors (inputs differ by bf16 rounding only)
    assert (out - g["out"]).abs().max().item() <= 2 * tol
    _assert_grads(grads, wgrads, torch.bfloat16)


# shapes of the reference's own kernel tests (profiles/test_sqrt_softmax.py:101-106) plus ragged ones
SHAPES = [(2, 4, 64, 16), (4, 20, 128, 32), (2, 20, 256, 32), (2, 3, 200, 64), (1, 2, 77, 32), (1, 1, 1, 16),
          (2, 2, 129, 64), (1, 2, 383, 32)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", SHAPES)
def test_seeded_inputs_against_oracle(shape, dtype):
    B, H, T, D = shape
    ts, cid, pad, grad = O.make_op_inputs(B, H, T, D, seed=42 + 100 * B + 10 * H + T, max_pad=min(64, T // 4))
    if dtype == torch.bfloat16:
        ts, grad = [t.bfloat16().float() for t in ts], grad.bfloat16().float()
    want, wgrads = O.multimer_attention_fwd_bwd(*ts, O.chain_mask_from_ids(cid), grad, key_pad=pad)
    out, grads = _run(ts, grad, dtype, chain_ids=cid.to(DEV), key_padding_mask=pad.to(DEV))
    if dtype == torch.float32:
        torch.testing.assert_close(out, want, rtol=F32_RTOL, atol=F32_ATOL)
    else:
        assert (out - want).abs().max().item() <= BF16_OUT_ATOL
    _assert_grads(grads, wgrads, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(2, 4, 64, 16), (2, 3, 200, 64), (1, 2, 383, 32), (2, 2, 300, 32)])
def test_sqrt_softmax_against_oracle(shape, dtype):
    """out = sum_j sqrt(p_j) v_j (mu_scaling/layer.py:162-163), with padded keys (gradient 0 there)."""
    B, H, T, D = shape
    ts, cid, pad, grad = O.make_op_inputs(B, H, T, D, seed=900 + T, max_pad=min(64, T // 4))
    if dtype == torch.bfloat16:
        ts, grad = [t.bfloat16().float() for t in ts], grad.bfloat16().float()
    want, wgrads = O.multimer_attention_fwd_bwd(*ts, O.chain_mask_from_ids(cid), grad, key_pad=pad, sqrt_softmax=True)
    out, grads = _run(ts, grad, dtype, chain_ids=cid.to(DEV), key_padding_mask=pad.to(DEV), sqrt_softmax=True)
    if dtype == torch.float32:
        torch.testing.assert_close(out, want, rtol=F32_RTOL, atol=F32_ATOL)
    else:
        assert (out - want).abs().max().item() <= BF16_OUT_ATOL * max(1.0, want.abs().max().item())   # outputs exceed 1
    _assert_grads(grads, wgrads, dtype)


def _edge_masks(T):
    cases = {}
    cid = torch.zeros(1, T, dtype=torch.int32)
    cases["single_chain"] = (cid.clone(), None)
    c = cid.clone(); c[:, 64:] = 1
    cases["split_on_tile_boundary"] = (c, None)
    c = cid.clone(); c[:, 63:] = 1
    cases["split_before_boundary"] = (c, None)
    c = cid.clone(); c[:, 65:] = 1
    cases["split_after_boundary"] = (c, None)
    c = cid.clone(); c[:, 1::2] = 1
    cases["alternating"] = (c, None)
    c = cid.clone(); c[:, T // 2:] = 1
    p = torch.zeros(1, T, dtype=torch.bool); p[:, T // 2 - 9:T // 2] = True; p[:, -64:] = True
    cases["pads_mid_and_full_tail_tile"] = (c, p)
    p = torch.zeros(1, T, dtype=torch.bool); p[:, 1:] = True
    cases["one_real_key"] = (c, p)
    c = torch.arange(T, dtype=torch.int32)[None] // 50
    cases["many_chains"] = (c, None)
    return cases


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", list(_edge_masks(200)))
def test_edge_masks(case, dtype):
    T, H, D = 200, 2, 32
    cid, pad = _edge_masks(T)[case]
    ts, _, _, grad = O.make_op_inputs(1, H, T, D, seed=7)
    if dtype == torch.bfloat16:
        ts, grad = [t.bfloat16().float() for t in ts], grad.bfloat16().float()
    want, wgrads = O.multimer_attention_fwd_bwd(*ts, O.chain_mask_from_ids(cid), grad, key_pad=pad)
    out, grads = _run(ts, grad, dtype, chain_ids=cid.to(DEV), key_padding_mask=None if pad is None else pad.to(DEV))
    if dtype == torch.float32:
        torch.testing.assert_close(out, want, rtol=F32_RTOL, atol=F32_ATOL)
    else:
        assert (out - want).abs().max().item() <= BF16_OUT_ATOL
    _assert_grads(grads, wgrads, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_reference_signature_with_arbitrary_mask(dtype):
    """fused_multi_pathway_attention: pre-scaled, pre-rotated inputs and a non-symmetric Bernoulli(0.4) mask with
    the diagonal forced intra (profiles/test_fused_attention.py:60-61 of the reference)."""
    B, H, T, D = 2, 4, 160, 32
    g = torch.Generator().manual_seed(3)
    ts = [torch.randn(B, H, T, D, generator=g) for _ in range(6)]
    ts[0] *= D ** -0.5
    ts[3] *= D ** -0.5
    mask = torch.rand(B, T, T, generator=g) < 0.4
    mask[:, torch.arange(T), torch.arange(T)] = False
    grad = torch.randn(B, H, T, D, generator=g)
    if dtype == torch.bfloat16:
        ts, grad = [t.bfloat16().float() for t in ts], grad.bfloat16().float()
    want, wgrads = O.multimer_attention_fwd_bwd(*ts, mask, grad, scale=1.0, rope=False)
    leaves = [t.to(DEV, dtype).requires_grad_(True) for t in ts]
    out = M.differentiable_multi_pathway_attention(*leaves, mask.to(DEV))
    grads = torch.autograd.grad(out, leaves, grad.to(DEV, dtype))
    ops.check_device_status()
    if dtype == torch.float32:
        torch.testing.assert_close(out.float().cpu(), want, rtol=F32_RTOL, atol=F32_ATOL)
    else:
        assert (out.float().cpu() - want).abs().max().item() <= BF16_OUT_ATOL
    _assert_grads([x.float().cpu() for x in grads], wgrads, dtype)


def test_mask_metadata_bits_are_exact():
    B, T = 3, 150
    g = torch.Generator().manual_seed(9)
    cid = torch.randint(0, 3, (B, T), generator=g, dtype=torch.int32)
    pad = torch.rand(B, T, generator=g) < 0.2
    meta = M.mask_meta_from_chain_ids(cid.to(DEV), pad.to(DEV))
    mask = O.chain_mask_from_ids(cid)
    meta2 = M.mask_meta_from_mask(mask.to(DEV), pad.to(DEV))
    TW = ((T + 31) // 32 + 3) // 4 * 4
    a256 = lambda x: (x + 255) // 256 * 256
    nbits, nkpad, ncls = B * T * TW * 4, B * TW * 4, B * ((T + 63) // 64) ** 2
    regions = [(0, nbits), (a256(nbits), nbits), (2 * a256(nbits), nkpad), (2 * a256(nbits) + a256(nkpad), ncls)]
    for off, n in regions:                       # the gaps between the 256-byte aligned arrays are never written
        assert torch.equal(meta.buf[off:off + n], meta2.buf[off:off + n])
    words = meta.buf[:B * T * TW * 4].view(torch.int32).view(B, T, TW).cpu()
    bits = ((words[..., None] >> torch.arange(32)) & 1).reshape(B, T, TW * 32)[:, :, :T].bool()
    assert torch.equal(bits, mask)
    # an asymmetric mask: the key-major copy is the transpose
    am = torch.rand(B, T, T, generator=g) < 0.5
    meta3 = M.mask_meta_from_mask(am.to(DEV))
    n = (B * T * TW * 4 + 255) // 256 * 256
    wt = meta3.buf[n:n + B * T * TW * 4].view(torch.int32).view(B, T, TW).cpu()
    bt = ((wt[..., None] >> torch.arange(32)) & 1).reshape(B, T, TW * 32)[:, :, :T].bool()
    assert torch.equal(bt, am.transpose(1, 2))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_forward_is_deterministic_and_padded_keys_are_inert(dtype):
    ts, cid, pad, _ = O.make_op_inputs(2, 4, 300, 32, seed=11, max_pad=40)
    pad[0, -7:] = True
    dts = [t.to(DEV, dtype) for t in ts]
    kw = dict(chain_ids=cid.to(DEV), key_padding_mask=pad.to(DEV))
    a = M.multimer_attention(*dts, **kw)
    b = M.multimer_attention(*dts, **kw)
    assert torch.equal(a, b)
    poisoned = [t.clone() for t in dts]
    for idx in (1, 2, 4, 5):                      # K and V of both pathways at padded positions
        poisoned[idx][pad.to(DEV)[:, None, :].expand(-1, 4, -1)] = 1e4
    c = M.multimer_attention(*poisoned, **kw)
    assert torch.equal(a, c)
    assert torch.isfinite(a).all()


@pytest.mark.parametrize("D", [32, 64])
def test_full_size_properties(D):
    """Benchmark-size inputs (B8 H20 T1024): rows of P sum to one, V-linearity, tensor-core path vs fp32 path."""
    B, H, T = 8, 20, 1024
    ts, cid, pad, grad = O.make_op_inputs(B, H, T, D, seed=2002)
    dts = [t.to(DEV, torch.bfloat16) for t in ts]
    kw = dict(chain_ids=cid.to(DEV), key_padding_mask=pad.to(DEV))
    ones = torch.ones_like(dts[2])
    s = M.multimer_attention(dts[0], dts[1], ones, dts[3], dts[4], ones, **kw).float()
    assert (s - 1).abs().max().item() <= 1e-2
    out = M.multimer_attention(*dts, **kw).float()
    ref = M.multimer_attention(*dts, force_simt=True, **kw).float()
    assert (out - ref).abs().max().item() <= BF16_OUT_ATOL
    half = [dts[0], dts[1], (dts[2].float() * 0.5).bfloat16(), dts[3], dts[4], (dts[5].float() * 0.5).bfloat16()]
    lin = M.multimer_attention(*half, **kw).float()
    assert (2 * lin - out).abs().max().item() <= BF16_OUT_ATOL
    # gradients of the two kernel families agree
    leaves = [t.clone().requires_grad_(True) for t in dts]
    go = grad.to(DEV, torch.bfloat16)
    g1 = torch.autograd.grad(M.multimer_attention(*leaves, **kw), leaves, go)
    g2 = torch.autograd.grad(M.multimer_attention(*leaves, force_simt=True, **kw), leaves, go)
    ops.check_device_status()
    for a, b in zip(g1, g2):
        scale = b.float().abs().max().item()
        assert (a.float() - b.float()).abs().max().item() <= BF16_GRAD_REL * scale


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_combine_from_materialised_logits(dtype):
    B, H, T, D = 2, 3, 70, 32
    ts, cid, pad, grad = O.make_op_inputs(B, H, T, D, seed=21, max_pad=6)
    mask = O.chain_mask_from_ids(cid)
    il = O.combined_logits(ts[0], ts[1], ts[3], ts[4], torch.zeros_like(mask), pad)
    el = O.combined_logits(ts[0], ts[1], ts[3], ts[4], torch.ones_like(mask), pad)
    if dtype == torch.bfloat16:
        il, el, ts, grad = il.bfloat16().float(), el.bfloat16().float(), [t.bfloat16().float() for t in ts], grad.bfloat16().float()
    leaves = [t.clone().requires_grad_(True) for t in (il, el, ts[2], ts[5])]
    want = O.combine_from_logits(leaves[0], leaves[1], mask, leaves[2], leaves[3])
    wg = torch.autograd.grad(want, leaves, grad)
    dl = [t.detach().to(DEV, dtype).requires_grad_(True) for t in (il, el, ts[2], ts[5])]
    out = M.differentiable_multimer_combine(dl[0], dl[1], mask.to(DEV), dl[2], dl[3])
    gg = torch.autograd.grad(out, dl, grad.to(DEV, dtype))
    if dtype == torch.float32:
        torch.testing.assert_close(out.cpu(), want.detach(), rtol=F32_RTOL, atol=F32_ATOL)
        for a, b in zip(gg, wg):
            torch.testing.assert_close(a.cpu(), b, rtol=1e-4, atol=5e-6)
    else:
        assert (out.float().cpu() - want.detach()).abs().max().item() <= BF16_OUT_ATOL
        for a, b in zip(gg, wg):
            assert (a.float().cpu() - b).abs().max().item() <= BF16_GRAD_REL * (b.abs().max().item() + 1e-6)


def test_layer_forward_backward_matches_oracle_composition():
    """TransformerLayer_MINT_plus on the GPU vs the same layer evaluated with the oracle attention on the CPU."""
    torch.manual_seed(5)
    E, H, T, B = 64, 4, 90, 2
    layer = M.TransformerLayer_MINT_plus(E, 4 * E, H, use_multimer=True, use_erf_gelu=True).float()
    x = torch.randn(T, B, E)
    cid = torch.zeros(B, T, dtype=torch.int32); cid[:, 40:] = 1
    pad = torch.zeros(B, T, dtype=torch.bool); pad[1, -11:] = True
    mask = O.chain_mask_from_ids(cid)

    def cpu_forward(x):
        h = layer.self_attn_layer_norm(x)
        qs, ks, vs = layer.self_attn.project_qkv_4d(h)
        qc, kc, vc = layer.multimer_attn.project_qkv_4d(h)
        a = O.multimer_attention(qs, ks, vs, qc, kc, vc, mask, pad)
        a = layer.self_attn.out_proj(a.permute(2, 0, 1, 3).reshape(T, B, E))
        y = x + a
        return y + layer.feed_forward(layer.final_layer_norm(y))

    xc = x.clone().requires_grad_(True)
    want = cpu_forward(xc)
    want.sum().backward()
    wgrad_x = xc.grad.clone()
    wgrad_w = layer.multimer_attn.fused_qkv.weight.grad.clone()
    layer.zero_grad()
    glayer = layer.to(DEV)
    xg = x.to(DEV).requires_grad_(True)
    out, _ = glayer(xg, self_attn_mask=mask.to(DEV), self_attn_padding_mask=pad.to(DEV))
    out.sum().backward()
    torch.testing.assert_close(out.detach().cpu(), want.detach(), rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(xg.grad.cpu(), wgrad_x, rtol=1e-3, atol=1e-4)
    torch.testing.assert_close(glayer.multimer_attn.fused_qkv.weight.grad.cpu(), wgrad_w, rtol=1e-3, atol=1e-4)
    layer.to("cpu")


@pytest.mark.parametrize("dtype,force_simt", [(torch.float32, False), (torch.bfloat16, False), (torch.bfloat16, True)])
@pytest.mark.parametrize("shape", [(2, 3, 200, 64), (2, 4, 130, 32), (1, 2, 77, 16)])
def test_sequence_first_output_layout(shape, dtype, force_simt):
    """out_seq_first writes (T,B,H,D) and takes the upstream gradient in that layout: same numbers, no permute copies."""
    B, H, T, D = shape
    ts, cid, pad, grad = O.make_op_inputs(B, H, T, D, seed=5 + T, max_pad=T // 5)
    kw = dict(chain_ids=cid.to(DEV), key_padding_mask=pad.to(DEV), force_simt=force_simt)
    leaves = [t.to(DEV, dtype).requires_grad_(True) for t in ts]
    out = M.multimer_attention(*leaves, **kw)
    g = grad.to(DEV, dtype)
    want = torch.autograd.grad(out, leaves, g)
    leaves2 = [t.to(DEV, dtype).requires_grad_(True) for t in ts]
    out2 = M.multimer_attention(*leaves2, out_seq_first=True, **kw)
    assert tuple(out2.shape) == (T, B, H, D) and out2.is_contiguous()
    torch.testing.assert_close(out2.permute(1, 2, 0, 3), out, rtol=0, atol=0)
    got = torch.autograd.grad(out2, leaves2, g.permute(2, 0, 1, 3).contiguous())
    ops.check_device_status()
    for a, b in zip(got, want):
        if dtype == torch.float32 or force_simt:
            torch.testing.assert_close(a, b, rtol=0, atol=0)          # deterministic kernels: bit-equal
        else:
            assert (a.float() - b.float()).abs().max().item() <= 1e-2 * b.float().abs().max().item() + 1e-6   # dQ atomics reorder


@pytest.mark.parametrize("sqrt_sm", [False, True])
@pytest.mark.parametrize("shape", [(2, 3, 300, 64), (3, 2, 200, 32), (2, 2, 130, 16)])
def test_backward_writes_row_major_gradients_and_packed_rows(shape, sqrt_sm):
    """MINTB_FLAG_QK_PREROTATED + MINTB_FLAG_GRAD_ROWMAJOR: for q, k of the self pathway rotated by the caller, the backward
    pass writes [dQ | dK | dV] of each pathway straight into a [T*B][3E] matrix, un-rotating dq_self / dk_self, and the
    values equal those of the ordinary call on the un-rotated tensors.  With a token-row map (mintb_attn_bwd_rows) only the
    unpadded tokens' rows exist, and they hold the same numbers."""
    B, H, T, D = shape
    E = H * D
    ts, cid, pad, grad = O.make_op_inputs(B, H, T, D, seed=11 + T, max_pad=T // 3)
    kw = dict(chain_ids=cid.to(DEV), key_padding_mask=pad.to(DEV), sqrt_softmax=sqrt_sm)
    dt = torch.bfloat16
    leaves = [t.to(DEV, dt).requires_grad_(True) for t in ts]
    out = M.multimer_attention(*leaves, **kw)                                  # rotates inside, scale D^-0.5
    g = grad.to(DEV, dt)
    want = torch.autograd.grad(out, leaves, g)

    cos, sin, _ = ops.rope_tables(T, D, torch.device(DEV))
    def rot(x):                                                                # rotary_embedding.py:16-24 on fp32 tables
        xf = x.float()
        x1, x2 = xf[..., : D // 2], xf[..., D // 2:]
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(dt)
    pre = [rot(leaves[0].detach()), rot(leaves[1].detach())] + [t.detach() for t in leaves[2:]]
    pre = [t.contiguous().requires_grad_(True) for t in pre]
    out2 = M.multimer_attention(*pre, rope=False, scale=D ** -0.5, out_seq_first=True, grad_rowmajor_tabs=(cos, sin), **kw)
    assert (out2.permute(1, 2, 0, 3).float() - out.float()).abs().max().item() <= 2e-2 * max(1.0, out.float().abs().max().item())
    got = torch.autograd.grad(out2, pre, g.permute(2, 0, 1, 3).contiguous())
    ops.check_device_status()
    g_s = ops._rowmajor_base(got[0], got[1], got[2], T, B, H, D)
    g_c = ops._rowmajor_base(got[3], got[4], got[5], T, B, H, D)
    assert g_s is not None and g_c is not None and tuple(g_s.shape) == (T * B, 3 * E)
    for a, b, n in zip(got, want, ("dq_s", "dk_s", "dv_s", "dq_c", "dk_c", "dv_c")):
        err, scale = (a.float() - b.float()).abs().max().item(), b.float().abs().max().item()
        assert err <= 3e-2 * scale + 1e-5, f"{n}: {err:.4g} vs scale {scale:.4g}"

    # the same backward pass with a token-row map: rows of the unpadded tokens only
    pack = ops.PackInfo(pad.to(DEV))
    meta = ops.mask_meta_from_chain_ids(cid.to(DEV), pad.to(DEV))
    flags = ops.L.FLAG_OUT_SEQ_FIRST | (ops.L.FLAG_SQRT_SOFTMAX if sqrt_sm else 0)
    ctx = ops._SubCtx((True,) * 6 + (False,) * 6)
    with torch.no_grad():
        out3 = ops._MultimerAttentionFn.forward(ctx, *[t.detach() for t in pre], meta, None, None, D ** -0.5, flags, (cos, sin))
        _, p_s, p_c = ops._attention_backward(ctx, g.permute(2, 0, 1, 3).contiguous(), pack)
    ops.check_device_status()
    torch.testing.assert_close(out3, out2, rtol=0, atol=0)
    assert tuple(p_s.shape) == (pack.n, 3 * E) and pack.n < T * B
    for packed, full in ((p_s, g_s), (p_c, g_c)):
        ref = full.index_select(0, pack.rows64)
        torch.testing.assert_close(packed[:, E:], ref[:, E:], rtol=0, atol=0)            # dK, dV: fixed-order sums
        assert (packed[:, :E].float() - ref[:, :E].float()).abs().max().item() <= 1e-2 * ref[:, :E].float().abs().max().item() + 1e-6


def test_back_to_back_calls_see_each_others_results_in_stream_order():
    """The small passes (rotation, statistics + accumulator clearing, dQ conversion) and the main kernels overlap their
    set-up with the pass before them (programmatic dependent launch).  Calls on two different input sets, issued back to
    back without a synchronisation in between (workspaces are handed back and forth by the caching allocator), must give what each set gives alone:
    outputs, dK and dV bit for bit (their sums have a fixed order), dQ within the run-to-run bound of its fp32 additions."""
    sets = []
    for seed in (11, 12):
        ts, cid, pad, grad = O.make_op_inputs(2, 4, 700, 32, seed=seed)
        leaves = [t.to(DEV, torch.bfloat16).requires_grad_(True) for t in ts]
        meta = M.mask_meta_from_chain_ids(cid.to(DEV), pad.to(DEV))
        sets.append((leaves, meta, grad.to(DEV, torch.bfloat16)))

    def step(s):
        leaves, meta, g = s
        out = M.multimer_attention(*leaves, meta=meta, rope=True)
        return out, torch.autograd.grad(out, leaves, g)

    alone = []
    for s in sets:
        out, grads = step(s)
        torch.cuda.synchronize()
        alone.append((out.clone(), [x.clone() for x in grads]))
    results = [step(sets[i % 2]) for i in range(24)]   # no synchronisation between the calls
    torch.cuda.synchronize()
    ops.check_device_status()
    for i, (out, grads) in enumerate(results):
        want_out, want = alone[i % 2]
        assert torch.equal(out, want_out), f"call {i}: output differs"
        for j, (g, w) in enumerate(zip(grads, want)):
            if j in (0, 3):   # dq_s, dq_c: fp32 additions in arrival order, then rounded to bf16
                scale = w.float().abs().max().item()
                assert (g.float() - w.float()).abs().max().item() <= 2e-2 * scale, f"call {i}: dq {j} differs"
            else:
                assert torch.equal(g, w), f"call {i}: gradient {j} differs"
