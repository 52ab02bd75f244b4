"""CPU restatement of one MINT layer with the rounding points of the bf16 / e4m3 GPU path.

TEST INFRASTRUCTURE ONLY.  Tests import it as the checker of the layer-level GPU path; the product package
never does.  It composes, on the CPU in fp32,

  * the projections          nn.Linear arithmetic, or the per-tensor-scaled e4m3 arithmetic of
                             mint_plus/models/alt/munit_scaling.py:22-34 (`fp8_e4m3_linear` of this package) with the
                             straight-through gradients of lines 36-55 taken on the un-quantised operands,
  * the attention            `oracle.multimer_attention` (mint_plus/models/modules.py:129-144, mu_scaling/layer.py:159-165),
  * the layer glue           Pre-LN (mint_plus/models/modules.py:179-195) or muS Res-Post-LN
                             (mint_plus/models/mu_scaling/layer.py:259-280),

and rounds every tensor that the GPU path stores as bf16 to bf16 (straight-through for autograd), so that a GPU layer
can be compared at a tolerance of a few bf16 steps instead of the accumulated quantisation error of the number format.
FP8 parity is unpinned: transformer_engine 2.16.0, which holds the production FP8 arithmetic, is neither vendored in the
reference nor installed here; the e4m3 branch checks the restated formula only.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F

from . import multimer_attention as O

E4M3_MAX = 448.0
E5M2_MAX = 57344.0


class _RoundBf16(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return x.bfloat16().float()

    @staticmethod
    def backward(ctx, g):
        return g


def bf16r(x: torch.Tensor) -> torch.Tensor:
    """Round to bf16 (kept as fp32); the gradient passes straight through."""
    return _RoundBf16.apply(x)


def weight_scale(*weights: torch.Tensor) -> float:
    """Per-tensor e4m3 scale amax / 448 of one weight, or of several that share a scale (fused Q/K/V)."""
    return max(max(float(w.detach().abs().amax()) for w in weights), 1e-12) / E4M3_MAX


def quant_e4m3(x: torch.Tensor, scale: float) -> torch.Tensor:
    """saturate(x * (1 / scale)) rounded to e4m3, returned as fp32 (still divided by the scale)."""
    inv = torch.tensor(1.0 / scale, dtype=torch.float32)
    return (x.float() * inv).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).float()


def quant_e5m2(g: torch.Tensor, scale: float) -> torch.Tensor:
    """saturate(g * (1 / scale)) rounded to e5m2, returned as fp32 (still divided by the scale)."""
    inv = torch.tensor(1.0 / scale, dtype=torch.float32)
    return (g.float() * inv).clamp(-E5M2_MAX, E5M2_MAX).to(torch.float8_e5m2).float()


class _QuantLinear(torch.autograd.Function):
    """y = (x_scale w_scale out_scale) q(x) q(w)^T + b, or with a residual ra r + rb y (the sum the GEMM epilogue forms).
    Backward, g_scale None: as for y = out_scale x w^T + b on the un-quantised operands (straight-through).  With g_scale
    (alt/munit_scaling.py:36-55): the gradient of the result (of the SUM when there is a residual) is cast to e5m2,
    g8 = q5(dy / g_scale), and dx = g8 q(w), dw = g8^T q(x), db = sum g8, each times its scales (and rb); the residual
    receives ra dy."""

    @staticmethod
    def forward(ctx, x, w, b, x_scale, w_scale, out_scale, g_scale, resid=None, ra=1.0, rb=1.0):
        alpha = torch.tensor(float(x_scale) * float(w_scale) * float(out_scale), dtype=torch.float32)
        y = (quant_e4m3(x, x_scale) @ quant_e4m3(w, w_scale).t()) * alpha
        if b is not None:
            y = y + b.float()
        if resid is not None:
            y = ra * resid + rb * y
        ctx.save_for_backward(x, w)
        ctx.cfg = (float(x_scale), float(w_scale), float(out_scale), g_scale, float(ra), float(rb) if resid is not None else 1.0)
        ctx.has_bias, ctx.has_res = b is not None, resid is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        x_scale, w_scale, out_scale, g_scale, ra, rb = ctx.cfg
        if g_scale is None:
            dx = (dy @ w) * (out_scale * rb)
            dw = (dy.t() @ x) * (out_scale * rb)
            db = dy.sum(0) * rb if ctx.has_bias else None
        else:
            g8 = quant_e5m2(dy, g_scale)
            # (the product leaves the GPU as bf16, and the next projection's e5m2 cast sees that rounding)
            dx = ((g8 @ quant_e4m3(w, w_scale)) * torch.tensor(g_scale * w_scale * out_scale * rb, dtype=torch.float32)).bfloat16().float()
            dw = (g8.t() @ quant_e4m3(x, x_scale)) * torch.tensor(g_scale * x_scale * out_scale * rb, dtype=torch.float32)
            db = g8.sum(0) * (g_scale * rb) if ctx.has_bias else None
        return dx, dw, db, None, None, None, None, (ra * dy if ctx.has_res else None), None, None


class _GeluKeepsBf16Preactivation(torch.autograd.Function):
    """gelu_erf(z) computed from the fp32 pre-activation (the GEMM epilogue), differentiated at the bf16 copy of z that the
    forward pass keeps for the backward pass."""

    @staticmethod
    def forward(ctx, z):
        ctx.save_for_backward(z.bfloat16().float())
        return O.gelu_erf(z)

    @staticmethod
    def backward(ctx, dy):
        (zb,) = ctx.saved_tensors
        return dy * (0.5 * (1.0 + torch.erf(zb * 0.7071067811865476)) + zb * torch.exp(-0.5 * zb * zb) * 0.3989422804014327)


def linear(x2d, w, b, fp8: Optional[dict] = None, w_scale: Optional[float] = None, name: Optional[str] = None, residual=None):
    """fp32 result of one projection on rows x2d [M,K] (not yet rounded to bf16).  `fp8` = {"x_scale", "out_scale", "g_scale"}
    selects the e4m3 arithmetic (g_scale: the 8-bit backward as well); an entry fp8["per"][name] overrides those fields for
    the projection `name` ("sa_qkv", "ma_qkv", "out", "fc1", "fc2").  `w_scale` overrides amax(w)/448."""
    if fp8 is None:
        y = F.linear(x2d, w, b)
        return y if residual is None else residual[1] * residual[0] + residual[2] * y
    cfg = dict(fp8)
    cfg.update(fp8.get("per", {}).get(name, {}))
    ws = weight_scale(w) if w_scale is None else w_scale
    res = (None, 1.0, 1.0) if residual is None else residual
    return _QuantLinear.apply(x2d, w, b, cfg.get("x_scale", 1.0), ws, cfg.get("out_scale", 1.0), cfg.get("g_scale"), *res)


def _heads(t2d, T, B, H, D):
    return t2d.reshape(T, B, H, D).permute(1, 2, 0, 3)


def _qkv(attn, x2d, T, B, H, D, rope: bool, fp8, name):
    """q, k, v (B,H,T,D) of one pathway as the fused QKV GEMM leaves them: bias added, q and k rotated in fp32, then bf16."""
    if getattr(attn, "fused_qkv", None) is not None:
        w, b = attn.fused_qkv.weight, attn.fused_qkv.bias
    else:
        w = torch.cat([attn.q_proj.weight, attn.k_proj.weight, attn.v_proj.weight], dim=0)
        b = torch.cat([attn.q_proj.bias, attn.k_proj.bias, attn.v_proj.bias], dim=0) if attn.q_proj.bias is not None else None
    qkv = linear(x2d, w, b, fp8, name=name)
    q, k, v = (_heads(t, T, B, H, D) for t in qkv.chunk(3, dim=-1))
    if rope:
        q, k = O.apply_rope(q), O.apply_rope(k)
    return bf16r(q), bf16r(k), bf16r(v)


def attention_block(layer, x, chain_mask, key_pad, fp8=None, sqrt_softmax=False, residual=None):
    """x (T,B,E) -> out_proj(attention) (T,B,E), every stored tensor rounded to bf16.  `residual` = (r, a, b): the result is
    a r + b out_proj(attention), formed in fp32 from the unrounded projection (the GEMM epilogue adds the residual) and
    rounded once."""
    T, B, E = x.shape
    sa, ma = layer.self_attn, layer.multimer_attn
    H = sa.num_heads
    D = E // H
    x2d = x.reshape(T * B, E)
    q_s, k_s, v_s = _qkv(sa, x2d, T, B, H, D, sa.rot_emb is not None, fp8, "sa_qkv")
    q_c, k_c, v_c = _qkv(ma, x2d, T, B, H, D, False, fp8, "ma_qkv")
    a = O.multimer_attention(q_s, k_s, v_s, q_c, k_c, v_c, chain_mask, key_pad, scale=D ** -0.5, rope=False,
                             sqrt_softmax=sqrt_softmax)
    a = bf16r(a.permute(2, 0, 1, 3).reshape(T * B, E))
    res = None if residual is None else (residual[0].reshape(T * B, E), residual[1], residual[2])
    return bf16r(linear(a, sa.out_proj.weight, sa.out_proj.bias, fp8, name="out", residual=res)).reshape(T, B, E)


def feed_forward(layer, x, fp8=None):
    """fc2(gelu_erf(fc1(x))).  bf16 path: gelu(.) is stored as bf16 between the products; e4m3 path: fc1's epilogue casts
    gelu(.) straight to fc2's e4m3 operand from the fp32 value (fc2's activation scale), no bf16 copy in between."""
    T, B, E = x.shape
    ff = layer.feed_forward
    z = linear(x.reshape(T * B, E), ff.fc1.weight, ff.fc1.bias, fp8, name="fc1")
    g = _GeluKeepsBf16Preactivation.apply(z)
    if fp8 is None:
        g = bf16r(g)
    return bf16r(linear(g, ff.fc2.weight, ff.fc2.bias, fp8, name="fc2")).reshape(T, B, E)


def mu_layer(layer, x, chain_mask, key_pad, tau: float, fp8=None, sqrt_softmax=False):
    """muS Res-Post-LN layer (mu_scaling/layer.py:259-280): x = sqrt(1-tau) x + sqrt(tau) attn(x);
    x = sqrt(1-tau) x + sqrt(tau) ffn(x); LayerNorm.  The first residual sum leaves the output projection's epilogue as bf16,
    the second feeds the LayerNorm in fp32, as the fused residual + LayerNorm pass computes it."""
    keep, add = math.sqrt(1.0 - tau), math.sqrt(tau)
    s1 = attention_block(layer, x, chain_mask, key_pad, fp8, sqrt_softmax, residual=(x, keep, add))
    s2 = keep * s1 + add * feed_forward(layer, s1, fp8)
    ln = layer.final_layer_norm
    return bf16r(F.layer_norm(s2, (s2.shape[-1],), ln.weight, ln.bias, ln.eps))


def pre_ln_layer(layer, x, chain_mask, key_pad, fp8=None):
    """Pre-LN layer (modules.py:179-195): x + attn(LN(x)), then + ffn(LN(.)); LayerNorm results and the residual sums
    are stored as bf16 (the second LayerNorm reads the stored first sum)."""
    E = x.shape[-1]
    n1, n2 = layer.self_attn_layer_norm, layer.final_layer_norm
    h = bf16r(F.layer_norm(x, (E,), n1.weight, n1.bias, n1.eps))
    y = attention_block(layer, h, chain_mask, key_pad, fp8, residual=(x, 1.0, 1.0))
    h2 = bf16r(F.layer_norm(y, (E,), n2.weight, n2.bias, n2.eps))
    return bf16r(y + feed_forward(layer, h2, fp8))
