"""FP8 (e4m3, per-tensor scaled) projections and the helpers around them, with the reference's entry points
(mint_plus/models/mu_scaling/__init__.py:42-135 `apply_fp8_to_model`, mu_scaling/init.py:23-56 `unit_variance_init_`).

The reference swaps nn.Linear for transformer_engine's te.Linear; here the swap is to `Fp8Linear`, whose forward is the
tcgen05 e4m3 GEMM of libmintb: x and W are cast to e4m3 with one scale per tensor (saturating at +-448, as
mint_plus/models/alt/munit_scaling.py:22-34 states the arithmetic), accumulated in fp32, multiplied by the product of the
two scales, and bias / erf-GELU are applied in the GEMM epilogue.  The weight scale is amax(W)/448, refreshed when the weight
changes; the activation scale is static (1.0 by default, which suits unit-variance muS activations; `calibrate_fp8`
measures it on a sample batch otherwise).  The backward products run on the library's dgrad / wgrad GEMMs: in 8 bits by
default (e5m2 gradient with a static scale against the e4m3 operands, alt/munit_scaling.py:36-55), or in bf16 on the
master weights with `fp8_grads=False`.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
from torch import nn

from . import ops
from .attention import MultiHeadAttention
from .modules_plus import VanillaFeedForward, _TwoPathwayLayer

E4M3_MAX = 448.0


def _w_grad(g8, xq, alpha, like):
    dw = ops.gemm_wgrad(g8, xq, alpha=alpha, out_dtype=torch.float32 if like.dtype == torch.float32 else torch.bfloat16)
    return dw if dw.dtype == like.dtype else dw.to(like.dtype)


class _Fp8LinearFn(torch.autograd.Function):
    """y = act(out_scale x W^T + b) on e4m3 operands.  Backward: with a GradScale `gs` both products run in 8 bits — the
    gradient cast to e5m2 with the static scale, against the e4m3 weight (dgrad) and the e4m3 activation kept from the
    forward pass (wgrad), as mint_plus/models/alt/munit_scaling.py:36-55 states them; without one, in bf16 on the master
    weight and the bf16 activation."""

    @staticmethod
    def forward(ctx, x2d, weight, bias, wq, w_scale, x_scale, gelu, out_scale, gs):
        xq = ops.quantize_e4m3(x2d, x_scale)
        keep = gelu and any(ctx.needs_input_grad[:3])
        res = ops.gemm_e4m3(xq, wq, x_scale * w_scale * out_scale, bias, gelu, save_preact=keep)
        out, z = res if keep else (res, None)
        ctx.save_for_backward(xq if gs is not None else x2d, weight, bias, z, wq)
        ctx.cfg = (float(out_scale), float(w_scale), float(x_scale), gs)
        return out

    @staticmethod
    def backward(ctx, dy):
        x_saved, weight, bias, z, wq = ctx.saved_tensors
        out_scale, w_scale, x_scale, gs = ctx.cfg
        n = ctx.needs_input_grad
        if gs is None:
            dx, dw, db, _ = ops.linear_backward(dy, x_saved, weight, bias, z, n, out_scale)
            return dx, dw, db, None, None, None, None, None, None
        want_db = bias is not None and n[2]
        g8, db, s = ops.f8_output_grad(dy.contiguous(), z, want_db, gs)
        dx = ops.gemm_dgrad(g8, wq, alpha=s * w_scale * out_scale) if n[0] else None
        dw = _w_grad(g8, x_saved, s * x_scale * out_scale, weight) if n[1] else None
        return dx, dw, (db.to(bias.dtype) if want_db else None), None, None, None, None, None, None


class _Fp8LinearResFn(torch.autograd.Function):
    """s = a r + b (out_scale x W^T + bias) on e4m3 operands with the residual sum formed in the GEMM epilogue; optionally the
    e4m3 copy of s for the next projection (second output).  Backward as `_Fp8LinearFn`, the factor b folded into the
    products' multipliers; the residual receives a dy."""

    @staticmethod
    def forward(ctx, x2d, weight, bias, resid2d, a, b, wq, w_scale, x_scale, out_scale, gs, quant_scale, xq):
        if xq is None:
            xq = ops.quantize_e4m3(x2d, x_scale)
        out, q8 = ops.gemm_res(xq, wq, x_scale * w_scale * out_scale, bias, resid2d, a, b, quant_scale)
        ctx.save_for_backward(xq if gs is not None else x2d, weight, bias, wq)
        ctx.cfg = (float(a), float(b), float(out_scale), float(w_scale), float(x_scale), gs)
        if q8 is not None:
            ctx.mark_non_differentiable(q8)
        return out, q8

    @staticmethod
    def backward(ctx, dy, _dq8=None):
        x_saved, weight, bias, wq = ctx.saved_tensors
        a, b, out_scale, w_scale, x_scale, gs = ctx.cfg
        n = ctx.needs_input_grad
        dy = dy.contiguous()
        tail = (None,) * 9
        d_res = (dy if a == 1.0 else dy * a) if n[3] else None
        if gs is None:
            dx, dw, db, _ = ops.linear_backward(dy, x_saved, weight, bias, None, n, out_scale * b)
            if db is not None and b != 1.0:
                db = db * b
            return (dx, dw, db, d_res) + tail
        want_db = bias is not None and n[2]
        g8, db, s = ops.f8_output_grad(dy, None, want_db, gs)
        dx = ops.gemm_dgrad(g8, wq, alpha=s * w_scale * out_scale * b) if n[0] else None
        dw = _w_grad(g8, x_saved, s * x_scale * out_scale * b, weight) if n[1] else None
        return (dx, dw, (db * b).to(bias.dtype) if want_db else None, d_res) + tail


class _Fp8FfnFn(torch.autograd.Function):
    """fc2(gelu(fc1(x))) on two e4m3 products as ONE differentiable step: fc1's epilogue writes gelu(.) directly as the e4m3
    operand of fc2 (with fc2's activation scale) beside the bf16 pre-activation z, so neither a bf16 copy of the 4E-wide
    activation nor a cast pass over it exists (mu_scaling/layer.py:236-241 and modules.py:323-335 of the reference; te.Linear
    there).  Backward with GradScales: four 8-bit products (e5m2 gradients; the e4m3 operands of the forward pass are the
    other sides, fc2's being that very gelu(.) copy); the gradient casts ride on the passes that form the bias gradients and
    gelu'(z) dy.  Without: bf16 products, gelu(z) rebuilt for fc2's weight gradient."""

    @staticmethod
    def forward(ctx, x2d, w1, b1, w2, b2, wq1, ws1, xs1, os1, wq2, ws2, xs2, os2, gs1, gs2, xq):
        a8, z = ops.gemm_e4m3(xq, wq1, xs1 * ws1 * os1, b1, True, out_e4m3_scale=xs2, save_preact=True)
        y = ops.gemm_e4m3(a8, wq2, xs2 * ws2 * os2, b2, False)
        f8 = gs1 is not None and gs2 is not None
        ctx.save_for_backward(xq if f8 else x2d, w1, b1, w2, b2, z, *((a8, wq1, wq2) if f8 else ()))
        ctx.cfg = (float(os1), float(os2), float(ws1), float(xs1), float(ws2), float(xs2), gs1 if f8 else None, gs2 if f8 else None)
        return y

    @staticmethod
    def backward(ctx, dy):
        os1, os2, ws1, xs1, ws2, xs2, gs1, gs2 = ctx.cfg
        n = ctx.needs_input_grad
        dy = dy.contiguous()
        tail = (None,) * 11
        if gs1 is None:
            x2d, w1, b1, w2, b2, z = ctx.saved_tensors
            # fc2: bias gradient, then the gradient of its input; its weight gradient waits for gelu(z)
            db2 = ops.gelu_bwd_colsum(dy, None, True)[1].to(b2.dtype) if (b2 is not None and n[4]) else None
            da = ops.gemm_dgrad(dy, ops._as_bf16(w2), alpha=os2)
            dz, db1, act = ops.gelu_bwd_colsum(da, z, b1 is not None and n[2], want_act=n[3])
            dw2 = None
            if n[3]:
                dw2 = ops.gemm_wgrad(dy, act, alpha=os2, out_dtype=torch.float32 if w2.dtype == torch.float32 else torch.bfloat16)
                if dw2.dtype != w2.dtype:
                    dw2 = dw2.to(w2.dtype)
            dx, dw1, db1, _ = ops.linear_backward(dz, x2d, w1, b1, None, (n[0], n[1], n[2]), os1, db=db1 if db1 is not None else False)
            return (dx, dw1, db1, dw2, db2) + tail
        xq, w1, b1, w2, b2, z, a8, wq1, wq2 = ctx.saved_tensors
        g2, db2, s2 = ops.f8_output_grad(dy, None, b2 is not None and n[4], gs2)
        da = ops.gemm_dgrad(g2, wq2, alpha=s2 * ws2 * os2)
        dw2 = _w_grad(g2, a8, s2 * xs2 * os2, w2) if n[3] else None
        g1, db1, s1 = ops.f8_output_grad(da, z, b1 is not None and n[2], gs1)
        dx = ops.gemm_dgrad(g1, wq1, alpha=s1 * ws1 * os1) if n[0] else None
        dw1 = _w_grad(g1, xq, s1 * xs1 * os1, w1) if n[1] else None
        return (dx, dw1, db1.to(b1.dtype) if db1 is not None else None, dw2, db2.to(b2.dtype) if db2 is not None else None) + tail


class Fp8Linear(nn.Module):
    """Drop-in for nn.Linear (same `weight`, `bias`, `in_features`, `out_features`) computing in e4m3 on the GPU."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, x_scale: float = 1.0):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None
        self.x_scale = float(x_scale)
        self.out_scale = 1.0        # static multiplier of x W^T (muS: 1/sqrt(fan_in)); 1.0 = plain linear
        self.fp8_grads = True       # backward products in 8 bits (e5m2 gradient); False: bf16 on the master weight
        self.grad_scale = ops.GradScale()   # static scale of the e5m2 cast, measured on the first backward pass
        self._wq: Optional[torch.Tensor] = None
        self._wq_key = None
        self._w_scale = 1.0

    @classmethod
    def from_linear(cls, lin: nn.Linear, x_scale: float = 1.0) -> "Fp8Linear":
        new = cls(lin.in_features, lin.out_features, lin.bias is not None, x_scale)
        new.to(device=lin.weight.device, dtype=lin.weight.dtype)
        with torch.no_grad():
            new.weight.copy_(lin.weight)
            if lin.bias is not None:
                new.bias.copy_(lin.bias)
        return new

    def _quantized_weight(self):
        key = (self.weight.data_ptr(), self.weight._version, self.weight.device)
        if self._wq is None or self._wq_key != key:
            w = self.weight.detach()
            amax = float(w.abs().amax())                      # host sync, only when the weight has changed
            self._w_scale = max(amax, 1e-12) / E4M3_MAX
            self._wq = ops.quantize_e4m3(w.to(torch.bfloat16).contiguous(), self._w_scale)
            self._wq_key = key
        return self._wq, self._w_scale

    def forward(self, x: torch.Tensor, gelu: bool = False) -> torch.Tensor:
        if not x.is_cuda:
            raise RuntimeError("Fp8Linear runs on CUDA tensors only (no CPU fallback)")
        wq, w_scale = self._quantized_weight()
        x2d = x.reshape(-1, x.shape[-1]).to(torch.bfloat16).contiguous()
        y = _Fp8LinearFn.apply(x2d, self.weight, self.bias, wq, w_scale, self.x_scale, gelu, self.out_scale,
                               self.grad_scale if self.fp8_grads else None)
        return y.view(*x.shape[:-1], self.out_features)

    def forward_res(self, x: torch.Tensor, resid: torch.Tensor, a: float, b: float, quant_scale: Optional[float] = None) -> torch.Tensor:
        """a * resid + b * self(x), the residual sum formed in the GEMM epilogue; with quant_scale the e4m3 copy of the sum is
        attached to it for the e4m3 projection that reads it next."""
        wq, w_scale = self._quantized_weight()
        x2d = x.reshape(-1, x.shape[-1]).to(torch.bfloat16).contiguous()
        xq = ops.e4m3_of(x, self.x_scale) if x.dtype == torch.bfloat16 else None
        out, q8 = _Fp8LinearResFn.apply(x2d, self.weight, self.bias, resid.reshape(-1, self.out_features), float(a), float(b), wq, w_scale,
                                        self.x_scale, self.out_scale, self.grad_scale if self.fp8_grads else None, quant_scale, xq)
        out = out.view(*x.shape[:-1], self.out_features)
        if q8 is not None:
            ops.attach_e4m3(out, q8, quant_scale)
        return out

    def extra_repr(self):
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, x_scale={self.x_scale}"


def fp8_ffn(fc1: "Fp8Linear", fc2: "Fp8Linear", x: torch.Tensor) -> torch.Tensor:
    """fc2(gelu_erf(fc1(x))) for two Fp8Linear modules on bf16 CUDA activations, as one differentiable step (`_Fp8FfnFn`)."""
    wq1, ws1 = fc1._quantized_weight()
    wq2, ws2 = fc2._quantized_weight()
    x2d = x.reshape(-1, x.shape[-1]).to(torch.bfloat16).contiguous()
    xq = ops.e4m3_of(x, fc1.x_scale) if x.dtype == torch.bfloat16 else ops.quantize_e4m3(x2d, fc1.x_scale)   # the pass that produced x may have left the copy
    f8 = fc1.fp8_grads and fc2.fp8_grads
    y = _Fp8FfnFn.apply(x2d, fc1.weight, fc1.bias, fc2.weight, fc2.bias, wq1, ws1, fc1.x_scale, fc1.out_scale,
                        wq2, ws2, fc2.x_scale, fc2.out_scale, fc1.grad_scale if f8 else None, fc2.grad_scale if f8 else None, xq)
    return y.view(*x.shape[:-1], fc2.out_features)


def fused_fp8_weight(owner: nn.Module, mods):
    """(e4m3 [3E][E] weight, its scale, activation scale, output multiplier, GradScale or None) of the Q/K/V projections `mods` (one fused Fp8Linear or three
    separate ones) for the head-major QKV GEMM.  Three separate weights share one scale (the largest amax of the three);
    the quantised concatenation is cached on `owner` until one of the weights changes."""
    f8_grads = all(m.fp8_grads for m in mods)
    if len(mods) == 1:
        wq, w_scale = mods[0]._quantized_weight()
        return wq, w_scale, mods[0].x_scale, mods[0].out_scale, (mods[0].grad_scale if f8_grads else None)
    if getattr(owner, "_fp8_qkv_grad_scale", None) is None:
        owner._fp8_qkv_grad_scale = ops.GradScale()       # the three projections share one gradient matrix, hence one scale
    key = tuple((m.weight.data_ptr(), m.weight._version) for m in mods)
    cached = getattr(owner, "_fp8_qkv_cache", None)
    if cached is None or cached[0] != key:
        w = torch.cat([m.weight.detach() for m in mods], dim=0)
        w_scale = max(m._quantized_weight()[1] for m in mods)   # amax of the concatenation / 448; a host read only where a copy is stale
        cached = (key, ops.quantize_e4m3(w.to(torch.bfloat16).contiguous(), w_scale), w_scale)
        owner._fp8_qkv_cache = cached
    return cached[1], cached[2], max(m.x_scale for m in mods), mods[0].out_scale, (owner._fp8_qkv_grad_scale if f8_grads else None)


def refresh_fp8_weights(model: nn.Module) -> nn.Module:
    """Drop every cached e4m3 weight copy of `model`, so that the next forward pass casts the master weights again.
    The caches notice in-place updates of a Parameter (optimizer steps, `weight.copy_`), which bump its version counter;
    writes through `weight.data` (sharded or apex-style optimizers, broadcasts into `.data`) do not - call this after such
    a write, or the forward pass keeps multiplying by the old e4m3 weights."""
    for m in model.modules():
        if isinstance(m, Fp8Linear):
            m._wq, m._wq_key = None, None
        if getattr(m, "_fp8_qkv_cache", None) is not None:
            m._fp8_qkv_cache = None
    return model


class Fp8WeightScaler:
    """Re-casts the e4m3 weight copies of every Fp8Linear of `model` after an optimizer step WITHOUT a host
    synchronisation in the step: `refresh()` measures all weight maxima with one multi-tensor pass on the device, starts
    their copy to pinned host memory, and casts each weight with the scale of the maxima measured by the refresh BEFORE
    (those arrived a whole step ago).  A weight that outgrew last step's maximum saturates at +-448 for one step, which an
    optimizer step's relative change keeps to the last e4m3 step of the very largest entries.  This is the delayed-scaling
    idea of the production FP8 recipe (transformer_engine's DelayedScaling keeps an amax history per tensor and derives the
    scale of a step from earlier steps), restated for the per-tensor weight scale amax / 448 of
    mint_plus/models/alt/munit_scaling.py:22-34.  The first refresh has no history and reads its maxima back at once.
    Without a scaler the copies refresh lazily in the forward pass, with one host read per changed weight."""

    def __init__(self, model: nn.Module):
        self.mods = [m for m in model.modules() if isinstance(m, Fp8Linear)]
        self.model = model
        self._host = None
        self._event = None

    @torch.no_grad()
    def refresh(self) -> None:
        if not self.mods:
            return
        ws = [m.weight.detach() for m in self.mods]
        amax = torch.stack([a.float() for a in torch._foreach_norm(ws, float("inf"))])
        if self._host is None:
            self._host = torch.empty(len(ws), dtype=torch.float32).pin_memory()
            prev = amax.cpu().tolist()                   # first use: no history yet
        else:
            self._event.synchronize()                    # recorded a step ago
            prev = self._host.tolist()
        self._host.copy_(amax, non_blocking=True)
        self._event = torch.cuda.Event()
        self._event.record()
        for m, w, a in zip(self.mods, ws, prev):
            m._w_scale = max(a, 1e-12) / E4M3_MAX
            m._wq = ops.quantize_e4m3(w.to(torch.bfloat16).contiguous(), m._w_scale)
            m._wq_key = (m.weight.data_ptr(), m.weight._version, m.weight.device)
        for m in self.model.modules():                   # concatenated copies are rebuilt from the new casts (no host read)
            if getattr(m, "_fp8_qkv_cache", None) is not None:
                m._fp8_qkv_cache = None
            if getattr(m, "_qkv6_cache", None) is not None:
                m._qkv6_cache = None


def _sublayers(model):
    for layer in model.layers:
        yield from (layer.layers if hasattr(layer, "layers") else [layer])


def apply_fp8_to_model(model: nn.Module, static_scale: bool = True, keep_embed_in_bf16: bool = True,
                       keep_lm_head_in_bf16: bool = True, fp8_grads: bool = True) -> nn.Module:
    """Swap the hidden projections of every layer for Fp8Linear, in place: self_attn q/k/v/out_proj (or its fused_qkv),
    multimer_attn.fused_qkv (or q/k/v), feed_forward fc1/fc2.  Embedding and LM head are left alone, as in the reference.
    `static_scale` is recorded (activation scales here are always static).  `fp8_grads`: the backward products run in 8 bits
    too, the gradient cast to e5m2 with a static scale that each projection measures on its first backward pass (the
    reference's te.Linear does the same under its HYBRID recipe); False keeps them in bf16 on the master weights."""
    def swap(mod, name):
        lin = getattr(mod, name, None)
        if isinstance(lin, nn.Linear):
            new = Fp8Linear.from_linear(lin)
            new.fp8_grads = fp8_grads
            setattr(mod, name, new)

    for sub in _sublayers(model):
        for attn_name in ("self_attn", "multimer_attn"):
            attn = getattr(sub, attn_name, None)
            if attn is None:
                continue
            for name in ("q_proj", "k_proj", "v_proj", "out_proj", "fused_qkv"):
                swap(attn, name)
        swap(sub.feed_forward, "fc1")
        swap(sub.feed_forward, "fc2")
    model._fp8_config = {"enabled": True, "static_scale": static_scale}
    return model


@torch.no_grad()
def calibrate_fp8(model: nn.Module, *forward_args, margin: float = 1.0, **forward_kwargs) -> nn.Module:
    """Run one forward pass and set every Fp8Linear's activation scale to amax(input) * margin / 448."""
    hooks, seen = [], {}

    def pre_hook(mod, args):
        seen[mod] = max(seen.get(mod, 0.0), float(args[0].detach().abs().amax()))

    for m in model.modules():
        if isinstance(m, Fp8Linear):
            hooks.append(m.register_forward_pre_hook(pre_hook))
    try:
        model(*forward_args, **forward_kwargs)
    finally:
        for h in hooks:
            h.remove()
    for m, amax in seen.items():
        m.x_scale = max(amax * margin, 1e-12) / E4M3_MAX
    return model


def qkv_activation_scale(layer) -> Optional[float]:
    """The activation scale with which the layer's fused QKV products cast their input to e4m3, or None when they are
    not FP8 projections (the scale `fused_fp8_weight` hands to the GEMM)."""
    sa = getattr(layer, "self_attn", None)
    if sa is None:
        return None
    fused = getattr(sa, "fused_qkv", None)
    mods = [fused] if fused is not None else [getattr(sa, n, None) for n in ("q_proj", "k_proj", "v_proj")]
    if all(isinstance(m, Fp8Linear) for m in mods):
        return max(m.x_scale for m in mods)
    return None


def compute_tau(num_layers: int) -> float:
    """Residual coefficient for a depth: 0.5 / sqrt(L) (mu_scaling/optim.py:20-41)."""
    return 0.5 / math.sqrt(max(1, num_layers))


class TransformerLayer_MINT_mu(_TwoPathwayLayer):
    """muS Res-Post-LN layer: x = sqrt(1-tau) x + sqrt(tau) attn(x); x = sqrt(1-tau) x + sqrt(tau) ffn(x); x = LN(x)
    (mu_scaling/layer.py:50-123, 240-280).  Same constructor and sub-module names as the reference, no
    `self_attn_layer_norm`; `tau` is a buffer so that it travels with the state dict."""

    def __init__(self, embed_dim: int, ffn_embed_dim: int, attention_heads: int, use_rotary_embeddings: bool = True,
                 use_multimer: bool = False, use_rmsnorm: bool = False, use_erf_gelu: bool = False,
                 tau: Optional[float] = None, num_layers: Optional[int] = None, use_sqrt_softmax: bool = True):
        super().__init__()
        self.embed_dim = embed_dim
        self.ffn_embed_dim = ffn_embed_dim
        self.attention_heads = attention_heads
        self.use_rotary_embeddings = use_rotary_embeddings
        self.use_multimer = use_multimer
        self.use_erf_gelu = use_erf_gelu
        self._use_fused_multi_pathway = True
        self._use_sqrt_softmax = use_sqrt_softmax
        if tau is None:
            tau = compute_tau(num_layers or 30)
        self.self_attn = MultiHeadAttention(embed_dim, attention_heads, use_rotary_embeddings=use_rotary_embeddings)
        self.multimer_attn = None
        if use_multimer:
            self.multimer_attn = MultiHeadAttention(embed_dim, attention_heads, use_rotary_embeddings=False, no_proj=True)
        self.feed_forward = VanillaFeedForward(embed_dim, ffn_embed_dim, use_erf_gelu=use_erf_gelu)
        self.final_layer_norm = nn.LayerNorm(embed_dim)
        self.register_buffer("_tau", torch.tensor(tau, dtype=torch.float32))
        self._tau_f = float(tau)

    _next_x_scale = None   # set by MINT.forward: the activation scale of the NEXT layer's FP8 QKV products, if any

    def forward(self, x, self_attn_mask=None, self_attn_padding_mask=None, chain_ids=None, pack=None):
        tau = self._tau_f                       # host copy of the buffer: no device read-back per call
        keep, add = math.sqrt(1.0 - tau), math.sqrt(tau)
        gpu_bf16 = x.is_cuda and x.dtype == torch.bfloat16
        fc1 = self.feed_forward.fc1
        fc1_scale = fc1.x_scale if isinstance(fc1, Fp8Linear) else None
        from . import modules_plus as _mp
        if self.use_multimer and gpu_bf16 and self._use_fused_multi_pathway and _mp.FUSE_OUT_RESIDUAL:
            # the first weighted residual sum is formed in the epilogue of the output projection (which also writes the e4m3
            # operand of fc1), the second one together with the closing LayerNorm in one fused pass (which writes the e4m3
            # operand of the next layer's QKV products)
            x, _ = self._multimer_attention_superfused(x, self_attn_mask, self_attn_padding_mask, chain_ids, pack,
                                                       residual=(x, keep, add), quant_scale=fc1_scale)
            _, y = ops.add_layernorm(x, self.feed_forward(x), keep, add, self.final_layer_norm, need_s=False,
                                     quant_scale=self._next_x_scale)
            return y, None
        if self.use_multimer:
            attn_out, _ = self._multimer_attention_plus(x, self_attn_mask, self_attn_padding_mask, chain_ids, pack)
        elif pack is not None:
            raise NotImplementedError("packed tokens need the two-pathway attention")
        else:
            attn_out, _ = self._standard_attention(x, self_attn_mask, self_attn_padding_mask)
        if gpu_bf16:
            # bf16 on the GPU: weighted residuals and the closing LayerNorm in two fused passes
            # (each pass also writes the e4m3 operand of the FP8 projection that reads its result next)
            x, _ = ops.add_layernorm(x, attn_out, keep, add, None, quant_scale=fc1_scale)
            _, y = ops.add_layernorm(x, self.feed_forward(x), keep, add, self.final_layer_norm, need_s=False,
                                     quant_scale=self._next_x_scale)
            return y, None
        x = keep * x + add * attn_out
        x = keep * x + add * self.feed_forward(x)
        return self.final_layer_norm(x), None

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)
        self._tau_f = float(self._tau)


def build_mint_mu(model_size: str = "150M", use_multimer: bool = True, tau: Optional[float] = None,
                  use_sqrt_softmax: bool = True, use_fp8: bool = False, fp8_static_scale: bool = True,
                  warm_start_esm2: bool = False, checkpoint_block_size: int = 0, use_fused_multi_pathway: bool = True,
                  num_layers: Optional[int] = None, embed_dim: Optional[int] = None,
                  attention_heads: Optional[int] = None, unit_scaled: bool = False):
    """MINT with muS layers (mu_scaling/__init__.py:142-250): Res-Post-LN, tau-weighted residuals, optional square-root
    softmax, optional FP8 projections.  The model is returned on the CPU with default initialisation.

    `num_layers`/`embed_dim`/`attention_heads` override the registry entry (for shapes the registry does not hold).
    `unit_scaled=True` applies `unit_variance_init_` and gives every projection the static 1/sqrt(fan_in) output
    multiplier that keeps unit-variance activations (mu_scaling/init.py:59-72 describes it; the reference builder leaves
    it switched off).  `checkpoint_block_size` > 0 groups the layers into CheckpointedBlocks.  Warm start from ESM-2
    files is outside this package."""
    from .esm2 import MINT, MODEL_REGISTRY
    from .modules import build_checkpointed_model
    if warm_start_esm2:
        raise NotImplementedError("warm_start_esm2 is not part of this package (load a state dict instead)")
    cfg = MODEL_REGISTRY[model_size]
    L_ = num_layers or cfg["num_layers"]
    E_ = embed_dim or cfg["embed_dim"]
    H_ = attention_heads or cfg["attention_heads"]
    if tau is None:
        tau = compute_tau(L_)
    model = MINT(num_layers=L_, embed_dim=E_, attention_heads=H_, use_multimer=use_multimer,
                 layer_factory=lambda: TransformerLayer_MINT_mu(E_, 4 * E_, H_, use_rotary_embeddings=True,
                                                                use_multimer=use_multimer, tau=tau, num_layers=L_,
                                                                use_sqrt_softmax=use_sqrt_softmax))
    for layer in model.layers:
        layer._use_fused_multi_pathway = use_fused_multi_pathway
    if unit_scaled:
        unit_variance_init_(model)
    if checkpoint_block_size > 0:
        build_checkpointed_model(model, block_size=checkpoint_block_size)
    if use_fp8:
        apply_fp8_to_model(model, static_scale=fp8_static_scale)
    if unit_scaled:
        set_unit_output_scales(model)
    model._mu_config = {"tau": tau, "use_sqrt_softmax": use_sqrt_softmax, "use_fp8": use_fp8, "unit_scaled": unit_scaled}
    return model


def build_mint_fp8(model_size: str = "150M", use_multimer: bool = True, static_scale: bool = True,
                   checkpoint_block_size: int = 3, use_fused_multi_pathway: bool = True):
    """The Pre-LN MINT of a registry size with every hidden projection swapped for Fp8Linear
    (mu_scaling/__init__.py:269-312): standard architecture and state-dict names, so pre-trained weights load unchanged;
    layers grouped into CheckpointedBlocks of `checkpoint_block_size` (0: none).  Returned on the CPU."""
    from .esm2 import MINT, MODEL_REGISTRY
    from .modules import build_checkpointed_model
    from .modules_plus import enable_fused_multi_pathway
    cfg = MODEL_REGISTRY[model_size]
    model = MINT(num_layers=cfg["num_layers"], embed_dim=cfg["embed_dim"], attention_heads=cfg["attention_heads"],
                 use_multimer=use_multimer)
    enable_fused_multi_pathway(model, enabled=use_fused_multi_pathway)
    if checkpoint_block_size > 0:
        build_checkpointed_model(model, block_size=checkpoint_block_size)
    return apply_fp8_to_model(model, static_scale=static_scale)


def set_unit_output_scales(model: nn.Module) -> nn.Module:
    """Give every Fp8Linear of the layers the static output multiplier 1/sqrt(fan_in) (alt/munit_scaling.py:22-34)."""
    for sub in _sublayers(model):
        for m in sub.modules():
            if isinstance(m, Fp8Linear):
                m.out_scale = 1.0 / math.sqrt(m.in_features)
    return model


def unit_variance_init_(module: nn.Module) -> nn.Module:
    """N(0,1) Linear / Embedding weights (padding row zero), zero biases, norm gains 1 (mu_scaling/init.py:23-56)."""
    for m in module.modules():
        if isinstance(m, (nn.Linear, Fp8Linear)):
            nn.init.normal_(m.weight, mean=0.0, std=1.0)
            if m.bias is not None:
                nn.init.zeros_(m.bias)
        elif isinstance(m, nn.Embedding):
            nn.init.normal_(m.weight, mean=0.0, std=1.0)
            if m.padding_idx is not None:
                with torch.no_grad():
                    m.weight[m.padding_idx].zero_()
        elif isinstance(m, nn.LayerNorm):
            nn.init.ones_(m.weight)
            nn.init.zeros_(m.bias)
        elif isinstance(m, nn.RMSNorm):
            nn.init.ones_(m.weight)
    return module
