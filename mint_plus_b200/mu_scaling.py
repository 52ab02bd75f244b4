"""FP8 (e4m3, per-tensor scaled) projections and the helpers around them, with the reference's entry points
(mint_plus/models/mu_scaling/__init__.py:42-135 `apply_fp8_to_model`, mu_scaling/init.py:23-56 `unit_variance_init_`).

The reference swaps nn.Linear for transformer_engine's te.Linear; here the swap is to `Fp8Linear`, whose forward is the
tcgen05 e4m3 GEMM of libmintb: x and W are cast to e4m3 with one scale per tensor (saturating at +-448, as
mint_plus/models/alt/munit_scaling.py:22-34 states the arithmetic), accumulated in fp32, multiplied by the product of the
two scales, and bias / erf-GELU are applied in the GEMM epilogue.  The weight scale is amax(W)/448, refreshed when the weight
changes; the activation scale is static (1.0 by default, which suits unit-variance muS activations; `calibrate_fp8`
measures it on a sample batch otherwise).  Gradients are computed in bf16 from the master weights (straight-through for
the casts).
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from . import ops

E4M3_MAX = 448.0


class _Fp8LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2d, weight, bias, wq, w_scale, x_scale, gelu):
        xq = ops.quantize_e4m3(x2d, x_scale)
        ctx.save_for_backward(x2d, weight, bias)
        ctx.gelu = gelu
        ctx.scales = (wq, w_scale, x_scale)
        return ops.gemm_e4m3(xq, wq, x_scale * w_scale, bias, gelu)

    @staticmethod
    def backward(ctx, dy):
        x2d, weight, bias = ctx.saved_tensors
        wb = weight if weight.dtype == torch.bfloat16 else weight.to(torch.bfloat16)
        dz = dy
        if ctx.gelu:
            wq, w_scale, x_scale = ctx.scales
            z = ops.gemm_e4m3(ops.quantize_e4m3(x2d, x_scale), wq, x_scale * w_scale, bias, False)
            dz = (dy.float() * ops._gelu_erf_grad(z)).to(torch.bfloat16)
        dx = dz @ wb if ctx.needs_input_grad[0] else None
        dw = (dz.t() @ x2d).to(weight.dtype) if ctx.needs_input_grad[1] else None
        db = dz.float().sum(0).to(bias.dtype) if (bias is not None and ctx.needs_input_grad[2]) else None
        return dx, dw, db, None, None, None, None


class Fp8Linear(nn.Module):
    """Drop-in for nn.Linear (same `weight`, `bias`, `in_features`, `out_features`) computing in e4m3 on the GPU."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, x_scale: float = 1.0):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None
        self.x_scale = float(x_scale)
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
        y = _Fp8LinearFn.apply(x2d, self.weight, self.bias, wq, w_scale, self.x_scale, gelu)
        return y.view(*x.shape[:-1], self.out_features)

    def extra_repr(self):
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, x_scale={self.x_scale}"


def _sublayers(model):
    for layer in model.layers:
        yield from (layer.layers if hasattr(layer, "layers") else [layer])


def apply_fp8_to_model(model: nn.Module, static_scale: bool = True, keep_embed_in_bf16: bool = True,
                       keep_lm_head_in_bf16: bool = True) -> nn.Module:
    """Swap the hidden projections of every layer for Fp8Linear, in place: self_attn q/k/v/out_proj (or its fused_qkv),
    multimer_attn.fused_qkv (or q/k/v), feed_forward fc1/fc2.  Embedding and LM head are left alone, as in the reference.
    `static_scale` is recorded (activation scales here are always static)."""
    def swap(mod, name):
        lin = getattr(mod, name, None)
        if isinstance(lin, nn.Linear):
            setattr(mod, name, Fp8Linear.from_linear(lin))

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
