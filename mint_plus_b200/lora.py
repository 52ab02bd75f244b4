"""LoRA adapters for the attention projections: y = W x + b + (alpha / r) B (A x), W and b frozen.

The reference takes these from the `peft` package (training/alt/trainer-Copy1.py:132-142: r=8, alpha=16, dropout 0.05,
targets the q/k/v projections); this is the same arithmetic restated on plain modules so that the LoRA training
configuration can run without that dependency.  A ~ Kaiming-uniform, B = 0 at initialisation, as usual for LoRA.
"""
from __future__ import annotations

import math

import torch
from torch import nn


class LoRALinear(nn.Module):
    def __init__(self, base: nn.Linear, r: int = 8, alpha: float = 16.0, dropout: float = 0.0):
        super().__init__()
        self.base = base
        for p in self.base.parameters():
            p.requires_grad_(False)
        self.in_features, self.out_features = base.in_features, base.out_features
        self.r, self.scaling = r, alpha / r
        self.lora_A = nn.Parameter(torch.empty(r, base.in_features, device=base.weight.device, dtype=base.weight.dtype))
        self.lora_B = nn.Parameter(torch.zeros(base.out_features, r, device=base.weight.device, dtype=base.weight.dtype))
        nn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))
        self.dropout = nn.Dropout(dropout) if dropout > 0 else nn.Identity()

    @property
    def weight(self):
        return self.base.weight

    @property
    def bias(self):
        return self.base.bias

    def forward(self, x):
        from . import ops
        if x.is_cuda and x.dtype == torch.bfloat16 and type(self.base) is nn.Linear:
            if isinstance(self.dropout, nn.Identity) or not self.training:
                # one product on the merged weight (tcgen05 GEMM); the adapters' gradients come from thin products
                return ops.lora_linear(x, self.base.weight, self.base.bias, self.lora_A, self.lora_B, self.scaling)
            y = ops.linear(x, self.base.weight, self.base.bias)       # frozen product on the tcgen05 GEMM
        else:
            y = self.base(x)
        return y + (self.dropout(x) @ self.lora_A.t()) @ self.lora_B.t() * self.scaling


def apply_lora(model: nn.Module, r: int = 8, alpha: float = 16.0, dropout: float = 0.0,
               targets=("q_proj", "k_proj", "v_proj", "out_proj")) -> nn.Module:
    """Freeze every parameter of `model` and wrap the named projections of both attention pathways of every layer."""
    for p in model.parameters():
        p.requires_grad_(False)
    for layer in model.layers:
        for sub in (layer.layers if hasattr(layer, "layers") else [layer]):
            for attn_name in ("self_attn", "multimer_attn"):
                attn = getattr(sub, attn_name, None)
                if attn is None:
                    continue
                for name in targets:
                    lin = getattr(attn, name, None)
                    if isinstance(lin, nn.Linear):
                        setattr(attn, name, LoRALinear(lin, r, alpha, dropout))
    return model
