"""TransformerLayer_MINT and RobertaLMHead with the reference's interface and state-dict keys
(mint_plus/models/modules.py:25-195, 338-369).

The base layer keeps three separate q/k/v projections per pathway (`self_attn.q_proj` ..., `multimer_attn.q_proj` ...,
the cross pathway without an output projection) so that reference checkpoints load by name.  Its attention runs on the
same fused CUDA operator as the `_plus` layer; the three weights of a pathway are concatenated to [Q;K;V] on the fly.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F
from torch import nn
from torch.nn import LayerNorm as ESM1bLayerNorm  # noqa: F401  (name kept for importers)

from .attention import MultiHeadAttention
from .modules_plus import VanillaFeedForward, _PreLnLayer, gelu_erf  # noqa: F401


class TransformerLayer_MINT(_PreLnLayer):
    def __init__(self, embed_dim, ffn_embed_dim, attention_heads, use_rotary_embeddings: bool = True,
                 use_multimer: bool = False, use_rmsnorm: bool = False, use_erf_gelu: bool = False):
        super().__init__()
        self.self_attn = MultiHeadAttention(embed_dim, attention_heads, use_rotary_embeddings=use_rotary_embeddings)
        if use_multimer:
            self.multimer_attn = MultiHeadAttention(embed_dim, attention_heads, use_rotary_embeddings=False, no_proj=True)
        self._init_common(embed_dim, ffn_embed_dim, attention_heads, use_rotary_embeddings, use_multimer, use_rmsnorm,
                          use_erf_gelu)


class RobertaLMHead(nn.Module):
    """dense -> GELU -> LayerNorm -> tied output projection + bias (modules.py:338-369)."""

    def __init__(self, embed_dim: int, output_dim: int, weight: torch.Tensor):
        super().__init__()
        self.dense = nn.Linear(embed_dim, embed_dim)
        self.layer_norm = nn.LayerNorm(embed_dim)
        self.weight = weight
        self.bias = nn.Parameter(torch.zeros(output_dim))

    def forward(self, features):
        if features.is_cuda and features.dtype == torch.bfloat16 and type(self.dense) is nn.Linear and self.weight.dtype == torch.bfloat16:
            # bf16 on the GPU: dense + erf-GELU in one tcgen05 GEMM, the LayerNorm kernel, and the tied projection as a GEMM on
            # the vocabulary padded to a multiple of 8 rows (the extra logits are sliced off again)
            from . import ops
            h = ops.linear(features, self.dense.weight, self.dense.bias, gelu=True)
            _, h = ops.add_layernorm(h, None, 1.0, 0.0, self.layer_norm, need_s=False)
            V = self.weight.shape[0]
            extra = (-V) % 8
            w = F.pad(self.weight, (0, 0, 0, extra)) if extra else self.weight
            b = F.pad(self.bias, (0, extra)) if extra else self.bias
            return ops.linear(h, w, b)[..., :V]
        x = self.layer_norm(F.gelu(self.dense(features)))
        return F.linear(x, self.weight) + self.bias


class CheckpointedBlock(nn.Module):
    """A run of consecutive layers that `MINT.forward` treats (and checkpoints) as one layer: same call signature and
    `(x, None)` result as a single layer (modules.py:420-457 of the reference)."""

    def __init__(self, layers: nn.ModuleList):
        super().__init__()
        self.layers = layers

    def forward(self, x, self_attn_padding_mask: Optional[torch.Tensor] = None, self_attn_mask: Optional[torch.Tensor] = None,
                chain_ids: Optional[torch.Tensor] = None, pack=None):
        kw = dict(self_attn_padding_mask=self_attn_padding_mask, self_attn_mask=self_attn_mask, chain_ids=chain_ids)
        if pack is not None:
            kw["pack"] = pack
        for layer in self.layers:
            x, _ = layer(x, **kw)
        return x, None

    def __len__(self):
        return len(self.layers)

    def __getitem__(self, idx):
        return self.layers[idx]


def build_checkpointed_model(model: nn.Module, block_size: int = 3) -> nn.Module:
    """Group `model.layers` into CheckpointedBlocks of `block_size` layers, in place; `block_size` must divide the number
    of layers (modules.py:460-510 of the reference)."""
    layers = list(model.layers)
    if block_size <= 0 or len(layers) % block_size != 0:
        raise ValueError(f"block_size={block_size} does not evenly divide {len(layers)} layers. Try a different block_size.")
    model.layers = nn.ModuleList(CheckpointedBlock(nn.ModuleList(layers[i:i + block_size]))
                                 for i in range(0, len(layers), block_size))
    model._checkpoint_block_size = block_size
    return model
