"""MultiHeadAttention and MultimerAttention with the reference's constructor arguments, attribute names,
state-dict keys and method signatures (mint_plus/models/attention.py:32-371).

`project_qkv_4d` feeds the fused kernels; `forward(..., before_softmax=True)` keeps the reference's
materialising contract (returns (B,H,T,T) logits and (B,H,T,D) values) for callers that still want it.
The incremental-state cache of the reference's MultiHeadAttention is decoder plumbing that MINT never
uses (esm2.py:124-132 passes none) and is not provided.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F
from torch import Tensor, nn

from .rotary_embedding import RotaryEmbedding


def _heads_4d(t: Tensor, T: int, B: int, H: int, D: int) -> Tensor:
    return t.reshape(T, B, H, D).permute(1, 2, 0, 3).contiguous()


class MultiHeadAttention(nn.Module):
    def __init__(self, embed_dim: int, num_heads: int, dropout: float = 0.0, bias: bool = True,
                 use_rotary_embeddings: bool = False, no_proj: bool = False, use_fused_qkv: bool = False):
        super().__init__()
        self.embed_dim = embed_dim
        self.num_heads = num_heads
        self.head_dim = embed_dim // num_heads
        assert self.head_dim * num_heads == embed_dim, "embed_dim must be divisible by num_heads"
        self.scaling = self.head_dim ** -0.5
        self.dropout = dropout
        self.use_fused_qkv = use_fused_qkv
        if use_fused_qkv:
            self.fused_qkv = nn.Linear(embed_dim, 3 * embed_dim, bias=bias)
            self.q_proj = self.k_proj = self.v_proj = None
        else:
            self.q_proj = nn.Linear(embed_dim, embed_dim, bias=bias)
            self.k_proj = nn.Linear(embed_dim, embed_dim, bias=bias)
            self.v_proj = nn.Linear(embed_dim, embed_dim, bias=bias)
        self.out_proj = None if no_proj else nn.Linear(embed_dim, embed_dim, bias=bias)
        self.rot_emb = RotaryEmbedding(dim=self.head_dim) if use_rotary_embeddings else None
        self._init_parameters()

    def _init_parameters(self):
        gain = 2 ** -0.5
        if self.use_fused_qkv:
            nn.init.xavier_uniform_(self.fused_qkv.weight, gain=gain)
            if self.fused_qkv.bias is not None:
                nn.init.zeros_(self.fused_qkv.bias)
        else:
            for proj in (self.q_proj, self.k_proj, self.v_proj):
                nn.init.xavier_uniform_(proj.weight, gain=gain)
        if self.out_proj is not None:
            nn.init.xavier_uniform_(self.out_proj.weight)
            if self.out_proj.bias is not None:
                nn.init.constant_(self.out_proj.bias, 0.0)

    def _project_qkv(self, x: Tensor) -> Tuple[Tensor, Tensor, Tensor]:
        if self.use_fused_qkv:
            q, k, v = self.fused_qkv(x).chunk(3, dim=-1)
            return q, k, v
        return self.q_proj(x), self.k_proj(x), self.v_proj(x)

    def project_qkv_4d(self, x: Tensor) -> Tuple[Tensor, Tensor, Tensor]:
        """x (T,B,E) -> q, k, v (B,H,T,D) contiguous; no scaling, no RoPE."""
        T, B, _ = x.shape
        H, D = self.num_heads, self.head_dim
        q, k, v = self._project_qkv(x)
        return _heads_4d(q, T, B, H, D), _heads_4d(k, T, B, H, D), _heads_4d(v, T, B, H, D)

    def forward_before_softmax(self, x: Tensor, key_padding_mask: Optional[Tensor] = None) -> Tuple[Tensor, Tensor]:
        T, B, _ = x.shape
        H, D = self.num_heads, self.head_dim
        q, k, v = self._project_qkv(x)
        q = q * self.scaling
        q = q.reshape(T, B * H, D).transpose(0, 1).contiguous()
        k = k.reshape(T, B * H, D).transpose(0, 1).contiguous()
        v = v.reshape(T, B * H, D).transpose(0, 1).contiguous()
        if self.rot_emb is not None:
            q, k = self.rot_emb(q), self.rot_emb(k)
        logits = torch.bmm(q, k.transpose(1, 2)).view(B, H, T, T)
        if key_padding_mask is not None:
            logits = logits.masked_fill(key_padding_mask[:, None, None, :], float("-inf"))
        return logits, v.view(B, H, T, D)

    def forward(self, x: Tensor, key_padding_mask: Optional[Tensor] = None, attn_mask: Optional[Tensor] = None,
                incremental_state=None, need_weights: bool = False, need_head_weights: bool = False,
                before_softmax: bool = False):
        if incremental_state is not None:
            raise NotImplementedError("incremental decoding state is not part of this implementation")
        T, B, E = x.shape
        H = self.num_heads
        logits, v = self.forward_before_softmax(x, None)
        if attn_mask is not None:
            logits = logits + attn_mask
        if key_padding_mask is not None:
            logits = logits.masked_fill(key_padding_mask[:, None, None, :], float("-inf"))
        if before_softmax:
            return logits, v
        probs = F.softmax(logits, dim=-1, dtype=torch.float32).type_as(logits)
        probs = F.dropout(probs, p=self.dropout, training=self.training)
        out = torch.matmul(probs, v)                                  # (B,H,T,D)
        out = out.permute(2, 0, 1, 3).reshape(T, B, E)
        if self.out_proj is not None:
            out = self.out_proj(out)
        weights = None
        if need_weights:
            weights = probs if need_head_weights else probs.mean(dim=1)
        return out, weights


class MultimerAttention(nn.Module):
    """Cross-chain pathway: fused QKV projection, no rotary embedding, no output projection."""

    def __init__(self, embed_dim: int, num_heads: int, dropout: float = 0.0, bias: bool = True):
        super().__init__()
        self.embed_dim = embed_dim
        self.num_heads = num_heads
        self.head_dim = embed_dim // num_heads
        assert self.head_dim * num_heads == embed_dim
        self.scaling = self.head_dim ** -0.5
        self.dropout = dropout
        self.fused_qkv = nn.Linear(embed_dim, 3 * embed_dim, bias=bias)
        self._init_parameters()

    def _init_parameters(self):
        nn.init.xavier_uniform_(self.fused_qkv.weight, gain=2 ** -0.5)
        if self.fused_qkv.bias is not None:
            nn.init.zeros_(self.fused_qkv.bias)

    def project_qkv_4d(self, x: Tensor) -> Tuple[Tensor, Tensor, Tensor]:
        T, B, _ = x.shape
        H, D = self.num_heads, self.head_dim
        q, k, v = self.fused_qkv(x).chunk(3, dim=-1)
        return _heads_4d(q, T, B, H, D), _heads_4d(k, T, B, H, D), _heads_4d(v, T, B, H, D)

    def forward(self, x: Tensor, key_padding_mask: Optional[Tensor] = None, before_softmax: Optional[bool] = None,
                **kwargs) -> Tuple[Tensor, Tensor]:
        q, k, v = self.project_qkv_4d(x)
        logits = torch.matmul(q * self.scaling, k.transpose(-1, -2))
        if key_padding_mask is not None:
            logits = logits.masked_fill(key_padding_mask[:, None, None, :], float("-inf"))
        return logits, v
