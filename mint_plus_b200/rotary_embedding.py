"""RotaryEmbedding with the reference's module interface (mint_plus/models/rotary_embedding.py:27-55).

The module keeps the `inv_freq` buffer (same state-dict key).  Inside the fused attention the rotation is
done by the CUDA kernels from this buffer; calling the module directly rotates a (..., T, D) tensor with
plain tensor arithmetic, as the reference does, for callers outside the fused path.
"""
from __future__ import annotations

import torch


def rotate_half(x):
    x1, x2 = x.chunk(2, dim=-1)
    return torch.cat((-x2, x1), dim=-1)


def apply_rotary_pos_emb(x, cos, sin):
    cos = cos[:, : x.shape[-2], :]
    sin = sin[:, : x.shape[-2], :]
    return (x * cos) + (rotate_half(x) * sin)


class RotaryEmbedding(torch.nn.Module):
    def __init__(self, dim: int, *_, **__):
        super().__init__()
        self.dim = dim
        self.register_buffer("inv_freq", self._frequencies(dim))

    @staticmethod
    def _frequencies(dim: int, device=None) -> torch.Tensor:
        return 1.0 / (10000 ** (torch.arange(0, dim, 2, device=device).float() / dim))

    def _apply(self, fn, *args, **kwargs):
        # A cast of the whole model (model.to(torch.bfloat16)) would round the frequencies to 8 bits, and a later .float()
        # does not bring them back: at position 2000 the angles are then off by radians.  The buffer therefore stays fp32:
        # after a cast it is rebuilt from `dim` on the device it has moved to.
        super()._apply(fn, *args, **kwargs)
        if self.inv_freq.dtype != torch.float32:
            self.inv_freq = self._frequencies(self.dim, self.inv_freq.device)
        return self

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        seq_len = x.shape[-2]
        # fp32 tables whatever dtype the module was cast to: a bf16 table is off by radians at T ~ 1000
        inv = self.inv_freq.float()
        t = torch.arange(seq_len, device=x.device, dtype=torch.float32)
        freqs = torch.outer(t, inv)
        emb = torch.cat((freqs, freqs), dim=-1)
        return apply_rotary_pos_emb(x, emb.cos()[None], emb.sin()[None])
