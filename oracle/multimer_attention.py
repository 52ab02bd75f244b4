"""CPU oracle for the two-pathway combined-softmax multimer attention.

TEST INFRASTRUCTURE ONLY.  This module is the checker: tests, the smoke check
and the benchmark's CPU-baseline leg may import it; the product package never
does.  It restates, in plain PyTorch fp32 on the CPU, the algorithm of the
reference's PyTorch (non-Triton) path:

  * projection-level steps     mint_plus/models/attention.py:172-242 (self pathway,
                               scaling 188, RoPE 219-220, bmm 223, key-padding fill 230-236)
                               mint_plus/models/attention.py:325-371 (cross pathway, no RoPE)
  * RoPE                       mint_plus/models/rotary_embedding.py:16-55
  * combine / softmax / split  mint_plus/models/modules.py:129-144 with the fp32 softmax of
                               mint_plus/models/mu_scaling/layer.py:159-165
  * sqrt-softmax               mint_plus/models/mu_scaling/layer.py:162-163
  * materialised-logit combine mint_plus/models/kernels/__init__.py:179-242 (same math from logits)

Parity pin: the reference holds no golden vectors for this path, so the oracle is pinned
against outputs of the reference's own modules run in the build container; the generating
script is tests/golden/make_golden.py and the vectors it wrote are tests/golden/*.npz.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------- RoPE
def rope_tables(T: int, D: int, dtype=torch.float32) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables (T, D), rotary_embedding.py:40-53: inv_freq[i] = 10000^(-2i/D),
    angle = position * inv_freq, the half-table duplicated along the last dim.  The position
    is the index in the padded, concatenated sequence (chain 2 does not restart at 0)."""
    inv_freq = 1.0 / (10000 ** (torch.arange(0, D, 2).float() / D))
    t = torch.arange(T).type_as(inv_freq)
    freqs = torch.outer(t, inv_freq)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """rotary_embedding.py:16-18: (x1, x2) -> (-x2, x1) on the two halves of the last dim."""
    x1, x2 = x.chunk(2, dim=-1)
    return torch.cat((-x2, x1), dim=-1)


def apply_rope(x: torch.Tensor) -> torch.Tensor:
    """rotary_embedding.py:21-24 on x[..., T, D]."""
    T, D = x.shape[-2], x.shape[-1]
    cos, sin = rope_tables(T, D, torch.float32)
    return x * cos + rotate_half(x) * sin


# --------------------------------------------------------------------------- masks
def chain_mask_from_ids(chain_ids: torch.Tensor) -> torch.Tensor:
    """esm2.py:89: True where the two positions belong to different chains -> (B, T, T) bool."""
    return ~torch.eq(chain_ids.unsqueeze(-1), chain_ids.unsqueeze(-2))


# --------------------------------------------------------------------------- the op
def combined_logits(q_self, k_self, q_cross, k_cross, chain_mask, key_pad=None,
                    scale: Optional[float] = None, rope: bool = True):
    """Pre-softmax logits of both pathways, selected per (query, key) by the chain mask.

    q/k: (B, H, T, D).  `scale` multiplies both Q (attention.py:188, 349); `rope` rotates the
    self pathway's Q and K only (modules.py:56-61).  Padded KEY columns are -inf in both
    pathways before the select (attention.py:230-236); padded QUERY rows are ordinary rows.
    """
    D = q_self.shape[-1]
    if scale is None:
        scale = D ** -0.5
    qs, qc = q_self * scale, q_cross * scale
    ks = k_self
    if rope:
        qs, ks = apply_rope(qs), apply_rope(ks)
    intra = torch.matmul(qs, ks.transpose(-1, -2))
    inter = torch.matmul(qc, k_cross.transpose(-1, -2))
    if key_pad is not None:
        fill = key_pad[:, None, None, :]
        intra = intra.masked_fill(fill, float("-inf"))
        inter = inter.masked_fill(fill, float("-inf"))
    return torch.where(chain_mask[:, None], inter, intra)


def multimer_attention(q_self, k_self, v_self, q_cross, k_cross, v_cross, chain_mask,
                       key_pad=None, scale: Optional[float] = None, rope: bool = True,
                       sqrt_softmax: bool = False, return_lse: bool = False):
    """out[B,H,T,D] = (P o ~M) V_self + (P o M) V_cross, P = softmax over keys of the combined logits
    (modules.py:129-144; fp32 softmax as mu_scaling/layer.py:159).  Tensors are computed in the dtype
    given (use fp32 for the tolerance anchor)."""
    logits = combined_logits(q_self, k_self, q_cross, k_cross, chain_mask, key_pad, scale, rope)
    probs = F.softmax(logits, dim=-1, dtype=torch.float32)
    if sqrt_softmax:
        # sqrt(p) with the derivative at p = 0 (padded keys) taken as 0; autograd through a plain sqrt gives 0 * inf = NaN
        # there, which is what the reference's PyTorch path produces when a batch holds padding (mu_scaling/layer.py:162-163)
        live = probs > 0
        probs = torch.where(live, probs, torch.ones_like(probs)).sqrt() * live
    probs = probs.to(v_self.dtype)
    m = chain_mask[:, None]
    out = torch.matmul(probs.masked_fill(m, 0.0), v_self) + torch.matmul(probs.masked_fill(~m, 0.0), v_cross)
    if return_lse:
        return out, torch.logsumexp(logits.float(), dim=-1)
    return out


def multimer_attention_fwd_bwd(q_self, k_self, v_self, q_cross, k_cross, v_cross, chain_mask, grad_out,
                               key_pad=None, scale=None, rope=True, sqrt_softmax=False):
    """Forward + torch.autograd backward through `multimer_attention` (what the reference's PyTorch
    path differentiates).  Returns (out, (dq_s, dk_s, dv_s, dq_c, dk_c, dv_c))."""
    leaves = [t.detach().clone().requires_grad_(True) for t in (q_self, k_self, v_self, q_cross, k_cross, v_cross)]
    out = multimer_attention(*leaves, chain_mask, key_pad, scale, rope, sqrt_softmax)
    grads = torch.autograd.grad(out, leaves, grad_out)
    return out.detach(), tuple(grads)


def combine_from_logits(intra_logits, inter_logits, chain_mask, intra_values, inter_values):
    """kernels/__init__.py:179-242 semantics from materialised logits (B,H,T,T): select, softmax
    (fp32), split by mask, two weighted sums."""
    m = chain_mask[:, None]
    probs = F.softmax(torch.where(m, inter_logits, intra_logits), dim=-1, dtype=torch.float32).to(intra_values.dtype)
    return torch.matmul(probs.masked_fill(m, 0.0), intra_values) + torch.matmul(probs.masked_fill(~m, 0.0), inter_values)


# --------------------------------------------------------------------------- layer-level pieces
def gelu_erf(x):
    """modules.py:16-23: x * 0.5 * (1 + erf(x / sqrt(2)))."""
    return x * 0.5 * (1.0 + torch.erf(x / math.sqrt(2.0)))


def project_qkv_4d(x, weight, bias, H):
    """attention.py:304-323: fused Linear(E, 3E) with rows ordered [Q;K;V], then (T,B,E) -> (B,H,T,D)."""
    T, B, E = x.shape
    D = E // H
    qkv = F.linear(x, weight, bias)
    q, k, v = qkv.chunk(3, dim=-1)
    return tuple(t.reshape(T, B, H, D).permute(1, 2, 0, 3).contiguous() for t in (q, k, v))


def fp8_e4m3_linear(x, weight, bias=None, out_scale: float = 1.0):
    """Per-tensor-scaled e4m3 linear, restating mint_plus/models/alt/munit_scaling.py:22-34:
    clamp to +-448, cast x and W to e4m3, fp32-accumulated matmul, + bias, x static output scale.
    Parity unpinned: the production FP8 arithmetic lives in transformer_engine 2.16.0, which is not
    vendored in the reference and not installed in the build container."""
    xq = x.float().clamp(-448.0, 448.0).to(torch.float8_e4m3fn).float()
    wq = weight.float().clamp(-448.0, 448.0).to(torch.float8_e4m3fn).float()
    y = xq @ wq.t()
    if bias is not None:
        y = y + bias.float()
    return y * out_scale


# --------------------------------------------------------------------------- synthetic inputs
def make_op_inputs(B, H, T, D, seed, dtype=torch.float32, split_lo=None, split_hi=None, max_pad=64):
    """Seeded inputs of the isolated-op benchmark shape: six N(0,1)/sqrt(D) tensors, a chain split point
    per sample uniform in [split_lo, split_hi], 0..max_pad trailing padded positions, N(0,1) upstream grad."""
    g = torch.Generator().manual_seed(seed)
    ts = [(torch.randn(B, H, T, D, generator=g) / math.sqrt(D)).to(dtype) for _ in range(6)]
    split_lo = T * 200 // 1024 if split_lo is None else split_lo
    split_hi = T * 824 // 1024 if split_hi is None else split_hi
    split = torch.randint(split_lo, split_hi + 1, (B,), generator=g)
    pad = torch.randint(0, min(max_pad, max(T - int(split.max()) - 1, 0)) + 1, (B,), generator=g)
    chain_ids = torch.zeros(B, T, dtype=torch.int32)
    key_pad = torch.zeros(B, T, dtype=torch.bool)
    for b in range(B):
        chain_ids[b, int(split[b]):] = 1
        if int(pad[b]) > 0:
            key_pad[b, T - int(pad[b]):] = True
    grad = torch.randn(B, H, T, D, generator=g).to(dtype)
    return ts, chain_ids, key_pad, grad
