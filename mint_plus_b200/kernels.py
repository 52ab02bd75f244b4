"""The reference's kernel-level call signatures (mint_plus/models/kernels/*), served by libmintb.

    fused_multi_pathway_attention          kernels/multi_pathway_attention.py:184-223
    differentiable_multi_pathway_attention kernels/differentiable_attention.py:69-85
    fused_multimer_combine                 kernels/__init__.py:179-199
    differentiable_multimer_combine        kernels/differentiable_attention.py:127-140

Differences from the reference, all on the side of what its PyTorch path computes: the results carry
autograd history whenever an input requires grad (the gradients equal torch.autograd through the
PyTorch path, not the reference's Triton backward); a `key_padding_mask` keyword is accepted by the
fused entry points, which the reference's fused kernel silently drops; dropout_p must be 0 (it is 0 in
every reference configuration) and `qpp` is accepted and ignored (a tuning knob of the Triton kernel).
"""
from __future__ import annotations

import torch

from . import ops


def _check_dropout(dropout_p: float, training: bool) -> None:
    if training and dropout_p != 0.0:
        raise NotImplementedError("attention dropout is not implemented (the reference never enables it)")


def fused_multi_pathway_attention(q_self, k_self, v_self, q_multi, k_multi, v_multi, chain_mask,
                                  dropout_p: float = 0.0, training: bool = True, qpp=None,
                                  sqrt_softmax: bool = False, key_padding_mask=None) -> torch.Tensor:
    """(B,H,T,D) x6 + chain_mask (B,T,T) bool -> (B,H,T,D).  As in the reference, Q is already scaled by
    D^-0.5 and the self pathway is already rotated by the caller."""
    _check_dropout(dropout_p, training)
    return ops.multimer_attention(q_self, k_self, v_self, q_multi, k_multi, v_multi, chain_mask=chain_mask,
                                  key_padding_mask=key_padding_mask, rope=False, scale=1.0,
                                  sqrt_softmax=sqrt_softmax)


def differentiable_multi_pathway_attention(q_self, k_self, v_self, q_multi, k_multi, v_multi, chain_mask,
                                           dropout_p: float = 0.0, training: bool = True, qpp=8,
                                           sqrt_softmax: bool = False, key_padding_mask=None) -> torch.Tensor:
    return fused_multi_pathway_attention(q_self, k_self, v_self, q_multi, k_multi, v_multi, chain_mask,
                                         dropout_p, training, qpp, sqrt_softmax, key_padding_mask)


def fused_multimer_combine(intra_logits, inter_logits, chain_mask, intra_values, inter_values,
                           dropout_p: float = 0.0) -> torch.Tensor:
    """Materialised (B,H,T,T) logits of both pathways -> (B,H,T,D)."""
    _check_dropout(dropout_p, True)
    return ops.multimer_combine(intra_logits, inter_logits, chain_mask, intra_values, inter_values)


def differentiable_multimer_combine(intra_logits, inter_logits, chain_mask, intra_values, inter_values,
                                    dropout_p: float = 0.0) -> torch.Tensor:
    return fused_multimer_combine(intra_logits, inter_logits, chain_mask, intra_values, inter_values, dropout_p)
