"""The masked-language-model training step of the reference's Lightning wrapper, as a plain function
(mint_plus/training/wrapper.py:48-86 `_shared_step`): 15 % of the non-special positions become targets, of those 80 % are
replaced by <mask>, 10 % by a random amino acid, 10 % kept; the loss is the cross-entropy averaged over the targets.
Trainer, optimiser and logging are outside this package."""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F


def mlm_corrupt(tokens: torch.Tensor, cls_idx: int, eos_idx: int, padding_idx: int, mask_idx: int,
                generator: Optional[torch.Generator] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """(corrupted tokens, boolean target mask), drawn on the tokens' device."""
    special = tokens.eq(cls_idx) | tokens.eq(eos_idx) | tokens.eq(padding_idx)
    dev = tokens.device
    target = (torch.rand(tokens.shape, device=dev, generator=generator) < 0.15) & ~special
    rand = torch.rand(tokens.shape, device=dev, generator=generator)
    randaa = torch.randint(4, 24, tokens.shape, device=dev, generator=generator)
    inp = torch.where((rand < 0.8) & target, torch.full_like(tokens, mask_idx), tokens)
    inp = torch.where((rand > 0.9) & target, randaa, inp)
    return inp, target


def shared_step(model, batch, generator: Optional[torch.Generator] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """(loss, perplexity) of one batch (tokens (B,T), chain_ids (B,T))."""
    tokens, chain_ids = batch
    inp, target = mlm_corrupt(tokens, 0, model.eos_idx, model.padding_idx, model.mask_idx, generator)
    out = model(inp, chain_ids=chain_ids)["logits"]
    if out.is_cuda and out.dtype == torch.bfloat16:
        from . import ops
        loss = ops.masked_cross_entropy(out, tokens, target)      # one pass over the logits, fp32 arithmetic
    else:
        loss = F.cross_entropy(out.float().transpose(1, 2), tokens, reduction="none")
        loss = (loss * target).sum() / target.sum()
    return loss, torch.exp(loss.detach())
