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


class GraphedTrainStep:
    """One training step - gradients dropped, MLM corruption, forward, masked cross-entropy, backward, then an optional
    callable (a gradient all-reduce, say) - captured once into a CUDA graph and replayed.  A step of a small model is a few
    thousand short kernels, and the host needs longer to launch them than the GPU to run them; replayed, the step costs the
    host one launch.  The batch shape is fixed by the example batch; `step(tokens, chain_ids)` copies a batch (device or
    pinned host tensors) into the graph's input buffers, replays, and returns the loss (a device scalar that the next
    replay overwrites).  The gradients are in `p.grad` of the parameters afterwards, at the same addresses every step.

    What the graph freezes: every value the library hands to its kernels by value at capture time.  For bf16 models there
    is none that changes; for FP8 models the per-tensor scales of the capture are replayed, so a loop that updates the
    weights has to run eagerly (or re-capture after `Fp8WeightScaler.refresh()`).  The MLM corruption is drawn by the
    device generator inside the graph and differs from replay to replay, as in eager mode.  Before constructing one, drop
    every reference to losses of earlier eager steps: a live autograd graph keeps its gradient-accumulation nodes bound to
    the stream they ran on, and their synchronisation with that stream invalidates the capture."""

    def __init__(self, model, tokens: torch.Tensor, chain_ids: torch.Tensor, params=None, after_backward=None, warmup: int = 2):
        dev = next(model.parameters()).device
        if dev.type != "cuda":
            raise RuntimeError("GraphedTrainStep needs a model on a CUDA device")
        self.model = model
        self.params = [p for p in (model.parameters() if params is None else params) if p.requires_grad]
        self.after_backward = after_backward
        self.tokens = tokens.to(dev).clone()
        self.chain_ids = chain_ids.to(dev).clone()
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):            # warm-up off the capturing stream: allocations, first-use measurements
            for _ in range(max(1, warmup)):
                self._body()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.loss = self._body()

    def _body(self) -> torch.Tensor:
        for p in self.params:
            p.grad = None
        loss, _ = shared_step(self.model, (self.tokens, self.chain_ids))
        loss.backward()
        if self.after_backward is not None:
            self.after_backward()
        return loss.detach()

    def step(self, tokens: Optional[torch.Tensor] = None, chain_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        if tokens is not None:
            self.tokens.copy_(tokens, non_blocking=True)
        if chain_ids is not None:
            self.chain_ids.copy_(chain_ids, non_blocking=True)
        self.graph.replay()
        return self.loss

    __call__ = step
