"""Data-parallel plumbing around the attention path: pairs shard across ranks and only trainable gradients are exchanged.

The attention path itself has no collective — every protein pair (batch row) is independent through the forward and the
backward pass — so N GPUs run N independent shards.  Training adds one all-reduce (average) of the trainable gradients per
step, issued on a flat buffer (the reference leaves this to Lightning's DDP strategy, training/trainer.py:95-110; its data
loader deals sample i to rank i mod world, data/data.py:51).
"""
from __future__ import annotations

from typing import Iterable, List, Sequence

import torch
import torch.distributed as dist


def shard_indices(n_items: int, rank: int, world: int) -> List[int]:
    """Indices rank `rank` owns when items are dealt round-robin (i mod world == rank)."""
    return list(range(rank, n_items, world))


def balanced_shards(lengths: Sequence[int], world: int) -> List[List[int]]:
    """Deal items to `world` ranks so that the summed cost per rank is even: longest first, each to the lightest rank.
    Attention cost grows with the square of the unpadded length, projections linearly; `lengths` should be the cost."""
    order = sorted(range(len(lengths)), key=lambda i: -lengths[i])
    loads, shards = [0.0] * world, [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda k: (loads[k], len(shards[k])))
        shards[r].append(i)
        loads[r] += float(lengths[i])
    return [sorted(s) for s in shards]


class FlatGradAllReduce:
    """Averages the gradients of `params` over the process group with one all-reduce of one flat buffer per step."""

    def __init__(self, params: Iterable[torch.nn.Parameter], group=None, dtype: torch.dtype = torch.float32):
        self.params = [p for p in params if p.requires_grad]
        self.group = group
        n = sum(p.numel() for p in self.params)
        dev = self.params[0].device if self.params else torch.device("cpu")
        self.flat = torch.zeros(n, dtype=dtype, device=dev)
        self.views, off = [], 0
        for p in self.params:
            self.views.append(self.flat[off:off + p.numel()].view_as(p))
            off += p.numel()

    @property
    def nbytes(self) -> int:
        return self.flat.numel() * self.flat.element_size()

    @torch.no_grad()
    def __call__(self):
        if not self.params:
            return
        for p, v in zip(self.params, self.views):
            if p.grad is None:
                v.zero_()
            else:
                v.copy_(p.grad)
        if dist.is_initialized() and dist.get_world_size(self.group) > 1:
            dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=self.group)
            self.flat.div_(dist.get_world_size(self.group))
        for p, v in zip(self.params, self.views):
            if p.grad is None:
                p.grad = v.to(p.dtype).clone()
            else:
                p.grad.copy_(v)


def reduce_max(values: Sequence[float], device, group=None) -> List[float]:
    """Max over ranks of a few host scalars (timings)."""
    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return t.tolist()


def reduce_sum(values: Sequence[float], device, group=None) -> List[float]:
    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return t.tolist()
