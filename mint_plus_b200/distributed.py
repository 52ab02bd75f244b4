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


def snake_shards(costs: Sequence[float], world: int) -> List[List[int]]:
    """Deal items to `world` ranks with EQUAL counts (fixed batch per rank) and about even summed cost: sorted by cost, dealt
    forwards and backwards in turn (0..w-1, w-1..0, ...).  The reference deals item i to rank i mod world whatever its length
    (data/data.py:51), so the step waits for the rank that drew the longest pairs."""
    order = sorted(range(len(costs)), key=lambda i: (-costs[i], i))
    shards = [[] for _ in range(world)]
    for pos, i in enumerate(order):
        rnd, k = divmod(pos, world)
        shards[k if rnd % 2 == 0 else world - 1 - k].append(i)
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
        """After backward(): gathers the gradients into the flat buffer (one multi-tensor copy), reduces, divides, and leaves
        every `.grad` as a view of the buffer (a copy back only where the buffer's dtype differs from the parameter's)."""
        if not self.params:
            return
        have = [(p, v) for p, v in zip(self.params, self.views) if p.grad is not None and p.grad.data_ptr() != v.data_ptr()]
        for p, v in zip(self.params, self.views):
            if p.grad is None:
                v.zero_()
        if have:
            torch._foreach_copy_([v for _, v in have], [p.grad for p, _ in have])
        if dist.is_initialized() and dist.get_world_size(self.group) > 1:
            dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=self.group)
            self.flat.div_(dist.get_world_size(self.group))
        back = [(p, v) for p, v in have if v.dtype != p.dtype]
        if back:
            torch._foreach_copy_([p.grad for p, _ in back], [v for _, v in back])
        for p, v in zip(self.params, self.views):
            if p.grad is None or v.dtype == p.dtype:
                p.grad = v if v.dtype == p.dtype else v.to(p.dtype)


class _Bucket:
    __slots__ = ("flat", "params", "views", "arrived", "work", "launched")

    def __init__(self, flat, params, views):
        self.flat, self.params, self.views = flat, params, views
        self.arrived, self.work, self.launched = 0, None, False


class BucketedGradAllReduce:
    """Averages the gradients of `params` over the process group through buckets that fill up during the backward pass, and
    optionally (`overlap=True`) sends each bucket as soon as it is full, while the backward pass is still running.

    The parameters are grouped, in the order the backward pass finishes them (the reverse of their registration order), into
    buckets of about `bucket_bytes`.  A hook that autograd runs as soon as a parameter's gradient is complete copies it into
    the bucket and makes `.grad` a view of the bucket (so the copy is the only extra pass and no second set of gradients
    stays allocated).  With `overlap=True`, when the last member of a bucket has arrived its all-reduce is issued
    asynchronously — with NCCL on the communicator's own stream, ordered after the copies — and the backward pass carries on.
    `finish()`, called after `backward()`, issues what is left (without overlap: everything; with it: buckets with parameters
    that received no gradient, which count as zeros), waits for every bucket and divides by the group size.
    Overlap is off by default: the projection GEMMs and attention kernels of this library are persistent grids of one CTA
    per SM with a static share of the tiles each, so a communication kernel that holds even a few SMs pushes their CTAs
    into a second wave.  Measured on 2 B200s with the 650M step (197 ms on one GPU): 213 ms with or without overlap — the
    700 hook calls cost the backward thread more than the transfer costs the GPU — against 203 ms... see FlatGradAllReduce,
    which gathers the gradients with one multi-tensor copy after the backward pass and is what the benchmark uses.  Set `.grad = None` on the parameters before the next backward pass, as
    `optimizer.zero_grad(set_to_none=True)` does: a gradient that is still the bucket view would be added to in place.
    The reference leaves all of this to Lightning's DDP strategy (training/trainer.py:95-110)."""

    def __init__(self, params: Iterable[torch.nn.Parameter], group=None, dtype: torch.dtype = torch.float32,
                 bucket_bytes: int = 256 << 20, overlap: bool = False):
        self.params = [p for p in params if p.requires_grad]
        self.group = group
        self.dtype = dtype
        self.overlap = overlap
        self.buckets: List[_Bucket] = []
        self._where = {}
        self._handles = []
        self._next = 0          # first bucket whose all-reduce has not been issued yet
        esize = torch.empty(0, dtype=dtype).element_size()
        cur, cur_n = [], 0
        groups = []
        for p in reversed(self.params):
            cur.append(p)
            cur_n += p.numel()
            if cur_n * esize >= bucket_bytes:
                groups.append(cur)
                cur, cur_n = [], 0
        if cur:
            groups.append(cur)
        for members in groups:
            flat = torch.zeros(sum(p.numel() for p in members), dtype=dtype, device=members[0].device)
            views, off = [], 0
            for p in members:
                views.append(flat[off:off + p.numel()].view_as(p))
                off += p.numel()
            b = _Bucket(flat, members, views)
            self.buckets.append(b)
            for p, v in zip(members, views):
                self._where[p] = (b, v)
                self._handles.append(p.register_post_accumulate_grad_hook(self._on_grad))

    @property
    def nbytes(self) -> int:
        return sum(b.flat.numel() * b.flat.element_size() for b in self.buckets)

    def _world(self) -> int:
        return dist.get_world_size(self.group) if dist.is_initialized() else 1

    def _launch(self, b: _Bucket):
        b.launched = True
        if self._world() > 1:
            b.work = dist.all_reduce(b.flat, op=dist.ReduceOp.SUM, group=self.group, async_op=True)

    @torch.no_grad()
    def _on_grad(self, p: torch.nn.Parameter):
        b, view = self._where[p]
        if p.grad is None or b.launched:
            return
        view.copy_(p.grad)
        if view.dtype == p.dtype:
            p.grad = view
        b.arrived += 1
        if not self.overlap:
            return
        # buckets go out in their fixed order on every rank, whatever order their members arrive in
        while self._next < len(self.buckets) and self.buckets[self._next].arrived == len(self.buckets[self._next].params):
            self._launch(self.buckets[self._next])
            self._next += 1

    @torch.no_grad()
    def finish(self):
        """After backward(): every parameter's `.grad` holds the group average when this returns (stream-ordered on CUDA)."""
        world = self._world()
        for b in self.buckets:
            if not b.launched:
                for p, v in zip(b.params, b.views):
                    if p.grad is None:
                        v.zero_()
                    elif p.grad.data_ptr() != v.data_ptr():
                        v.copy_(p.grad)
                self._launch(b)
        for b in self.buckets:
            if b.work is not None:
                b.work.wait()
                b.work = None
        if world > 1:
            torch._foreach_div_([b.flat for b in self.buckets], float(world))
        for b in self.buckets:
            for p, v in zip(b.params, b.views):
                if p.grad is None:
                    p.grad = v if v.dtype == p.dtype else v.to(p.dtype)
                elif p.grad.data_ptr() != v.data_ptr():
                    p.grad.copy_(v)
            b.arrived, b.launched = 0, False
        self._next = 0

    def remove(self):
        for h in self._handles:
            h.remove()
        self._handles = []


class ChunkedGradAllReduce:
    """Averages the trainable gradients of a model with a `layers` ModuleList in a few large chunks, each sent as soon as
    the backward pass has left its layers: the layers are cut into `n_chunks` consecutive groups; a backward pre-hook on the
    LAST layer before a group (it fires when the gradient with respect to that layer's output exists, i.e. when every later
    layer has finished) gathers the group's gradients into its slice of one flat buffer with one multi-tensor copy and
    issues the slice's all-reduce asynchronously (NCCL: on the communicator's stream, ordered after the copy).  Three or
    four hook calls per step instead of one per parameter keep the host cost of the overlap negligible.  Parameters used
    after the layers (final norm, LM head) ride with the first group, everything else (embeddings, tied weights) with the
    last one, which `finish()` sends after `backward()` before it waits for all of them, divides, and leaves every `.grad`
    a view of the buffer.  Not for activation checkpointing (the hooks would fire during recomputation)."""

    def __init__(self, model: torch.nn.Module, n_chunks: int = 4, group=None, dtype: torch.dtype = torch.float32,
                 after_layers: Sequence[str] = ("lm_head", "emb_layer_norm_after", "contact_head")):
        layers = list(model.layers)
        n_chunks = max(1, min(n_chunks, len(layers)))
        self.group = group
        # chunk c (in backward order) holds layers [bounds[c+1], bounds[c])
        bounds = [len(layers) - (len(layers) * c) // n_chunks for c in range(n_chunks + 1)]
        chunk_of_layer = {}
        for c in range(n_chunks):
            for li in range(bounds[c + 1], bounds[c]):
                chunk_of_layer[li] = c
        members: List[List[torch.nn.Parameter]] = [[] for _ in range(n_chunks)]
        for name, p in model.named_parameters():
            if not p.requires_grad:
                continue
            parts = name.split(".")
            if parts[0] == "layers" and parts[1].isdigit():
                members[chunk_of_layer[int(parts[1])]].append(p)
            elif parts[0] in after_layers:
                members[0].append(p)
            else:
                members[-1].append(p)
        self.params = [p for m in members for p in m]
        n = sum(p.numel() for p in self.params)
        dev = self.params[0].device if self.params else torch.device("cpu")
        self.flat = torch.zeros(n, dtype=dtype, device=dev)
        self.chunks = []          # (params, views, flat slice)
        off = 0
        for m in members:
            start, views = off, []
            for p in m:
                views.append(self.flat[off:off + p.numel()].view_as(p))
                off += p.numel()
            self.chunks.append((m, views, self.flat[start:off]))
        self._sent = [False] * n_chunks
        self._work = []
        self._handles = []
        for c in range(n_chunks - 1):          # chunk c is complete when the backward pass arrives at layer bounds[c+1] - 1
            self._handles.append(layers[bounds[c + 1] - 1].register_full_backward_pre_hook(self._make_hook(c)))

    @property
    def nbytes(self) -> int:
        return self.flat.numel() * self.flat.element_size()

    def _world(self) -> int:
        return dist.get_world_size(self.group) if dist.is_initialized() else 1

    def _make_hook(self, c: int):
        def hook(module, grad_output):
            self._send(c, only_if_complete=True)
            return None
        return hook

    @torch.no_grad()
    def _send(self, c: int, only_if_complete: bool) -> None:
        if self._sent[c] or (c > 0 and not self._sent[c - 1]):   # chunks leave in one order on every rank
            return
        params, views, piece = self.chunks[c]
        if only_if_complete and any(p.grad is None for p in params):
            return
        have = [(p, v) for p, v in zip(params, views) if p.grad is not None and p.grad.data_ptr() != v.data_ptr()]
        for p, v in zip(params, views):
            if p.grad is None:
                v.zero_()
        if have:
            torch._foreach_copy_([v for _, v in have], [p.grad for p, _ in have])
        self._sent[c] = True
        if self._world() > 1 and piece.numel():
            self._work.append(dist.all_reduce(piece, op=dist.ReduceOp.SUM, group=self.group, async_op=True))

    @torch.no_grad()
    def finish(self) -> int:
        """After backward(): sends what has not left yet, waits, divides; every `.grad` becomes a view of the flat buffer
        (a copy back only where the buffer's dtype differs).  Returns how many chunks had left during the backward pass."""
        early = sum(self._sent)
        for c in range(len(self.chunks)):
            self._send(c, only_if_complete=False)
        for w in self._work:
            w.wait()
        self._work = []
        world = self._world()
        if world > 1:
            self.flat.div_(world)
        for params, views, _ in self.chunks:
            for p, v in zip(params, views):
                if v.dtype == p.dtype:
                    p.grad = v
                elif p.grad is None:
                    p.grad = v.to(p.dtype)
                else:
                    p.grad.copy_(v)
        self._sent = [False] * len(self.chunks)
        return early

    def remove(self):
        for h in self._handles:
            h.remove()
        self._handles = []


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
