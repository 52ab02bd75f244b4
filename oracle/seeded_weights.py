"""Deterministic, name-keyed parameter values for model-level parity cases.

Test infrastructure only (used by tests/ and by tests/golden/make_golden.py): it lets the reference model in the
generating container and the model under test on another machine hold identical weights without shipping them —
every tensor of a state dict is refilled from a generator seeded by (seed, crc32 of its key), so the values do not
depend on construction order or on which module class owns the tensor.

Matrices get Xavier-uniform values, biases small non-zero values (so bias paths are exercised), norm gains values near
one.  Buffers (`inv_freq`, `_tau`) and the tied `lm_head.weight` alias are left alone.
"""
from __future__ import annotations

import math
import zlib

import numpy as np
import torch

SKIP_SUFFIXES = ("inv_freq", "_tau", "lm_head.weight")


def _values(key: str, shape, seed: int) -> torch.Tensor:
    rng = np.random.Generator(np.random.PCG64([seed, zlib.crc32(key.encode())]))
    u = torch.from_numpy(rng.random(size=tuple(shape), dtype=np.float64) * 2.0 - 1.0)
    if len(shape) == 2:
        bound = math.sqrt(6.0 / (shape[0] + shape[1]))
        return u * bound
    if "norm" in key and key.endswith("weight"):
        return 1.0 + 0.1 * u
    return 0.05 * u


def fill_state_dict_(module: torch.nn.Module, seed: int) -> torch.nn.Module:
    with torch.no_grad():
        for key, t in sorted(module.state_dict().items()):
            if key.endswith(SKIP_SUFFIXES):
                continue
            t.copy_(_values(key, t.shape, seed).to(t.dtype))
    return module


def c1_batch(seed: int = 1001, B: int = 4, T: int = 512, lo: int = 64, hi: int = 200):
    """Token / chain-id batch of the MINT-8M forward case: B pairs, per chain a length uniform in [lo, hi] of tokens
    uniform over the 20 standard amino-acid ids 4..23, laid out <cls> chain A <eos> <cls> chain B <eos>, padded with id 1
    to T; chain ids 0 for the first block and 1 from the second <cls> to the end (pads included)."""
    g = torch.Generator().manual_seed(seed)
    tokens = torch.full((B, T), 1, dtype=torch.int64)
    chain_ids = torch.zeros(B, T, dtype=torch.int64)
    for b in range(B):
        la, lb = (int(torch.randint(lo, hi + 1, (1,), generator=g)) for _ in range(2))
        a = torch.randint(4, 24, (la,), generator=g)
        c = torch.randint(4, 24, (lb,), generator=g)
        row = torch.cat([torch.tensor([0]), a, torch.tensor([2, 0]), c, torch.tensor([2])])
        tokens[b, :row.numel()] = row
        chain_ids[b, la + 2:] = 1
    return tokens, chain_ids
