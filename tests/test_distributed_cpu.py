"""The N > 1 path on CPU: pairs shard across ranks with no data-path collective, trainable gradients are averaged with one
flat all-reduce, timings reduce by max.  Two `gloo` ranks, spawned as child processes."""
import os
import socket

import pytest

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mint_plus_b200.distributed import (FlatGradAllReduce, BucketedGradAllReduce, ChunkedGradAllReduce, balanced_shards, reduce_max, reduce_sum,
                                        shard_indices, snake_shards)
from mint_plus_b200.lora import LoRALinear, apply_lora


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)                                   # same parameters on every rank
        model = torch.nn.Sequential(torch.nn.Linear(8, 8), torch.nn.Linear(8, 4))
        model[0].weight.requires_grad_(False)                  # frozen parameters are not exchanged
        data = torch.arange(6 * 8, dtype=torch.float32).view(6, 8) / 10.0
        mine = shard_indices(6, rank, world)
        model(data[mine]).square().sum().backward()
        sync = FlatGradAllReduce(model.parameters())
        assert sync.nbytes == 4 * (8 + 4 * 8 + 4)
        sync()
        tmax = reduce_max([float(rank + 1), 5.0 - rank], "cpu")
        tsum = reduce_sum([float(len(mine))], "cpu")
        torch.save({"grads": [p.grad.clone() for p in model.parameters() if p.requires_grad], "tmax": tmax, "tsum": tsum,
                    "mine": mine}, os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_two_ranks_average_trainable_gradients_over_disjoint_shards(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    r0, r1 = (torch.load(tmp_path / f"rank{r}.pt") for r in range(world))
    assert sorted(r0["mine"] + r1["mine"]) == list(range(6)) and not set(r0["mine"]) & set(r1["mine"])
    # both ranks end with the same gradients: the mean of the per-shard gradients
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(8, 8), torch.nn.Linear(8, 4))
    model[0].weight.requires_grad_(False)
    data = torch.arange(6 * 8, dtype=torch.float32).view(6, 8) / 10.0
    want = None
    for r in range(world):
        model.zero_grad()
        model(data[shard_indices(6, r, world)]).square().sum().backward()
        g = [p.grad.clone() for p in model.parameters() if p.requires_grad]
        want = g if want is None else [a + b for a, b in zip(want, g)]
    want = [w / world for w in want]
    for got0, got1, w in zip(r0["grads"], r1["grads"], want):
        torch.testing.assert_close(got0, w)
        torch.testing.assert_close(got1, w)
    assert r0["tmax"] == [2.0, 5.0] and r1["tmax"] == [2.0, 5.0]
    assert r0["tsum"] == [6.0]


def _overlap_worker(rank, world, port, out_dir, with_unused, overlap):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        model = torch.nn.Sequential(torch.nn.Linear(8, 8), torch.nn.Tanh(), torch.nn.Linear(8, 8), torch.nn.Linear(8, 4))
        unused = torch.nn.Parameter(torch.ones(3))             # never reached by the loss: counts as a zero gradient
        params = list(model.parameters()) + ([unused] if with_unused else [])
        # small buckets, filled in reverse registration order: `unused` shares the first one, which therefore only goes out in finish()
        sync = BucketedGradAllReduce(params, bucket_bytes=140, overlap=overlap)
        data = torch.arange(6 * 8, dtype=torch.float32).view(6, 8) / 10.0
        mine = shard_indices(6, rank, world)
        results = []
        launched_in_backward = []
        for step in range(2):                                  # the second step checks that the state resets
            for p in params:
                p.grad = None
            model(data[mine] * (step + 1)).square().sum().backward()
            launched_in_backward.append(sum(b.launched for b in sync.buckets))
            sync.finish()
            results.append([p.grad.clone() for p in params])
        views = all(p.grad.data_ptr() == sync._where[p][1].data_ptr() for p in params)
        torch.save({"grads": results, "views": views, "n_buckets": len(sync.buckets), "nbytes": sync.nbytes,
                    "launched_in_backward": launched_in_backward},
                   os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("with_unused,overlap", [(False, True), (True, True), (False, False)])
def test_two_ranks_bucketed_gradient_average(tmp_path, with_unused, overlap):
    world = 2
    mp.spawn(_overlap_worker, args=(world, _free_port(), str(tmp_path), with_unused, overlap), nprocs=world, join=True)
    r0, r1 = (torch.load(tmp_path / f"rank{r}.pt") for r in range(world))
    assert r0["n_buckets"] >= 3 and r0["views"] and r1["views"]
    assert r0["nbytes"] == 4 * ((3 if with_unused else 0) + 2 * (64 + 8) + 32 + 4)
    # with every gradient arriving, all buckets are on the wire before backward() returns; a parameter without a gradient
    # holds its bucket (and, to keep one order on all ranks, the later ones) back until finish()
    assert r0["launched_in_backward"] == ([0, 0] if (with_unused or not overlap) else [r0["n_buckets"]] * 2)
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(8, 8), torch.nn.Tanh(), torch.nn.Linear(8, 8), torch.nn.Linear(8, 4))
    data = torch.arange(6 * 8, dtype=torch.float32).view(6, 8) / 10.0
    for step in range(2):
        want = None
        for r in range(world):
            model.zero_grad()
            model(data[shard_indices(6, r, world)] * (step + 1)).square().sum().backward()
            g = [p.grad.clone() for p in model.parameters()]
            want = g if want is None else [a + b for a, b in zip(want, g)]
        want = [w / world for w in want] + ([torch.zeros(3)] if with_unused else [])
        for got0, got1, w in zip(r0["grads"][step], r1["grads"][step], want):
            torch.testing.assert_close(got0, w)
            torch.testing.assert_close(got1, w)


def test_balanced_shards_even_out_skewed_costs():
    lengths = [1900, 30, 1800, 40, 900, 950, 50, 60]
    shards = balanced_shards([l * l for l in lengths], 2)
    assert sorted(shards[0] + shards[1]) == list(range(8))
    loads = [sum(lengths[i] ** 2 for i in s) for s in shards]
    assert max(loads) / min(loads) < 1.35
    assert balanced_shards([1, 1, 1], 4)[3] == []


class _Stack(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.embed = torch.nn.Linear(8, 8)
        self.layers = torch.nn.ModuleList([torch.nn.Linear(8, 8) for _ in range(5)])
        self.lm_head = torch.nn.Linear(8, 4)
        self.lm_head.weight = torch.nn.Parameter(self.lm_head.weight.detach().clone())

    def forward(self, x):
        x = self.embed(x)
        for layer in self.layers:
            x = torch.tanh(layer(x))
        return self.lm_head(x)


def _chunk_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        model = _Stack()
        model.layers[1].bias.requires_grad_(False)
        sync = ChunkedGradAllReduce(model, n_chunks=3)
        data = torch.arange(6 * 8, dtype=torch.float32).view(6, 8) / 10.0
        mine = shard_indices(6, rank, world)
        results, early = [], []
        for step in range(2):
            for p in model.parameters():
                p.grad = None
            model(data[mine] * (step + 1)).square().sum().backward()
            early.append(sync.finish())
            results.append({n: p.grad.clone() for n, p in model.named_parameters() if p.requires_grad})
        views = all(p.grad.untyped_storage().data_ptr() == sync.flat.untyped_storage().data_ptr()
                    for p in model.parameters() if p.requires_grad)
        torch.save({"grads": results, "early": early, "views": views}, os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_two_ranks_chunked_gradient_average_leaves_during_backward(tmp_path):
    world = 2
    mp.spawn(_chunk_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    r0, r1 = (torch.load(tmp_path / f"rank{r}.pt") for r in range(world))
    assert r0["early"] == [2, 2] and r1["early"] == [2, 2] and r0["views"]      # two of three chunks left before finish()
    torch.manual_seed(0)
    model = _Stack()
    data = torch.arange(6 * 8, dtype=torch.float32).view(6, 8) / 10.0
    for step in range(2):
        want = None
        for r in range(world):
            model.zero_grad()
            model(data[shard_indices(6, r, world)] * (step + 1)).square().sum().backward()
            g = {n: p.grad.clone() for n, p in model.named_parameters()}
            want = g if want is None else {n: want[n] + g[n] for n in g}
        for n, got in r0["grads"][step].items():
            torch.testing.assert_close(got, want[n] / world)
            torch.testing.assert_close(r1["grads"][step][n], want[n] / world)
        assert "layers.1.bias" not in r0["grads"][step]


def test_snake_shards_give_equal_counts_and_even_costs():
    g = torch.Generator().manual_seed(3)
    lengths = torch.randint(200, 1800, (128,), generator=g).tolist()
    costs = [float(l) ** 2 for l in lengths]
    shards = snake_shards(costs, 8)
    assert sorted(i for s in shards for i in s) == list(range(128)) and all(len(s) == 16 for s in shards)
    loads = [sum(costs[i] for i in s) for s in shards]
    naive = [sum(costs[i] for i in shard_indices(128, r, 8)) for r in range(8)]
    assert max(loads) / min(loads) < 1.05 < max(naive) / min(naive)
    assert snake_shards([3.0, 1.0, 2.0], 1) == [[0, 1, 2]]


def test_lora_adapter_freezes_base_and_matches_the_formula():
    torch.manual_seed(1)
    lin = torch.nn.Linear(16, 12)
    lora = LoRALinear(lin, r=4, alpha=8.0)
    with torch.no_grad():
        lora.lora_B.normal_(0, 0.1)
    x = torch.randn(5, 16)
    want = lin(x) + (x @ lora.lora_A.t()) @ lora.lora_B.t() * 2.0
    torch.testing.assert_close(lora(x), want)
    assert not lin.weight.requires_grad and lora.lora_A.requires_grad

    class Layer(torch.nn.Module):
        def __init__(self):
            super().__init__()
            import mint_plus_b200 as M
            self.self_attn = M.MultiHeadAttention(16, 2, use_rotary_embeddings=True)
            self.multimer_attn = M.MultiHeadAttention(16, 2, no_proj=True)

    class Model(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.layers = torch.nn.ModuleList([Layer()])

    m = apply_lora(Model())
    names = [n for n, p in m.named_parameters() if p.requires_grad]
    assert len(names) == 2 * 7 and all("lora_" in n for n in names)      # self q,k,v,out + cross q,k,v
