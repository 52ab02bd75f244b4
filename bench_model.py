"""Whole-model workloads of bench.py (`--workload mint650m_fp8 | mint150m_lora | mint3b_infer | mint8m_fwd`).

Each is one of the reference's model-level configurations on seeded synthetic protein pairs (tokens uniform over the 20
amino-acid ids, `<cls> A <eos> <cls> B <eos>`, padded with id 1; chain ids 0/1), random-init weights of the named
architecture.  A step is one forward (+ backward) over the rank's batch of pairs; the metric is pairs per second over all
ranks.  Pairs shard across ranks with no data-path collective; training workloads add one flat all-reduce of the trainable
gradients per step.
"""
from __future__ import annotations

import json
import math
import os
import statistics
import time

import torch

WORKLOADS = {
    # the reference's 650M FP8 training configuration
    "mint650m_fp8": dict(layers=33, embed=1280, heads=20, pairs=16, T=2048, lo=100, hi=900, seed=4004, train=True,
                         kind="mu_fp8", dtype="e4m3 GEMMs / bf16 attention",
                         desc="MINT-650M muS Res-Post-LN, e4m3 projections, bf16 attention, fwd+bwd, 16 pairs padded to 2048"),
    # the reference's 150M LoRA training configuration
    "mint150m_lora": dict(layers=30, embed=640, heads=20, pairs=32, T=1024, lo=50, hi=500, seed=3003, train=True,
                          kind="lora", dtype="bf16",
                          desc="MINT-150M frozen base + LoRA r=8 on q/k/v/out, bf16, training step, 32 pairs padded to 1024"),
    # the reference's large inference (embedding extraction) configuration
    "mint3b_infer": dict(layers=36, embed=2560, heads=40, pairs=64, T=2048, lo=30, hi=80, lo2=800, hi2=1900, seed=5005,
                         train=False, kind="plus", dtype="bf16",
                         desc="MINT 36x2560 (40 heads) inference forward, bf16, 64 pairs with skewed chain lengths padded to 2048"),
    # the 650M training step followed by a fused AdamW step and the re-cast of every e4m3 weight copy (Fp8WeightScaler)
    "mint650m_fp8_optim": dict(layers=33, embed=1280, heads=20, pairs=16, T=2048, lo=100, hi=900, seed=4004, train=True,
                               kind="mu_fp8", dtype="e4m3 GEMMs / bf16 attention", optimizer="adamw",
                               desc="MINT-650M muS FP8 fwd+bwd + fused AdamW step + e4m3 weight re-cast, 16 pairs padded to 2048"),
    # the same two with padded positions dropped from the token-wise work and from the attention's query tiles
    # (MINT.pack_padding): same values at real positions, zeros at padded ones; FLOPs are counted on real tokens only
    "mint650m_fp8_packed": dict(layers=33, embed=1280, heads=20, pairs=16, T=2048, lo=100, hi=900, seed=4004, train=True,
                                kind="mu_fp8", dtype="e4m3 GEMMs / bf16 attention", pack=True,
                                desc="MINT-650M muS FP8 fwd+bwd, 16 pairs padded to 2048, padding dropped (variable-length packing)"),
    "mint3b_infer_packed": dict(layers=36, embed=2560, heads=40, pairs=64, T=2048, lo=30, hi=80, lo2=800, hi2=1900, seed=5005,
                                train=False, kind="plus", dtype="bf16", pack=True,
                                desc="MINT 36x2560 inference forward, 64 skewed pairs padded to 2048, padding dropped (variable-length packing)"),
    # the reference's CPU-runnable 8M forward configuration (a latency line; its parity is a test)
    "mint8m_fwd": dict(layers=6, embed=320, heads=20, pairs=4, T=512, lo=64, hi=200, seed=1001, train=False,
                       kind="base_fp32", dtype="f32",
                       desc="MINT-8M forward, fp32, 4 pairs padded to 512"),
}


def make_pairs(cfg, rank=0, world=1):
    """Seeded synthetic pairs of the workload's length distribution.  One global list of world x pairs pairs comes from one
    seed (the first `pairs` of it are the single-GPU batch); with several ranks the list is dealt so that every rank holds
    `pairs` of them with about the same attention cost (squared unpadded length, `distributed.snake_shards`)."""
    from mint_plus_b200.distributed import snake_shards
    g = torch.Generator().manual_seed(cfg["seed"])
    B, T = cfg["pairs"], cfg["T"]
    n = B * world
    tokens = torch.full((n, T), 1, dtype=torch.int64)
    chain_ids = torch.zeros(n, T, dtype=torch.int64)
    cost = []
    for b in range(n):
        la = int(torch.randint(cfg["lo"], cfg["hi"] + 1, (1,), generator=g))
        lb = int(torch.randint(cfg.get("lo2", cfg["lo"]), cfg.get("hi2", cfg["hi"]) + 1, (1,), generator=g))
        a = torch.randint(4, 24, (la,), generator=g)
        c = torch.randint(4, 24, (lb,), generator=g)
        row = torch.cat([torch.tensor([0]), a, torch.tensor([2, 0]), c, torch.tensor([2])])
        tokens[b, :row.numel()] = row
        chain_ids[b, la + 2:] = 1
        cost.append(float(row.numel()) ** 2)
    if world == 1:
        return tokens, chain_ids
    mine = torch.tensor(snake_shards(cost, world)[rank])
    return tokens[mine].contiguous(), chain_ids[mine].contiguous()


def build_model(cfg, device):
    import mint_plus_b200 as M
    from mint_plus_b200.lora import apply_lora
    torch.manual_seed(cfg["seed"])
    L_, E_, H_ = cfg["layers"], cfg["embed"], cfg["heads"]
    kind = cfg["kind"]
    with torch.device(device):          # parameters are created (and initialised) on the GPU
        if kind == "mu_fp8":
            model = M.build_mint_mu("650M", num_layers=L_, embed_dim=E_, attention_heads=H_, use_fp8=True, unit_scaled=True)
        elif kind == "lora":
            model = M.MINT(num_layers=L_, embed_dim=E_, attention_heads=H_, use_multimer=True)
        elif kind == "plus":
            model = M.MINT(num_layers=L_, embed_dim=E_, attention_heads=H_, use_multimer=True,
                           layer_factory=lambda: M.TransformerLayer_MINT_plus(E_, 4 * E_, H_, use_multimer=True))
        else:
            model = M.MINT(num_layers=L_, embed_dim=E_, attention_heads=H_, use_multimer=True, use_erf_gelu=True)
    if kind != "base_fp32":
        model = model.to(torch.bfloat16)
    model = model.to(device)
    for layer in model.layers:           # rotary tables in fp32 whatever the model dtype (as under bf16-mixed training)
        rot = layer.self_attn.rot_emb
        if rot is not None:
            rot.inv_freq = rot.inv_freq.float()
    if kind == "lora":
        apply_lora(model, r=8, alpha=16.0)
        with torch.no_grad():           # B = 0 would make dA identically zero at step 0: draw B ~ N(0, 0.02) instead
            for n, p in model.named_parameters():
                if n.endswith("lora_B"):
                    p.normal_(0.0, 0.02)
    model.train(cfg["train"])
    model.pack_padding = bool(cfg.get("pack", False))
    return model


def algorithmic_flops(cfg, tokens):
    """GEMMs: 30 E^2 per token per layer forward (both QKV projections, out_proj, FFN), x3 with dgrad+wgrad, x2 when the
    weights are frozen (LoRA; the low-rank terms are left out).  Attention: 4 H T Tk D forward, 14 with backward, Tk = the
    sample's unpadded keys, every query row of the padded length counted as the reference computes them."""
    L_, E_, H_ = cfg["layers"], cfg["embed"], cfg["heads"]
    D = E_ // H_
    B, T = tokens.shape
    tk = (tokens != 1).sum(1).double()
    if cfg.get("pack"):       # padding dropped: only real tokens go through the projections, only real queries through attention
        gemm_fwd = 30.0 * E_ * E_ * float(tk.sum()) * L_
        attn_fwd = float((4.0 * H_ * tk * tk * D).sum()) * L_
    else:
        gemm_fwd = 30.0 * E_ * E_ * B * T * L_
        attn_fwd = float((4.0 * H_ * T * tk * D).sum()) * L_
    if not cfg["train"]:
        return gemm_fwd + attn_fwd, gemm_fwd, attn_fwd
    gemm = gemm_fwd * (2.0 if cfg["kind"] == "lora" else 3.0)
    return gemm + 3.5 * attn_fwd, gemm, 3.5 * attn_fwd


def cpu_baseline(cfg, seconds_budget=25.0):
    """The same model restated on the host cores: the package's host-side model with its attention call routed to the
    oracle, fp32.  One layer on one pair is timed (forward, plus backward for training workloads) and scaled by layers x
    pairs — an extrapolation, stated as such."""
    import mint_plus_b200 as M
    from mint_plus_b200 import ops
    from oracle import multimer_attention as O
    torch.set_num_threads(os.cpu_count() or 1)
    E_, H_, T = cfg["embed"], cfg["heads"], cfg["T"]
    sub = dict(cfg, pairs=1)
    tokens, chain_ids = make_pairs(sub)
    layer = M.TransformerLayer_MINT(E_, 4 * E_, H_, use_multimer=True)
    layer.train(cfg["train"])
    pad = tokens.eq(1)
    mask = chain_ids.unsqueeze(-1) != chain_ids.unsqueeze(-2)

    def oracle_attention(q_s, k_s, v_s, q_c, k_c, v_c, *, chain_mask=None, key_padding_mask=None, rope=True, scale=None,
                         sqrt_softmax=False, out_seq_first=False, **kw):
        out = O.multimer_attention(q_s, k_s, v_s, q_c, k_c, v_c, chain_mask, key_padding_mask, scale=scale, rope=rope,
                                   sqrt_softmax=sqrt_softmax)
        return out.permute(2, 0, 1, 3).contiguous() if out_seq_first else out   # the reference's own permute copy

    saved = ops.multimer_attention
    ops.multimer_attention = oracle_attention
    try:
        x = torch.randn(T, 1, E_, requires_grad=cfg["train"])
        times = []
        t_end = time.perf_counter() + seconds_budget
        for it in range(4):
            t0 = time.perf_counter()
            with torch.set_grad_enabled(cfg["train"]):
                y, _ = layer(x, self_attn_mask=mask, self_attn_padding_mask=pad)
                if cfg["train"]:
                    y.square().mean().backward()
            dt = time.perf_counter() - t0
            if it > 0 or time.perf_counter() > t_end:
                times.append(dt)
            if time.perf_counter() > t_end:
                break
    finally:
        ops.multimer_attention = saved
    sec_layer_pair = statistics.median(times)
    sec_pair = sec_layer_pair * cfg["layers"]
    return {"value": 1.0 / sec_pair, "unit": "pairs/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"one layer on one pair (T={T}, E={E_}), fp32, {'fwd+bwd' if cfg['train'] else 'fwd'}: "
                      f"{sec_layer_pair:.2f} s (median of {len(times)}), extrapolated x{cfg['layers']} layers"}


def run_reference(name, args, rank):
    if rank != 0:
        return
    cfg = WORKLOADS[name]
    base = cpu_baseline(cfg, seconds_budget=min(60.0, 10.0 * max(1, args.steps)))
    line = {"impl": "reference", "metric": "ppi_pairs_per_sec", "value": base["value"], "unit": "pairs/s",
            "n_gpus": args.gpus, "steps": 1, "warmup": 1, "ms_per_step": 1e3 * cfg["pairs"] / base["value"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": cfg["desc"] + " per GPU", "device": "cpu"}, "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": "pairs/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def run(name, args, rank, world, local, ClockSampler, peaks, peak_src, steps=None, with_cpu_baseline=True):
    """Runs the workload on this rank; returns the JSON line (a dict) on rank 0 and None elsewhere."""
    import torch.distributed as dist
    from mint_plus_b200 import _lib as L, ops
    from mint_plus_b200.distributed import ChunkedGradAllReduce, FlatGradAllReduce, reduce_max, reduce_sum
    from mint_plus_b200.training import shared_step

    cfg = dict(WORKLOADS[name])
    if getattr(args, "layers", 0):
        cfg["layers"] = args.layers
        cfg["desc"] += f" [REDUCED to {args.layers} layers: profiling case, not a benchmark value]"
    dev = torch.device("cuda", local)
    steps, warmup = (steps or args.steps), max(args.warmup, 3)
    model = build_model(cfg, dev)
    tokens, chain_ids = make_pairs(cfg, rank, world)
    h_tok, h_cid = tokens.pin_memory(), chain_ids.pin_memory()
    h_lab = None
    flops_step, flops_gemm, flops_attn = algorithmic_flops(cfg, tokens)
    trainable = [p for p in model.parameters() if p.requires_grad] if cfg["train"] else []
    # one all-reduce (average) of the trainable gradients after the backward pass, on a flat buffer filled by one multi-tensor copy
    sync_grads = None
    if cfg["train"] and world > 1:
        gdt = torch.float32 if cfg["kind"] == "lora" else torch.bfloat16
        if os.environ.get("MINTB_GRAD_CHUNKS", "0") != "0":   # a few large chunks, each sent as the backward pass leaves its layers
            sync_grads = ChunkedGradAllReduce(model, n_chunks=int(os.environ["MINTB_GRAD_CHUNKS"]), dtype=gdt)
        else:
            sync_grads = FlatGradAllReduce(trainable, dtype=gdt)
    opt = scaler = None
    if cfg.get("optimizer") == "adamw":
        from mint_plus_b200 import Fp8WeightScaler
        opt = torch.optim.AdamW(trainable, lr=1e-5, weight_decay=0.01, fused=True)
        scaler = Fp8WeightScaler(model)
    lib = L.lib()
    loss_host = torch.zeros(1, dtype=torch.float32).pin_memory()
    out_host = None

    def step(tok, cid, lab):
        if cfg["train"]:
            for p in trainable:
                p.grad = None
            # the reference's training step: MLM corruption drawn on the device, forward, masked cross-entropy, backward
            loss, _ = shared_step(model, (tok, cid))
            loss.backward()
            if sync_grads is not None:
                sync_grads.finish() if isinstance(sync_grads, ChunkedGradAllReduce) else sync_grads()
            if opt is not None:
                opt.step()
                scaler.refresh()        # no host read: scales from the maxima measured one step earlier
            return loss.detach()
        with torch.no_grad():
            res = model(tok, cid, repr_layers=[cfg["layers"]])
            return res["representations"][cfg["layers"]]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    d_tok, d_cid = h_tok.to(dev), h_cid.to(dev)
    d_lab = h_lab.to(dev) if h_lab is not None else None
    for _ in range(warmup):
        step(d_tok, d_cid, d_lab)
    barrier()
    launches0 = lib.mintb_kernel_launches()
    step(d_tok, d_cid, d_lab)
    launches_per_step = lib.mintb_kernel_launches() - launches0
    barrier()

    # Launch mode.  A training step whose weights do not change between steps (no optimiser in the timed loop) is captured
    # once into a CUDA graph and replayed: the same kernels in the same order, launched by the host in one call.  With an
    # optimiser the FP8 scales change from step to step and reach the kernels by value, so that variant stays eager, as
    # does inference (a few hundred long kernels).  MINTB_BENCH_EAGER=1 forces eager launches.
    launch_mode = "eager"
    if cfg["train"] and opt is None and cfg.get("graph", True) and os.environ.get("MINTB_BENCH_EAGER", "0") == "0":
        from mint_plus_b200.training import GraphedTrainStep
        try:
            after = None
            if sync_grads is not None:
                after = sync_grads.finish if isinstance(sync_grads, ChunkedGradAllReduce) else sync_grads
            graphed = GraphedTrainStep(model, d_tok, d_cid, params=trainable, after_backward=after, warmup=1)
            eager_step = step

            def step(tok, cid, lab):        # noqa: F811 - same arguments as the eager step
                return graphed.step(tok, cid)
            launch_mode = "cuda graph (one captured step replayed)"
            for _ in range(2):
                step(d_tok, d_cid, d_lab)
            barrier()
        except Exception as exc:            # capture refused (an operation that is not capturable): stay eager, say why
            launch_mode = f"eager (graph capture failed: {type(exc).__name__}: {str(exc)[:120]})"
            torch.cuda.synchronize()

    sampler = ClockSampler(local)
    sampler.start()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    barrier()
    for s, e in ev:             # every step touches gigabytes of activations and weights: far more than the 126 MB L2
        s.record()
        step(d_tok, d_cid, d_lab)
        e.record()
    barrier()
    ms_total = sum(s.elapsed_time(e) for s, e in ev)

    # end to end: tokens, chain ids (and labels) from pinned host memory; loss / mean-pooled embedding back to the host
    e2e_steps = min(steps, 10)
    ev2 = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(e2e_steps)]
    h2d = h_tok.numel() * 8 + h_cid.numel() * 8 + (h_lab.numel() * 8 if h_lab is not None else 0)
    d2h = 4
    if not cfg["train"]:
        out_host = torch.empty(cfg["pairs"], cfg["embed"], dtype=torch.float32).pin_memory()
        d2h = out_host.numel() * 4
    barrier()
    for s, e in ev2:
        s.record()
        tok, cid = h_tok.to(dev, non_blocking=True), h_cid.to(dev, non_blocking=True)
        lab = h_lab.to(dev, non_blocking=True) if h_lab is not None else None
        r = step(tok, cid, lab)
        if cfg["train"]:
            loss_host.copy_(r.float().view(1), non_blocking=True)
        else:                                                       # embedding extraction: mean over unpadded positions
            keep = (tok != 1).unsqueeze(-1)
            out_host.copy_(((r.float() * keep).sum(1) / keep.sum(1)), non_blocking=True)
        e.record()
    barrier()
    e2e_ms = sum(s.elapsed_time(e) for s, e in ev2)
    clocks = sampler.finish()
    ops.check_device_status(dev)

    # the largest projection GEMM of the model in isolation (fc1: [pairs*T, E] x [4E, E]^T), for the roofline entry
    E_ = cfg["embed"]
    Mtok = cfg["pairs"] * cfg["T"]
    gemm = None
    if cfg["kind"] != "base_fp32":
        x = torch.randn(Mtok, E_, device=dev, dtype=torch.bfloat16)
        w = torch.randn(4 * E_, E_, device=dev, dtype=torch.bfloat16) / math.sqrt(E_)
        b = torch.zeros(4 * E_, device=dev, dtype=torch.bfloat16)
        if cfg["kind"] == "mu_fp8":
            xq, wq = ops.quantize_e4m3(x, 1.0), ops.quantize_e4m3(w, 1.0)
            fn = lambda: ops.gemm_e4m3(xq, wq, 1.0, b, True)
            peak, peak_name = peaks.get("fp8_tflops", 2.0 * peaks["bf16_tflops"]), "2 x measured bf16 peak (no measured e4m3 figure)"
            if "fp8_tflops" in peaks:
                peak_name = "measured e4m3 peak"
        else:
            fn = lambda: ops.gemm_bf16(x, w, b, True)
            peak, peak_name = peaks["bf16_tflops"], f"{peak_src} bf16 peak"
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        evs = []
        for _ in range(10):
            a, c = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); c.record()
            evs.append((a, c))
        torch.cuda.synchronize()
        g_ms = statistics.median(a.elapsed_time(c) for a, c in evs)
        g_tf = 2.0 * Mtok * E_ * 4 * E_ / (g_ms * 1e-3) / 1e12
        gemm = {"ms": g_ms, "tflops": g_tf, "peak": peak, "peak_name": peak_name}

    ms_total, e2e_ms = reduce_max([ms_total, e2e_ms], dev)
    pairs_total, flops_total = reduce_sum([cfg["pairs"], flops_step], dev)
    if rank == 0:
        value = pairs_total * steps / (ms_total * 1e-3)
        tf = flops_total * steps / (ms_total * 1e-3) / 1e12 / world            # per GPU
        roof = {"bound": "tensor", "kernel": "whole step (all kernels and library calls)", "achieved": tf,
                "peak": peaks["bf16_tflops_sustained"] if "bf16_tflops_sustained" in peaks else peaks["bf16_tflops"],
                "unit": "TFLOP/s", "traffic": None, "peak_source": peak_src + " (sustained bf16)",
                "flops_per_step": flops_step, "gemm_flops": flops_gemm, "attention_flops": flops_attn}
        roof["frac"] = roof["achieved"] / roof["peak"]
        if cfg["kind"] == "mu_fp8":
            # every projection product (forward, dgrad, wgrad) runs on 8-bit operands (twice the bf16 rate), the attention
            # on bf16: the time the step needs at those peaks is the blended bound
            f8 = flops_gemm
            t_min = (f8 / 2.0 + (flops_step - f8)) / (roof["peak"] * 1e12)
            roof["blended_peak"] = flops_step / t_min / 1e12
            roof["frac_blended"] = roof["achieved"] / roof["blended_peak"]
            roof["blended_note"] = "projection GEMM FLOPs (forward e4m3 x e4m3, backward e5m2 x e4m3) at 2 x the sustained bf16 peak, attention FLOPs at 1 x"
        if gemm is not None:
            roof["largest_gemm"] = {"shape": [Mtok, 4 * E_, E_], "epilogue": "bias + erf-GELU", **gemm,
                                    "frac": gemm["tflops"] / gemm["peak"]}
        line = {"metric": "ppi_pairs_per_sec", "value": value, "unit": "pairs/s", "n_gpus": world, "steps": steps,
                "warmup": warmup, "ms_per_step": ms_total / steps, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": cfg["dtype"], "data": "synthetic",
                "config": {"workload": cfg["desc"] + " per GPU", "l2": "working set per step far exceeds L2 (no flush)",
                           "launch": launch_mode, "checkpointing": ("per layer" if getattr(model, "last_forward_checkpointed", False) else
                                             "off (activations of all layers fit in HBM)") if cfg["train"] else "none",
                           "grad_allreduce_bytes": sync_grads.nbytes if sync_grads is not None else 0,
                           "dealing": "one seeded list of n_gpus x pairs, dealt to ranks in equal counts by squared length (snake order)"
                           if world > 1 else "single batch"},
                "roofline": roof,
                "e2e": {"value": pairs_total * e2e_steps / (e2e_ms * 1e-3), "unit": "pairs/s", "h2d_bytes_per_step": h2d,
                        "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / e2e_steps},
                "gpu_launches": int(launches_per_step * steps), "clocks": clocks}
        if world == 1 and with_cpu_baseline and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(cfg)
        return line
    return None
