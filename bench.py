#!/usr/bin/env python
"""Benchmark of the fused two-pathway multimer attention (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload: the isolated-op configuration — B=8 pairs, H=20, head_dim=32, T=1024, bf16, RoPE on the self
pathway, chain split uniform in [200,824], 0..64 trailing padded keys, seeded synthetic N(0,1)/sqrt(32) inputs.
A step is one forward + backward over one batch.  One process per GPU; each rank owns its own batch (pairs
shard, no data-path collective) so the scaling is weak.  Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = dict(B=8, H=20, T=1024, D=32)
METRIC = "fused_multimer_attention_fwd_bwd_tflops"
UNIT = "TFLOP/s"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
MIN_TIMED_SECONDS = 0.5      # the K-step sweep is repeated until at least this much device time has been measured
# DRAM bytes (read + write) of ONE launch of the backward kernel on this workload, from an ncu capture of that kernel
# (dram__bytes_read.sum + dram__bytes_write.sum = 124.1 MB + 45.5 MB).  A constant of the kernel, not of the run: it is
# reported beside the bytes computed from the tensor sizes and has to be refreshed when the kernel's data movement changes.
NCU_TRAFFIC_BYTES = 169.1e6


def algorithmic_flops(H, T, D, key_pad, fwd=True, bwd=True):
    """One logit and one P.V term per (query, unpadded key): fwd 4*H*T*Tk*D, bwd 2.5x that (recompute S, dP, dV,
    dQ, dK)."""
    tk = (~key_pad).sum(dim=1).double()          # per sample
    per = (4.0 if fwd else 0.0) + (10.0 if bwd else 0.0)
    return float((per * H * T * tk * D).sum())


def algorithmic_bytes(B, H, T, D):
    """HBM bytes the backward call has to move at least once (bf16 tensors): the six inputs, O and dO in, six gradients
    out, the log-sum-exp in, and the fp32 dQ accumulators of both pathways written and read back once."""
    elems = B * H * T * D
    return 14 * elems * 2 + B * H * T * 4 + 2 * 2 * elems * 4


def make_op_inputs(B, H, T, D, seed, max_pad=64):
    """Seeded inputs of the isolated-op configuration: six N(0,1)/sqrt(D) tensors, a chain split point per sample uniform
    in [200, 824] (scaled with T), 0..max_pad trailing padded positions, N(0,1) upstream gradient.  Draws the same numbers
    as the generator of the parity tests (a test compares the two)."""
    g = torch.Generator().manual_seed(seed)
    ts = [torch.randn(B, H, T, D, generator=g) / math.sqrt(D) for _ in range(6)]
    split = torch.randint(T * 200 // 1024, T * 824 // 1024 + 1, (B,), generator=g)
    pad = torch.randint(0, min(max_pad, max(T - int(split.max()) - 1, 0)) + 1, (B,), generator=g)
    chain_ids = torch.zeros(B, T, dtype=torch.int32)
    key_pad = torch.zeros(B, T, dtype=torch.bool)
    for b in range(B):
        chain_ids[b, int(split[b]):] = 1
        if int(pad[b]) > 0:
            key_pad[b, T - int(pad[b]):] = True
    grad = torch.randn(B, H, T, D, generator=g)
    return ts, chain_ids, key_pad, grad


def make_inputs(seed):
    return make_op_inputs(WORKLOAD["B"], WORKLOAD["H"], WORKLOAD["T"], WORKLOAD["D"], seed=seed)


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.stop_flag = index, [], threading.Event()
        self.proc = None

    def run(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            for line in self.proc.stdout:
                self.samples.append([x.strip() for x in line.split(",")])
                if self.stop_flag.is_set():
                    break
        except Exception:
            pass

    def finish(self):
        self.stop_flag.set()
        if self.proc is not None:
            self.proc.terminate()          # the exact child started above
        self.join(timeout=2)
        mhz, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                mhz.append(float(s[0]))
                mx = max(mx, float(s[1]))
                for n, v in zip(names, s[2:6]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except (ValueError, IndexError):
                continue
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(mhz)}


def time_shape(M, dev, flush, B, H, T, D, seed, iters):
    """Forward and forward+backward time of the attention op at another shape: chains of 100..900 positions per pair padded
    to T, inputs resident in HBM (larger than L2, which is flushed between iterations as well)."""
    g = torch.Generator().manual_seed(seed)
    ts = [(torch.randn(B, H, T, D, generator=g) / math.sqrt(D)).bfloat16().to(dev) for _ in range(6)]
    la = torch.randint(100, 901, (B,), generator=g)
    lb = torch.randint(100, 901, (B,), generator=g)
    cid = torch.zeros(B, T, dtype=torch.int32)
    pad = torch.zeros(B, T, dtype=torch.bool)
    for b in range(B):
        cid[b, int(la[b]):] = 1
        pad[b, int(la[b]) + int(lb[b]):] = True
    grad = torch.randn(B, H, T, D, generator=g).bfloat16().to(dev)
    meta = M.mask_meta_from_chain_ids(cid.to(dev), pad.to(dev))

    def fwd():
        with torch.no_grad():
            return M.multimer_attention(*ts, meta=meta)

    def step():
        leaves = [t.requires_grad_(True) for t in ts]
        return torch.autograd.grad(M.multimer_attention(*leaves, meta=meta), leaves, grad)

    res = {}
    for name, fn in (("fwd", fwd), ("step", step)):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        evs = []
        for _ in range(iters):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record()
            evs.append((a, b))
        torch.cuda.synchronize()
        res[name] = statistics.median(a.elapsed_time(b) for a, b in evs)
    f_fwd = algorithmic_flops(H, T, D, pad, bwd=False)
    f_all = algorithmic_flops(H, T, D, pad)
    return {"shape": {"B": B, "H": H, "T": T, "D": D, "chains": "100..900 residues each, padded to T"},
            "fwd_ms": res["fwd"], "fwd_bwd_ms": res["step"], "fwd_tflops": f_fwd / (res["fwd"] * 1e-3) / 1e12,
            "fwd_bwd_tflops": f_all / (res["step"] * 1e-3) / 1e12, "launch": "eager", "iters": iters}


def cpu_baseline(seconds_budget=20.0):
    """The oracle (a port of the reference's PyTorch path) on the host cores, on a bounded sample: a few steps of the
    same batch (8 pairs), fp32, forward + autograd backward."""
    from oracle import multimer_attention as O
    torch.set_num_threads(os.cpu_count() or 1)
    ts, cid, pad, grad = make_inputs(2002)
    mask = O.chain_mask_from_ids(cid)
    flops = algorithmic_flops(WORKLOAD["H"], WORKLOAD["T"], WORKLOAD["D"], pad)
    times = []
    t_end = time.perf_counter() + seconds_budget
    for it in range(4):
        t0 = time.perf_counter()
        O.multimer_attention_fwd_bwd(*ts, mask, grad, key_pad=pad)
        dt = time.perf_counter() - t0
        if it > 0:
            times.append(dt)
        if time.perf_counter() > t_end and times:
            break
    sec = statistics.median(times)
    return {"value": flops / sec / 1e12, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"the benchmark batch (B=8,H=20,T=1024,D=32), fp32, fwd+autograd bwd, "
                      f"median of {len(times)} steps after 1 warm-up, {sec:.2f} s each"}, sec


def load_peaks():
    """Roofline denominators: the measured figures file if present, else the stated fallback."""
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        with open(peaks_path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def run_reference(args, rank, world):
    """The reference's CPU implementation of the path (oracle port; the reference itself is Python + Triton and its
    checkout is not on the GPU box), timed on the host cores with every thread."""
    if rank != 0:
        return
    from oracle import multimer_attention as O
    torch.set_num_threads(os.cpu_count() or 1)
    ts, cid, pad, grad = make_inputs(2002)
    mask = O.chain_mask_from_ids(cid)
    flops = algorithmic_flops(WORKLOAD["H"], WORKLOAD["T"], WORKLOAD["D"], pad)
    steps = max(1, min(args.steps, 5))
    warm = max(1, min(args.warmup, 1))
    for _ in range(warm):
        O.multimer_attention_fwd_bwd(*ts, mask, grad, key_pad=pad)
    t0 = time.perf_counter()
    for _ in range(steps):
        O.multimer_attention_fwd_bwd(*ts, mask, grad, key_pad=pad)
    sec = (time.perf_counter() - t0) / steps
    val = flops / sec / 1e12
    sample = (f"each step = the benchmark batch (B=8,H=20,T=1024,D=32), fp32, fwd + autograd bwd; "
              f"{steps} steps after {warm} warm-up (bounded from the requested {args.steps}/{args.warmup})")
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
            "warmup": warm, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "isolated combined-softmax multimer attention fwd+bwd, B=8 H=20 D=32 T=1024 per GPU",
                       "device": "cpu"},
            "cpu_baseline": {"value": val, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                             "sample": sample},
            "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="attn",
                    help="attn (default: the isolated attention op) or a whole-model workload of bench_model.py: "
                         "mint650m_fp8, mint650m_fp8_optim, mint150m_lora, mint3b_infer, mint8m_fwd, mint650m_fp8_packed, mint3b_infer_packed")
    ap.add_argument("--no-model-metric", action="store_true",
                    help="attn workload: skip the model-level measurements that are added to the line as `model_650m`, "
                         "`model_650m_optim`, `model_150m_lora` and `model_3b_infer`")
    ap.add_argument("--layers", type=int, default=0,
                    help="whole-model workloads only: run this many layers instead of the configuration's (a smaller case for "
                         "profiler captures; the line is then not a benchmark value and says so)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.workload != "attn":
        import bench_model
        if args.workload not in bench_model.WORKLOADS:
            raise SystemExit(f"unknown workload {args.workload!r}; choose attn or one of {sorted(bench_model.WORKLOADS)}")
        if args.impl == "reference":
            bench_model.run_reference(args.workload, args, rank)
            return
        import torch.distributed as dist
        torch.cuda.set_device(local)
        if world > 1:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        peaks, peak_src = load_peaks()
        line = bench_model.run(args.workload, args, rank, world, local, ClockSampler, peaks, peak_src)
        if line is not None:
            print(json.dumps(line), flush=True)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch.distributed as dist
    import mint_plus_b200 as M
    from mint_plus_b200 import _lib as L, ops

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    steps, warmup = args.steps, max(args.warmup, 3)
    B, H, T, D = (WORKLOAD[k] for k in "BHTD")

    ts, cid, pad, grad = make_inputs(2002 + rank)               # each rank owns its own pairs
    flops_step = algorithmic_flops(H, T, D, pad)
    flops_fwd = algorithmic_flops(H, T, D, pad, bwd=False)
    flops_bwd = algorithmic_flops(H, T, D, pad, fwd=False)
    host = [t.bfloat16().pin_memory() for t in ts] + [grad.bfloat16().pin_memory()]
    host_cid, host_pad = cid.pin_memory(), pad.pin_memory()
    dts = [t.to(dev, non_blocking=True) for t in host[:6]]
    dgrad = host[6].to(dev)
    meta = M.mask_meta_from_chain_ids(host_cid.to(dev), host_pad.to(dev))
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)   # > 126 MB L2

    def step_resident():
        leaves = [t.requires_grad_(True) for t in dts]
        out = M.multimer_attention(*leaves, meta=meta)
        return torch.autograd.grad(out, leaves, dgrad)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    lib = L.lib()
    for _ in range(warmup):
        step_resident()
    barrier()

    # The step is launch-bound on the host (nine small launches around two ~100-300 us kernels), so the timed loop
    # replays a CUDA graph of one forward (+ backward) captured through the same public API.
    def capture(fn):
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()                                     # warm the allocator on the capture stream
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        with torch.cuda.graph(g):
            keep = fn()
        return g, keep

    def fwd_only():
        with torch.no_grad():
            return M.multimer_attention(*[t.detach() for t in dts], meta=meta)

    use_graph = True
    try:
        g_step, _k1 = capture(step_resident)
        g_fwd, _k2 = capture(fwd_only)
        run_step, run_fwd = g_step.replay, g_fwd.replay
        launches0 = lib.mintb_kernel_launches()
        step_resident()
        launches_per_step = lib.mintb_kernel_launches() - launches0
    except Exception as exc:                          # capture not possible: time the eager launches
        use_graph = False
        sys.stderr.write(f"bench: CUDA graph capture failed ({exc}); timing eager launches\n")
        run_step, run_fwd = step_resident, fwd_only
        launches0 = lib.mintb_kernel_launches()
        step_resident()
        launches_per_step = lib.mintb_kernel_launches() - launches0
    for _ in range(3):
        run_step()
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    # ---- device-resident inputs: sweeps of K steps, each step bracketed by its own events, L2 flushed between steps.
    # One sweep of this workload lasts a few milliseconds, so the sweep is repeated until MIN_TIMED_SECONDS of device time
    # have been measured; the line reports the MEDIAN sweep (exactly K steps).
    sweep_ms = []
    barrier()
    while True:
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        for s, e in ev:
            flush.zero_()
            s.record()
            run_step()
            e.record()
        torch.cuda.synchronize()
        sweep_ms.append(sum(s.elapsed_time(e) for s, e in ev))
        more = torch.tensor([1.0 if sum(sweep_ms) < MIN_TIMED_SECONDS * 1e3 and len(sweep_ms) < 2000 else 0.0], device=dev)
        if world > 1:
            dist.all_reduce(more, op=dist.ReduceOp.MAX)        # every rank runs the same number of sweeps
        if more.item() == 0.0:
            break
    barrier()
    n_sweeps = len(sweep_ms)
    launches = launches_per_step * steps
    ms_total = statistics.median(sweep_ms)

    # ---- the forward call alone (same method); the backward call is the difference
    fwd_ms = []
    for _ in range(100):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        run_fwd()
        b.record()
        torch.cuda.synchronize()
        fwd_ms.append(a.elapsed_time(b))
    bwd_ms = [ms_total / steps - statistics.mean(fwd_ms)]

    # ---- end to end: pinned host inputs -> device, fwd+bwd through the public API, results -> pinned host
    out_host = [torch.empty(B, H, T, D, dtype=torch.bfloat16).pin_memory() for _ in range(7)]
    h2d = sum(t.numel() * t.element_size() for t in host) + host_cid.numel() * 4 + host_pad.numel()
    d2h = sum(t.numel() * t.element_size() for t in out_host)

    # Three streams, so that the copy engines and the SMs work at the same time: step i's inputs are copied in while step
    # i-1 computes and step i-2's results are copied out.  Every step still moves all of its inputs and results.
    NBUF = 3
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    s_main = torch.cuda.current_stream()
    in_bufs = [[torch.empty(B, H, T, D, dtype=torch.bfloat16, device=dev) for _ in range(7)] for _ in range(NBUF)]
    id_bufs = [(torch.empty_like(host_cid, device=dev), torch.empty_like(host_pad, device=dev)) for _ in range(NBUF)]
    res_bufs = [None] * NBUF
    ev_in = [torch.cuda.Event() for _ in range(NBUF)]
    ev_done = [torch.cuda.Event() for _ in range(NBUF)]
    ev_out = [torch.cuda.Event() for _ in range(NBUF)]
    out_hosts = [out_host] + [[torch.empty_like(t).pin_memory() for t in out_host] for _ in range(NBUF - 1)]

    def step_e2e(i):
        k = i % NBUF
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_done[k])                       # the step that last used these device buffers has computed
            for dst, src in zip(in_bufs[k], host):
                dst.copy_(src, non_blocking=True)
            id_bufs[k][0].copy_(host_cid, non_blocking=True)
            id_bufs[k][1].copy_(host_pad, non_blocking=True)
            ev_in[k].record(s_in)
        s_main.wait_event(ev_in[k])
        s_main.wait_event(ev_out[k])                          # its previous results have left the device
        d = [t.detach().requires_grad_(True) for t in in_bufs[k][:6]]
        o = M.multimer_attention(*d, chain_ids=id_bufs[k][0], key_padding_mask=id_bufs[k][1])
        grads = torch.autograd.grad(o, d, in_bufs[k][6])
        res_bufs[k] = (o.detach(), *grads)
        ev_done[k].record(s_main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_done[k])
            for dst, src in zip(out_hosts[k], res_bufs[k]):
                dst.copy_(src, non_blocking=True)
            ev_out[k].record(s_out)

    def drain_e2e():
        s_main.wait_stream(s_in)
        s_main.wait_stream(s_out)

    for i in range(3):
        step_e2e(i)
    drain_e2e()
    barrier()
    def time_e2e(n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        flush.zero_()
        e0.record()
        for i in range(n):
            step_e2e(i)
        drain_e2e()
        e1.record()
        barrier()
        return e0.elapsed_time(e1)

    # a short run sizes the timed one so that it lasts at least MIN_TIMED_SECONDS (the same count on every rank)
    est = torch.tensor([time_e2e(10) / 10], device=dev)
    if world > 1:
        dist.all_reduce(est, op=dist.ReduceOp.MIN)
    e2e_steps = int(min(4000, max(steps, MIN_TIMED_SECONDS * 1e3 / max(est.item(), 1e-3) + 1)))
    e2e_ms = time_e2e(e2e_steps)
    clocks = sampler.finish()
    ops.check_device_status(dev)

    # ---- the attention shape of the MINT-650M workload (H=20, D=64, T=2048; 8 pairs with chains of 100..900 residues),
    # timed the same way on rank 0's GPU (eager launches: its kernels last a millisecond), for a second roofline entry
    d64 = None
    if rank == 0:
        d64 = time_shape(M, dev, flush, B=8, H=20, T=2048, D=64, seed=4004, iters=30)

    # max over ranks of the timed totals; whole-job work = every rank's flops
    stats = torch.tensor([ms_total, e2e_ms], dtype=torch.float64, device=dev)
    work = torch.tensor([flops_step], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(work, op=dist.ReduceOp.SUM)
    ms_total, e2e_ms = stats.tolist()
    total_flops_step = float(work.item())

    # The model-level metrics, measured in the same run and attached to the line: PPI pairs/s of the MINT-650M FP8
    # forward+backward step (the second headline metric), of the MINT-150M LoRA training step and of the 36 x 2560
    # inference forward (short runs of those workloads of bench_model.py; every rank takes part).
    model_lines = {}
    if not args.no_model_metric:
        import bench_model
        del dts, dgrad, in_bufs, res_bufs, flush
        torch.cuda.empty_cache()
        peaks_m, peak_src_m = load_peaks()
        for key, workload, k_steps in (("model_650m", "mint650m_fp8", max(2, min(steps, 4))),
                                       ("model_650m_optim", "mint650m_fp8_optim", max(2, min(steps, 4))),
                                       ("model_150m_lora", "mint150m_lora", max(2, min(steps, 4))),
                                       ("model_3b_infer", "mint3b_infer", 2)):
            try:
                model_lines[key] = bench_model.run(workload, args, rank, world, local, ClockSampler, peaks_m, peak_src_m,
                                                   steps=k_steps, with_cpu_baseline=False)
            except Exception as exc:                   # the attention line must not be lost with it
                if world > 1:
                    raise                              # ranks would fall out of step: let the launcher see the failure
                sys.stderr.write(f"bench: the {workload} measurement failed: {exc!r}\n")
                model_lines[key] = {"error": repr(exc)}
            torch.cuda.empty_cache()
    if rank == 0:
        peaks, peak_src = load_peaks()
        value = total_flops_step * steps / (ms_total * 1e-3) / 1e12
        fwd_t, bwd_t = statistics.mean(fwd_ms), statistics.mean(bwd_ms)
        dom = ("attention backward call", flops_bwd, bwd_t) if bwd_t >= fwd_t else ("attention forward call", flops_fwd, fwd_t)
        achieved = dom[1] / (dom[2] * 1e-3) / 1e12
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": ms_total / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "isolated combined-softmax multimer attention fwd+bwd, B=8 H=20 D=32 T=1024 per GPU",
                       "rope": "self pathway", "l2": "flushed between timed steps (256 MiB write)",
                       "launch": "CUDA graph replay of one step" if use_graph else "eager launches",
                       "flops": "14*H*T*Tk*D per pair, Tk = unpadded keys",
                       "sweeps": f"{n_sweeps} sweeps of {steps} steps timed ({sum(sweep_ms) * 1e-3:.2f} s of device time); "
                                 "value and ms_per_step are the median sweep",
                       "e2e": "host->device copies, compute and device->host copies of consecutive steps overlap on three "
                              "streams; every step moves all of its inputs and results"},
            "roofline": {"bound": "tensor", "kernel": dom[0], "achieved": achieved, "peak": peaks["bf16_tflops"],
                         "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops"], "traffic": NCU_TRAFFIC_BYTES,
                         "traffic_source": "ncu capture of one launch of the backward kernel at this workload (constant)",
                         "algorithmic_bytes": algorithmic_bytes(B, H, T, D),
                         "peak_source": peak_src, "fwd_ms": fwd_t, "bwd_ms": bwd_t,
                         "fwd_tflops": flops_fwd / (fwd_t * 1e-3) / 1e12, "bwd_tflops": flops_bwd / (bwd_t * 1e-3) / 1e12},
            "roofline_d64_t2048": None if d64 is None else {
                "bound": "tensor", "kernel": "attention forward + backward calls", "achieved": d64["fwd_bwd_tflops"],
                "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": d64["fwd_bwd_tflops"] / peaks["bf16_tflops"],
                "traffic": None, "peak_source": peak_src, **d64},
            "e2e": {"value": total_flops_step * e2e_steps / (e2e_ms * 1e-3) / 1e12, "unit": UNIT,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / e2e_steps},
            "gpu_launches": int(launches),
            "clocks": clocks,
        }
        for key, ml in model_lines.items():
            if ml is not None:
                line[key] = {k: ml[k] for k in ("metric", "value", "unit", "ms_per_step", "steps", "dtype", "config",
                                                "roofline", "e2e", "gpu_launches", "error") if k in ml}
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"], _ = cpu_baseline()
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
