#!/usr/bin/env python
"""MoE-layer throughput benchmark.

A step is one pass of the MoE layer over one batch of synthetic tokens. At one GPU the workload
is the gpt-oss-20b-shaped layer (32 MXFP4 experts, top-4, hidden = ffn = 2880) at a prefill of
2048 tokens; with N GPUs every rank runs that layer on its own 2048 tokens (experts are small
enough to replicate, no exchange on the data path: weak scaling).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--tokens T]
    python bench.py --impl reference ...        # the CPU arm: the C++ restatement on the host cores

One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from oco_b200 import synth  # noqa: E402

METRIC = "MoE-layer tokens/s at gpt-oss-20b shape; % of HBM / FP4 tensor roofline"
WORKLOADS = {
    # name: (config, default tokens)
    "gpt-oss-20b-prefill": ("gpt-oss-20b", 2048),
    "gpt-oss-20b-decode": ("gpt-oss-20b", 1),
    "qwen3-30b-a3b-prefill": ("qwen3-30b-a3b", 512),
    "nemotron-h-prefill": ("nemotron-h", 1024),
    "nemotron-h-decode": ("nemotron-h", 1),
    "qwen3-30b-a3b-decode": ("qwen3-30b-a3b", 1),
    # 128 experts: one GPU holds them all; with N > 1 ranks the experts are sharded 128/N per GPU and
    # the batch (fixed in total: strong scaling) is dispatched and combined with all-to-all
    "gpt-oss-120b-prefill": ("gpt-oss-120b", 8192),
    "gpt-oss-120b-decode64": ("gpt-oss-120b", 64),
}
EXPERT_PARALLEL = {"gpt-oss-120b-prefill", "gpt-oss-120b-decode64"}
# DRAM bytes (read + write) of one launch of the dominant kernels, from the ncu captures that are
# summarised under profiles/ (grouped_gemm_wide_gpt-oss-20b-prefill.md,
# grouped_gemm_wide_qwen3-30b-a3b-prefill.md, token_kernels_gpt-oss-20b-decode.md); a profiler is
# never attached to a timed run.
NCU_TRAFFIC = {
    ("gpt-oss-20b-prefill", "up_tiles"): 334.5e6 + 38.7e6,
    ("gpt-oss-20b-prefill", "down_tiles"): 190.6e6 + 28.9e6,
    ("qwen3-30b-a3b-prefill", "up_tiles"): 243.4e6 + 7.2e6,
    ("qwen3-30b-a3b-prefill", "down_tiles"): 119.6e6 + 8.1e6,
    ("gpt-oss-20b-decode", "expand"): 35.39e6,
    ("gpt-oss-20b-decode", "down_combine"): 17.76e6,
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=p["hbm_gbs"], tflops=p["bf16_tflops"], tflops_sustained=p.get("bf16_tflops_sustained"),
                    source="measured")
    return dict(hbm_gbs=6650.0, tflops=1590.0, tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
                for name, val in zip(names, r[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            except (ValueError, IndexError):
                continue
        # samples under load: the upper half of the observed clocks
        sm_sorted = sorted(sm)
        load = sm_sorted[len(sm_sorted) // 2:] if sm_sorted else []
        return dict(sm_mhz=float(np.median(load)) if load else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


def algorithmic(layer: synth.Layer, tokens: int, ids: np.ndarray):
    """Algorithmic bytes and FLOPs of one step: every touched expert's packed weights and biases
    once, the router once, the input rows in and the residual rows in and out."""
    touched = len(np.unique(ids))
    io = tokens * layer.hidden * 2 * 3
    total_bytes = touched * layer.expert_bytes() + layer.shared_bytes() + layer.router_bytes() + io
    return total_bytes, layer.flops(tokens), touched


def cpu_baseline(layer, tokens, seed, budget_tokens, threads=None):
    """Times the CPU restatement (f32 FMA accumulation, all host threads) on a bounded sample of
    the same workload: the first `budget_tokens` tokens of the batch."""
    import oracle
    # all the cores this process may use, whatever OMP_NUM_THREADS says (torchrun sets it to 1)
    oracle.set_num_threads(threads or len(os.sched_getaffinity(0)))
    n = max(1, min(tokens, budget_tokens))
    x, res = synth.make_tokens(layer.hidden, tokens, seed, "normal")
    x, res = x[:n], res[:n]
    mode = 1 if tokens == 1 else 2
    oracle.moe_forward(layer, x[:1], res[:1], mode=mode, accumulate_f32=True, trace=False)  # page in
    t0 = time.perf_counter()
    oracle.moe_forward(layer, x, res, mode=mode, accumulate_f32=True, trace=False)
    dt = time.perf_counter() - t0
    return dict(value=n / dt, unit="tokens/s", cores=oracle.num_threads(), kind="port",
                sample=f"first {n} of {tokens} tokens, one pass, {dt:.2f} s wall clock; C++ restatement of the "
                       f"reference's Metal path (the reference is Metal-only and cannot run on this host)"), dt


def run_reference(args):
    """CPU arm: the reference's MoE arithmetic restated in C++ (oracle/), timed on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    cfg, default_tokens = WORKLOADS[args.workload]
    tokens = args.tokens or default_tokens
    layer = synth.make_config(cfg, seed=args.seed)
    sample = min(tokens, args.cpu_tokens)
    times = []
    base = None
    for i in range(args.warmup + args.steps):
        base, dt = cpu_baseline(layer, tokens, args.seed + i, sample)
        if i >= args.warmup:
            times.append(dt)
    ms = 1e3 * float(np.mean(times))
    value = sample / (ms / 1e3)
    base["value"] = value
    line = dict(metric=METRIC, impl="reference", value=value, unit="tokens/s", n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=ms, higher_is_better=True, scaling="weak", vs_baseline=None,
                dtype="f32", data="synthetic",
                config=dict(workload=args.workload, tokens_per_step=sample, full_batch=tokens,
                            note="each step is a bounded sample of the batch on the host cores"),
                cpu_baseline=base, e2e=dict(value=value, unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line))
    return 0


class _Recorded:
    """all_to_all_single that keeps what each call received, so that a later pass can replay the
    same step with device-local copies in place of the exchange."""

    def __init__(self, dist):
        self.dist, self.log = dist, []

    def __call__(self, out, inp, out_split=None, in_split=None, group=None):
        self.dist.all_to_all_single(out, inp, out_split, in_split, group=group)
        self.log.append(out.clone())


class _Replayed:
    def __init__(self, log):
        self.log, self.i = log, 0

    def __call__(self, out, inp, out_split=None, in_split=None, group=None):
        out.copy_(self.log[self.i % len(self.log)])
        self.i += 1


def run_expert_parallel(args, torch, dist, world, rank, local):
    """Experts sharded over the ranks, the batch split evenly between them (its total is fixed as N
    grows), dispatch and combine as all-to-all over NCCL."""
    from oco_b200 import ep
    cfg, default_tokens = WORKLOADS[args.workload]
    total = args.tokens or default_tokens
    if total % world:
        raise SystemExit(f"{total} tokens do not divide over {world} ranks")
    T = total // world
    layer = synth.make_config(cfg, seed=args.seed)
    E, K, H, F = layer.experts, layer.top_k, layer.hidden, layer.ffn
    be = ep.CudaBackend(layer, rank, world, max_rows=T)
    backend = be.backend()
    x_bits, res_bits = synth.make_tokens(H, total, args.seed, "normal")
    x_bits, res_bits = x_bits[rank * T:(rank + 1) * T], res_bits[rank * T:(rank + 1) * T]
    hx = torch.from_numpy(x_bits.view(np.int16).copy()).pin_memory()
    hres = torch.from_numpy(res_bits.view(np.int16).copy()).pin_memory()
    x, res = hx.cuda(), hres.cuda()
    stream = torch.cuda.current_stream()

    def timed(n, exchange=None):
        dist.barrier(); torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        launches = 0
        for _ in range(n):
            ep.forward(x, res, backend, E, exchange=exchange, uniform=True)
            launches += be.launches()
        b.record(stream)
        torch.cuda.synchronize(); dist.barrier()
        t = torch.tensor([a.elapsed_time(b) / n], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), launches

    for _ in range(max(3, args.warmup)):
        ep.forward(x, res, backend, E, uniform=True)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start(); time.sleep(0.3)
    ms_per_step, launches = timed(args.steps)
    clocks = sampler.stop() if rank == 0 else {}
    be.router_plan.poll(); be.expert_plan.poll()
    # the same step with the exchange replaced by device-local copies of what it delivered
    rec = _Recorded(dist)
    ep.forward(x, res, backend, E, exchange=rec)
    ms_local, _ = timed(args.steps, exchange=_Replayed(rec.log))
    # per-stage times of single steps
    tm, acc = {}, {}
    be.expert_plan.set_profiling(True)
    for _ in range(min(5, args.steps)):
        ep.forward(x, res, backend, E, timings=tm, uniform=True)
        for k, v in tm.items():
            acc.setdefault(k, []).append(v)
        for k, v in be.expert_plan.phase_times().items():
            acc.setdefault(k, []).append(v)
    be.expert_plan.set_profiling(False)
    phases = {k: float(np.mean(v)) for k, v in acc.items()}
    routes_here = int(phases.pop("routes_received"))
    # end to end: pinned host rows in, the layer, residual rows back
    e2e_steps = max(3, min(args.steps, 10))
    dist.barrier(); torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        x.copy_(hx, non_blocking=True); res.copy_(hres, non_blocking=True)
        ep.forward(x, res, backend, E, uniform=True)
        hres.copy_(res, non_blocking=True)
        torch.cuda.synchronize()
    t = torch.tensor([1e3 * (time.perf_counter() - t0) / e2e_steps], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item())
    if rank != 0:
        dist.destroy_process_group()
        return 0
    peaks = measured_peaks()
    row_bytes = T * H * 2
    e2e = dict(value=total / (e2e_ms / 1e3), unit="tokens/s", ms_per_step=e2e_ms, h2d_bytes_per_step=2 * row_bytes,
               d2h_bytes_per_step=row_bytes, api="oco_b200.ep.forward (pinned host rows in, residual rows back), per rank")
    roofline = None
    if "up_tiles" in phases:
        flops = 2.0 * routes_here * 2 * F * H
        ach = flops / (phases["up_tiles"] / 1e3) / 1e12
        roofline = dict(bound="tensor", kernel="up_tiles", achieved=ach, peak=peaks["tflops"], unit="TFLOP/s",
                        frac=ach / peaks["tflops"], traffic=None, peak_source=f"{peaks['source']} dense bf16 cuBLAS, burst",
                        algorithmic_flops_per_launch=flops, launch_ms=phases["up_tiles"], routes_on_rank0=routes_here)
    base = None
    if not args.no_cpu_baseline:
        base, _ = cpu_baseline(layer, total, args.seed, args.cpu_tokens)
    line = dict(
        metric=METRIC, value=total / (ms_per_step / 1e3), unit="tokens/s", n_gpus=world, steps=args.steps,
        warmup=args.warmup, ms_per_step=ms_per_step, higher_is_better=True, scaling="strong", vs_baseline=None,
        dtype="f16", data="synthetic",
        config=dict(workload=args.workload, tokens_total=total, tokens_per_gpu=T, hidden=H, ffn=F, experts=E, top_k=K,
                    weight_format="MXFP4", experts_per_gpu=E // world, parallelism=f"ep{world}",
                    cache="every step reads the rank's whole expert shard (%.0f MB), more than the 126 MB L2"
                          % (E // world * layer.expert_bytes() / 1e6)),
        all_to_all=dict(exposed_ms=ms_per_step - ms_local, ms_per_step_with_local_copies=ms_local,
                        dispatch_ms=phases.get("dispatch_ms"), combine_ms=phases.get("combine_a2a_ms"),
                        route_bytes_each_way_per_gpu=T * K * H * 2),
        clocks=clocks, e2e=e2e, gpu_launches=launches, phases_ms=phases, roofline=roofline, cpu_baseline=base)
    print(json.dumps(line))
    dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gpt-oss-20b-prefill", choices=sorted(WORKLOADS))
    ap.add_argument("--tokens", type=int, default=0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--cpu-tokens", type=int, default=32, help="tokens in the CPU baseline's bounded sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="single-token workloads: launch kernels directly instead of replaying CUDA graphs")
    ap.add_argument("--layers", type=int, default=0, help="distinct weight copies rotated per step (0 = auto)")
    ap.add_argument("--with-norm", action="store_true",
                    help="time the fused entry point: residual add + RMS norm + layer (the step either side of the layer)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist
    from oco_b200 import build, moe
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU path for this library")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if rank == 0:
        build.build()
    if world > 1:
        dist.barrier()

    if world > 1 and args.workload in EXPERT_PARALLEL:
        return run_expert_parallel(args, torch, dist, world, rank, local)

    cfg, default_tokens = WORKLOADS[args.workload]
    tokens = args.tokens or default_tokens
    layer = synth.make_config(cfg, seed=args.seed)
    decode = tokens == 1
    # Cold-cache protocol. Prefill reads every expert (hundreds of MB, more than the 126 MB L2) each
    # step, so the inputs themselves exceed L2. A single token touches only top_k experts (tens of
    # MB), so distinct weight copies are rotated step by step and never revisited within L2 reach.
    per_step_bytes = layer.top_k * layer.expert_bytes() if decode else layer.experts * layer.expert_bytes()
    copies = args.layers or (max(2, int(np.ceil(600e6 / per_step_bytes))) if decode else 1)
    weights = [moe._Weights.from_layer(layer) for _ in range(copies)]
    plans = []
    for w in weights:
        p = moe.plan_for(layer)
        p.reserve(tokens)
        p.bind(w)
        plans.append(p)
    x_bits, res_bits = synth.make_tokens(layer.hidden, tokens, args.seed + 1000 * rank, "normal")
    x = torch.from_numpy(x_bits.view(np.int16)).cuda()
    res = torch.from_numpy(res_bits.view(np.int16).copy()).cuda()
    stream = torch.cuda.current_stream()
    norm_w = torch.ones(layer.hidden, dtype=torch.float32, device="cuda")

    graphs = [None] * copies

    def step(i, profile=False):
        p = plans[i % copies]
        if graphs[i % copies] is not None and not profile:
            graphs[i % copies].replay()       # launch-bound single-token step: one graph launch
            return p
        p.set_profiling(profile)
        if args.with_norm:
            p.add_norm_forward(res, x, norm_w, 1e-5, layer.arch == synth.ARCH_GPT_OSS, tokens)   # x stands in for the mixer's output
        else:
            p.forward(x, res, tokens)
        return p

    for i in range(max(args.warmup, copies if decode else 0)):
        step(i)
    torch.cuda.synchronize()
    plans[0].poll()
    if decode and not args.no_graph:
        # A single token is a handful of microsecond kernels: capture each weight copy's step in a
        # CUDA graph so the timed region measures the GPU, not the host's launch rate.
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for c in range(copies):
                plans[c].set_profiling(False)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    step_plain = plans[c].add_norm_forward(res, x, norm_w, 1e-5, layer.arch == synth.ARCH_GPT_OSS, tokens) \
                        if args.with_norm else plans[c].forward(x, res, tokens)
                graphs[c] = g
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
    # routing of this batch (for the algorithmic byte count)
    routing = moe.Routing(); routing.plan, routing.rows = plans[(args.warmup - 1) % copies if args.warmup else 0], tokens
    if not args.warmup:
        step(0); torch.cuda.synchronize()
    ids = routing.read()["ids"]
    alg_bytes, alg_flops, touched = algorithmic(layer, tokens, ids)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    phase_acc = {}
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    launches = 0
    t_wall = time.perf_counter()
    for i in range(args.steps):
        starts[i].record(stream)
        p = step(args.warmup + i, profile=graphs[0] is None)
        ends[i].record(stream)
        launches += p.launch_count()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    wall = time.perf_counter() - t_wall
    # Per-kernel durations: the phase events of a plan hold its last call, so a few more steps are
    # run one at a time and read back (same kernels, same inputs, still rotating weight copies).
    for i in range(min(10, args.steps)):
        p = step(args.warmup + args.steps + i, profile=True)
        torch.cuda.synchronize()
        for k, v in p.phase_times().items():
            phase_acc.setdefault(k, []).append(v)
    clocks = sampler.stop() if rank == 0 else {}
    step_ms = [s.elapsed_time(e) for s, e in zip(starts, ends)]
    total_ms = starts[0].elapsed_time(ends[-1])
    ms_per_step = total_ms / args.steps
    if world > 1:
        t = torch.tensor([ms_per_step], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_per_step = float(t.item())
    plans[0].poll()
    value = world * tokens / (ms_per_step / 1e3)

    # ---- end to end through the host-buffer entry point -----------------------------------------
    hx = torch.from_numpy(x_bits.view(np.int16)).pin_memory()
    hres = torch.from_numpy(res_bits.view(np.int16).copy()).pin_memory()
    hx_np, hres_np = hx.numpy().view(np.uint16), hres.numpy().view(np.uint16)
    e2e_steps = max(3, min(args.steps, 20))
    for i in range(2):
        plans[i % copies].set_profiling(False)
        plans[i % copies].forward_host(hx_np, hres_np, tokens)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        plans[i % copies].forward_host(hx_np, hres_np, tokens)   # H2D x + residual, layer, D2H residual, stream sync
    e2e_ms = 1e3 * (time.perf_counter() - t0) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    row_bytes = tokens * layer.hidden * 2
    e2e = dict(value=world * tokens / (e2e_ms / 1e3), unit="tokens/s", ms_per_step=e2e_ms,
               h2d_bytes_per_step=2 * row_bytes, d2h_bytes_per_step=row_bytes,
               api="oco_moe_forward_host (pinned host buffers in, residual rows back)")

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return 0

    # ---- roofline of the dominant kernel ---------------------------------------------------------
    peaks = measured_peaks()
    phases = {k: float(np.mean(v)) for k, v in phase_acc.items()}
    expert_phases = {k: v for k, v in phases.items() if k in ("expand", "down", "down_combine", "up_rows", "down_rows", "up_tiles", "down_tiles")}
    dominant = max(expert_phases, key=expert_phases.get) if expert_phases else None
    roofline = None
    if dominant:
        dur_s = phases[dominant] / 1e3
        H, F, R = layer.hidden, layer.ffn, tokens * layer.top_k
        n_up = 1 if layer.arch == synth.ARCH_NEMOTRON else 2
        # below the ridge (FLOP per byte at which the tensor peak meets the copy bandwidth) the step is memory-bound
        hbm_bound = alg_flops / alg_bytes < peaks["tflops"] * 1e12 / (peaks["hbm_gbs"] * 1e9)
        if hbm_bound:
            # the phase streams the packed rows of the experts it touches once
            rb_up, rb_dn = synth.row_bytes(layer.fmt, H), synth.row_bytes(layer.fmt, F)
            n_exp = layer.top_k if decode else touched
            up_bytes, dn_bytes = n_exp * n_up * F * rb_up, n_exp * H * rb_dn
            per = {"expand": up_bytes, "down": dn_bytes, "down_combine": dn_bytes, "up_rows": up_bytes, "down_rows": dn_bytes,
                   "up_tiles": up_bytes, "down_tiles": dn_bytes}
            units = per.get(dominant, alg_bytes)
            achieved = units / dur_s / 1e9
            roofline = dict(bound="hbm", kernel=dominant, achieved=achieved, peak=peaks["hbm_gbs"], unit="GB/s",
                            frac=achieved / peaks["hbm_gbs"], traffic=NCU_TRAFFIC.get((args.workload, dominant)),
                            peak_source=f"{peaks['source']} copy bandwidth",
                            algorithmic_bytes_per_launch=units, launch_ms=phases[dominant],
                            whole_step=dict(bytes=alg_bytes, gbs=alg_bytes / (ms_per_step / 1e3) / 1e9,
                                            frac=alg_bytes / (ms_per_step / 1e3) / 1e9 / peaks["hbm_gbs"]))
        else:
            per = {"up_tiles": 2.0 * R * n_up * F * H, "down_tiles": 2.0 * R * H * F}
            units = per.get(dominant, alg_flops)
            achieved = units / dur_s / 1e12
            long_run = wall > 2.0 and peaks.get("tflops_sustained")
            peak = peaks["tflops_sustained"] if long_run else peaks["tflops"]
            roofline = dict(bound="tensor", kernel=dominant, achieved=achieved, peak=peak, unit="TFLOP/s",
                            frac=achieved / peak, traffic=NCU_TRAFFIC.get((args.workload, dominant)) if tokens == default_tokens else None,
                            peak_source=f"{peaks['source']} dense bf16 cuBLAS, {'sustained' if long_run else 'burst'}",
                            algorithmic_flops_per_launch=units, launch_ms=phases[dominant],
                            whole_step=dict(flops=alg_flops, tflops=alg_flops / (ms_per_step / 1e3) / 1e12,
                                            bytes=alg_bytes, gbs=alg_bytes / (ms_per_step / 1e3) / 1e9))
    base = None
    if not args.no_cpu_baseline:
        base, _ = cpu_baseline(layer, tokens, args.seed, args.cpu_tokens)

    line = dict(
        metric=METRIC, value=value, unit="tokens/s", n_gpus=world, steps=args.steps, warmup=args.warmup,
        ms_per_step=ms_per_step, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f16",
        data="synthetic",
        config=dict(workload=args.workload, tokens_per_gpu=tokens, hidden=layer.hidden, ffn=layer.ffn,
                    experts=layer.experts, top_k=layer.top_k, weight_format={39: "MXFP4", 12: "Q4_K", 2: "Q4_0"}[layer.fmt],
                    experts_touched=touched, weight_copies=copies,
                    cache="every step reads all expert weights (%.0f MB), more than the 126 MB L2" % (per_step_bytes / 1e6)
                    if not decode else "%d weight copies rotated per step (%.0f MB between reuses)" % (copies, copies * per_step_bytes / 1e6),
                    cuda_graph=graphs[0] is not None, fused_add_norm=bool(args.with_norm),
                    parallelism="replicas" if world > 1 else "single"),
        clocks=clocks, e2e=e2e, gpu_launches=launches, phases_ms=phases, roofline=roofline, cpu_baseline=base,
        step_ms_min=min(step_ms), step_ms_max=max(step_ms))
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
