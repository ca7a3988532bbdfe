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
# the dense products either side of the layer (oco_dense_*): name -> (kind, format, hidden, ffn, default rows)
DENSE_WORKLOADS = {
    "nemotron-shared-ffn-prefill": ("relu2", "Q4_0", 2688, 3712, 1024),
    "nemotron-shared-ffn-decode": ("relu2", "Q4_0", 2688, 3712, 1),
    "qwen3-dense-ffn-prefill": ("silu_gate", "Q4_K", 2048, 6144, 512),
}
# DRAM bytes (read + write) of one launch of the dominant kernels, from ncu captures of the same commands
# (dram__bytes_read.sum + dram__bytes_write.sum of one launch); a profiler is never attached to a timed run.
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


FP4_NOMINAL_TFLOPS, FP8_NOMINAL_TFLOPS = 9000.0, 4500.0   # dense, per GPU (vendor figures)


def tensor_peaks():
    """Tensor-pipe ceilings measured on this GPU with the library's own issue loop (tcgen05.mma, M128 N256,
    zero operands): what a kernel of each kind could reach at best, beside the vendor's nominal figures."""
    import ctypes as C
    from oco_b200 import _lib
    out = {}
    for kind, name in enumerate(("f16_tcgen05", "fp8_tcgen05", "mxfp8_tcgen05", "mxfp4_tcgen05")):
        v = C.c_float(0.0)
        rc = _lib.lib().oco_tensor_peak(kind, 4096, C.byref(v))
        out[name + "_tflops"] = float(v.value) if rc == _lib.OK else None
    out["fp4_nominal_tflops"], out["fp8_nominal_tflops"] = FP4_NOMINAL_TFLOPS, FP8_NOMINAL_TFLOPS
    out["how"] = "oco_tensor_peak: 4096 x 4 back-to-back tcgen05.mma per SM, best of 3, CUDA events"
    return out


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
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50"],
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
                    reasons=sorted(reasons), samples=len(sm), sm_mhz_all=sm)


def algorithmic(layer: synth.Layer, tokens: int, ids: np.ndarray):
    """Algorithmic bytes and FLOPs of one step: every touched expert's packed weights and biases
    once, the router once, the input rows in and the residual rows in and out."""
    touched = len(np.unique(ids))
    io = tokens * layer.hidden * 2 * 3
    total_bytes = touched * layer.expert_bytes() + layer.shared_bytes() + layer.router_bytes() + io
    return total_bytes, layer.flops(tokens), touched


def cpu_baseline(layer, tokens, seed, sample_tokens, threads=None):
    """Times the CPU restatement (f32 FMA accumulation, all host threads) on a bounded sample of
    the same workload: the first `sample_tokens` tokens of the batch."""
    import oracle
    # all the cores this process may use, whatever OMP_NUM_THREADS says (torchrun sets it to 1)
    oracle.set_num_threads(threads or len(os.sched_getaffinity(0)))
    n = max(1, min(tokens, sample_tokens))
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
    """CPU arm: the reference's MoE arithmetic restated in C++ (oracle/), timed on the host cores with all the
    threads the process may use. A step is the whole batch when K + W of them fit in about four minutes
    (they do for the default workload), else a bounded sample of it."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    cfg, default_tokens = WORKLOADS[args.workload]
    tokens = args.tokens or default_tokens
    layer = synth.make_config(cfg, seed=args.seed)
    probe = min(tokens, 64)
    _, dt = cpu_baseline(layer, tokens, args.seed, probe)
    runs = args.warmup + args.steps
    # per-token cost falls as the batch grows (each expert's rows are decoded once per batch), so the probe's
    # rate is a safe upper bound on the time of a larger step
    sample = tokens if dt / probe * tokens * runs <= 240.0 else max(probe, int(240.0 / runs / (dt / probe)))
    sample = min(sample, tokens)
    times = []
    base = None
    for i in range(runs):
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
                            note="each step is the whole batch on the host cores" if sample == tokens else
                                 "each step is a bounded sample of the batch on the host cores"),
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


def run_expert_parallel(args, torch, dist, world, rank, local, workload, steps, warmup, with_cpu=False):
    """Experts sharded over the ranks, the batch split evenly between them (its total is fixed as N
    grows). The timed step is oco_b200.ep.forward_window: the expert stage gathers token rows from
    the peers' memory and stores route outputs into it, two small collectives order the ranks. The
    all-to-all form of the same layer (ep.forward) is timed beside it. Returns rank 0's record
    (None elsewhere)."""
    from oco_b200 import ep
    cfg, default_tokens = WORKLOADS[workload]
    total = (args.tokens if workload == args.workload and args.tokens else default_tokens)
    if total % world:
        raise SystemExit(f"{total} tokens do not divide over {world} ranks")
    T = total // world
    layer = synth.make_config(cfg, seed=args.seed)
    E, K, H, F = layer.experts, layer.top_k, layer.hidden, layer.ffn
    be = ep.CudaBackend(layer, rank, world, max_rows=T)
    backend = be.backend()
    # every rank must have its windows, or none uses them
    win, why = None, ""
    try:
        win = ep.Windows(H, K, T)
    except Exception as e:     # the driver's virtual-memory calls or descriptor passing are unavailable here
        why = f"{type(e).__name__}: {e}"[:200]
    ok = torch.tensor([1.0 if win is not None else 0.0], device="cuda")
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if ok.item() == 0.0:
        raise RuntimeError("expert-parallel windows could not be set up on every rank" + (f" ({why})" if why else ""))
    x_all, res_all = synth.make_tokens(H, total, args.seed, "normal")
    x_bits, res_bits = x_all[rank * T:(rank + 1) * T], res_all[rank * T:(rank + 1) * T]
    hx = torch.from_numpy(x_bits.view(np.int16).copy()).pin_memory()
    hres = torch.from_numpy(res_bits.view(np.int16).copy()).pin_memory()
    x, res = win.x_local[:T], hres.cuda()
    x.copy_(hx)
    stream = torch.cuda.current_stream()

    def step_window(timings=None):
        ep.forward_window(x, res, be, win, timings=timings)

    def step_all_to_all(exchange=None):
        ep.forward(x, res, backend, E, exchange=exchange, uniform=True)

    # ---- parity of this rank's rows against the CPU checker (a token sample), before any timing ----
    import oracle
    step_window()
    torch.cuda.synchronize()
    got = res.cpu().numpy().view(np.uint16)
    ids_gpu, _ = be.route(x)
    ids_gpu = ids_gpu.cpu().numpy().astype(np.uint32)
    pick = np.unique(np.linspace(0, T - 1, 4).astype(int))
    ref = oracle.moe_forward(layer, x_bits[pick], res_bits[pick], mode=2, trace=False)
    _, ids_ref, _ = oracle.router_gptoss(x_bits, layer.router_w, layer.router_b, K)
    g = synth.bf16_bits_to_f32(got[pick]).astype(np.float64)
    r = synth.bf16_bits_to_f32(ref.out).astype(np.float64)
    par = torch.tensor([float(np.array_equal(ids_gpu, ids_ref.astype(np.uint32))),
                        float(np.linalg.norm(g - r) / max(np.linalg.norm(r), 1e-30))], device="cuda", dtype=torch.float64)
    worst = par.clone()
    dist.all_reduce(worst[1:], op=dist.ReduceOp.MAX)
    dist.all_reduce(par[:1], op=dist.ReduceOp.MIN)
    parity = dict(ids_exact=bool(par[0].item() == 1.0), rel_l2=float(worst[1].item()), tolerance=1e-3,
                  sample=f"{len(pick)} tokens per rank against the CPU checker; ids of all tokens; worst rank")
    res.copy_(hres)

    def timed(n, fn, count=lambda: be.launches()):
        dist.barrier(); torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        launches = 0
        for _ in range(n):
            fn()
            launches += count()
        b.record(stream)
        torch.cuda.synchronize(); dist.barrier()
        t = torch.tensor([a.elapsed_time(b) / n], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), launches

    for _ in range(max(3, warmup)):
        step_window()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start(); time.sleep(0.2)
    ms_per_step, launches = timed(steps, step_window)
    clocks = sampler.stop() if rank == 0 else {}
    clocks.pop("sm_mhz_all", None)
    be.router_plan.poll(); be.expert_plan.poll()
    # per-stage times of single steps
    tm, acc = {}, {}
    be.expert_plan.set_profiling(True)
    for _ in range(min(5, steps)):
        step_window(tm)
        for k, v in tm.items():
            acc.setdefault(k, []).append(v)
        for k, v in be.expert_plan.phase_times().items():
            acc.setdefault(k, []).append(v)
    be.expert_plan.set_profiling(False)
    phases = {k: float(np.mean(v)) for k, v in acc.items()}
    # routes this rank's shard owned (for the flop count of its tiles)
    epr = E // world
    ids_every = torch.empty(world * T * K, dtype=torch.int32, device="cuda")
    dist.all_gather_into_tensor(ids_every, torch.from_numpy(ids_ref.astype(np.int32).reshape(-1)).cuda())
    routes_here = int(((ids_every // epr) == rank).sum().item())
    # the all-to-all form of the same layer, and the same with the exchange replaced by device-local copies
    for _ in range(3):
        step_all_to_all()
    ms_a2a, _ = timed(steps, step_all_to_all)
    rec = _Recorded(dist)
    step_all_to_all(rec)
    ms_local, _ = timed(steps, lambda: step_all_to_all(_Replayed(rec.log)))
    # end to end: pinned host rows into the window slot, the layer, residual rows back
    e2e_steps = max(3, min(steps, 10))
    dist.barrier(); torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        x.copy_(hx, non_blocking=True); res.copy_(hres, non_blocking=True)
        step_window()
        hres.copy_(res, non_blocking=True)
        torch.cuda.synchronize()
    t = torch.tensor([1e3 * (time.perf_counter() - t0) / e2e_steps], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item())
    x = None
    win.close()
    del be, backend, win
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    peaks = measured_peaks()
    row_bytes = T * H * 2
    e2e = dict(value=total / (e2e_ms / 1e3), unit="tokens/s", ms_per_step=e2e_ms, h2d_bytes_per_step=2 * row_bytes,
               d2h_bytes_per_step=row_bytes,
               api="oco_b200.ep.forward_window (pinned host rows into the rank's window slot, residual rows back), per rank")
    roofline = None
    if "up_tiles" in phases:
        flops = 2.0 * routes_here * 2 * F * H
        ach = flops / (phases["up_tiles"] / 1e3) / 1e12
        roofline = dict(bound="tensor", kernel="up_tiles", achieved=ach, peak=peaks["tflops"], unit="TFLOP/s",
                        frac=ach / peaks["tflops"], traffic=None, peak_source=f"{peaks['source']} dense bf16 cuBLAS, burst",
                        algorithmic_flops_per_launch=flops, launch_ms=phases["up_tiles"], routes_on_rank0=routes_here)
    base = None
    if with_cpu:
        base, _ = cpu_baseline(layer, total, args.seed, args.cpu_tokens)
    remote = (world - 1) / world
    return dict(
        value=total / (ms_per_step / 1e3), unit="tokens/s", n_gpus=world, steps=steps, warmup=warmup, ms_per_step=ms_per_step,
        scaling="strong", dtype="f16",
        config=dict(workload=workload, tokens_total=total, tokens_per_gpu=T, hidden=H, ffn=F, experts=E, top_k=K,
                    weight_format="MXFP4", experts_per_gpu=E // world, parallelism=f"ep{world}",
                    exchange="windows over peer memory: token rows gathered by the expert stage's own loads, outputs "
                             "stored to their owners by the down tiles; one all-gather of ids and one one-word all-reduce",
                    cache="every step reads the rank's whole expert shard (%.0f MB), more than the 126 MB L2"
                          % (E // world * layer.expert_bytes() / 1e6)),
        peer_traffic=dict(rows_read_from_peers_bytes=int(routes_here * remote * H * 2),
                          rows_stored_to_peers_bytes=int(routes_here * remote * H * 2),
                          note="expected share (world - 1) / world of this shard's routes, each way"),
        all_to_all_form=dict(ms_per_step=ms_a2a, ms_per_step_with_local_copies=ms_local, exposed_ms=ms_a2a - ms_local,
                             route_bytes_each_way_per_gpu=T * K * H * 2,
                             note="ep.forward: NCCL all_to_all_single each way, sort/gather/scatter in torch"),
        parity=parity, clocks=clocks, e2e=e2e, gpu_launches=launches, phases_ms=phases, roofline=roofline, cpu_baseline=base)


def run_dense(args, ctx):
    """A dense feed-forward (oco_dense_forward) on this rank's GPU: device-timed steps over rotated weight
    copies (more bytes between reuses than the L2 holds), the end-to-end call with pinned host rows, a token
    sample against the CPU checker, the checker timed as the CPU baseline. Returns rank 0's record."""
    torch, dist, world, rank, local = ctx
    from oco_b200 import dense
    import oracle
    kind_name, fmt_name, H, F, default_rows = DENSE_WORKLOADS[args.workload]
    kind = dict(relu2=dense.FFN_RELU2, silu_gate=dense.FFN_SILU_GATE)[kind_name]
    fmt = dict(Q4_0=synth.FMT_Q4_0, Q4_K=synth.FMT_Q4_K)[fmt_name]
    rows = args.tokens or default_rows
    n_mat = 3 if kind == dense.FFN_SILU_GATE else 2
    weight_bytes = n_mat * F * synth.row_bytes(fmt, H) if kind != dense.FFN_RELU2 else F * synth.row_bytes(fmt, H) + H * synth.row_bytes(fmt, F)
    if kind == dense.FFN_SILU_GATE:
        weight_bytes = 2 * F * synth.row_bytes(fmt, H) + H * synth.row_bytes(fmt, F)
    copies = max(2, int(np.ceil(600e6 / weight_bytes)))
    rng = np.random.default_rng(args.seed)
    gen = synth._RANDOM[fmt]
    plans, host_w = [], None
    for c in range(copies):
        w = (gen(rng, F, H), gen(rng, F, H) if kind == dense.FFN_SILU_GATE else None, gen(rng, H, F))
        host_w = host_w or w
        p = dense.DensePlan(kind, fmt, H, F)
        p.reserve(rows)
        p.bind(*w)
        plans.append(p)
    x_bits, _ = synth.make_tokens(H, rows, args.seed + 1000 * rank, "zero")
    x_bits = synth.f32_to_bf16_bits(synth.bf16_bits_to_f32(x_bits) * np.float32(0.25))
    hx = torch.from_numpy(x_bits.view(np.int16).copy()).pin_memory()
    hy = torch.empty((rows, H), dtype=torch.int16).pin_memory()
    x, y = hx.cuda(), torch.empty((rows, H), dtype=torch.int16, device="cuda")
    stream = torch.cuda.current_stream()
    # parity first: a row sample of the first weight copy against the checker
    plans[0].forward(x, y, rows)
    torch.cuda.synchronize(); plans[0].poll()
    pick = np.unique(np.linspace(0, rows - 1, 8).astype(int))
    ref = oracle.dense_forward(kind, fmt, H, F, host_w[0], host_w[1], host_w[2], x_bits[pick], tile=rows > 1)
    g = synth.bf16_bits_to_f32(y.cpu().numpy().view(np.uint16)[pick]).astype(np.float64)
    r = synth.bf16_bits_to_f32(ref).astype(np.float64)
    parity = dict(rel_l2=float(np.linalg.norm(g - r) / max(np.linalg.norm(r), 1e-30)), tolerance=1e-3, sample=f"{len(pick)} rows against the CPU checker")
    for i in range(max(3, args.warmup)):
        plans[i % copies].forward(x, y, rows)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start(); time.sleep(0.2)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(stream)
    launches = 0
    for i in range(args.steps):
        plans[i % copies].forward(x, y, rows)
        launches += plans[i % copies].launch_count()
    b.record(stream)
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / args.steps], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.barrier()
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    clocks = sampler.stop() if rank == 0 else {}
    clocks.pop("sm_mhz_all", None)
    plans[0].poll()
    e2e_steps = max(3, min(args.steps, 10))
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        x.copy_(hx, non_blocking=True)
        plans[i % copies].forward(x, y, rows)
        hy.copy_(y, non_blocking=True)
        torch.cuda.synchronize()
    e2e_ms = 1e3 * (time.perf_counter() - t0) / e2e_steps
    if rank != 0:
        return None
    peaks = measured_peaks()
    flops = 2.0 * rows * H * F * n_mat
    bytes_step = weight_bytes + rows * H * 2 * 2
    tensor_bound = rows > 64
    ach = flops / (ms / 1e3) / 1e12 if tensor_bound else bytes_step / (ms / 1e3) / 1e9
    peak = peaks["tflops"] if tensor_bound else peaks["hbm_gbs"]
    roofline = dict(bound="tensor" if tensor_bound else "hbm", kernel="whole call (two tile or two token launches plus the row conversion)",
                    achieved=ach, peak=peak, unit="TFLOP/s" if tensor_bound else "GB/s", frac=ach / peak, traffic=None,
                    peak_source=f"{peaks['source']} " + ("dense bf16 cuBLAS, burst" if tensor_bound else "HBM copy"),
                    algorithmic_flops_per_step=flops, algorithmic_bytes_per_step=bytes_step)
    cpu = None
    if not args.no_cpu_baseline:
        n = min(rows, args.cpu_tokens)
        t0 = time.perf_counter()
        oracle.dense_forward(kind, fmt, H, F, host_w[0], host_w[1], host_w[2], x_bits[:n], tile=rows > 1)
        dt = time.perf_counter() - t0
        cpu = dict(value=n / dt, unit="tokens/s", cores=oracle.num_threads(), kind="port",
                   sample=f"first {n} of {rows} rows, one pass, {dt:.2f} s wall clock; C++ restatement of the reference's dense products")
    return dict(metric="dense feed-forward tokens/s (the step beside the MoE layer)", value=world * rows / (ms / 1e3), unit="tokens/s",
                n_gpus=world, steps=args.steps, warmup=args.warmup, ms_per_step=ms, higher_is_better=True, scaling="weak",
                vs_baseline=None, dtype="f16" if rows > 1 else "f32", data="synthetic",
                config=dict(workload=args.workload, rows_per_gpu=rows, hidden=H, ffn=F, kind=kind_name, weight_format=fmt_name,
                            weight_copies=copies, cache="%d weight copies rotated per step (%.0f MB between reuses)" % (copies, copies * weight_bytes / 1e6),
                            parallelism="replicas"),
                clocks=clocks, e2e=dict(value=world * rows / (e2e_ms / 1e3), unit="tokens/s", ms_per_step=e2e_ms, h2d_bytes_per_step=rows * H * 2,
                                        d2h_bytes_per_step=rows * H * 2, api="oco_dense_forward (pinned host rows in, result rows back)"),
                gpu_launches=launches, roofline=roofline, parity=parity, cpu_baseline=cpu)


def block_scaled_distance(workload, tokens, seed, repacked):
    """What the opt-in block-scaled mode costs in accuracy: a token sample of its output against the checker that
    carries the reference's arithmetic."""
    from oco_b200 import moe as _moe
    import oracle
    cfg_name, dt = WORKLOADS[workload]
    tk = tokens or dt
    lay = synth.make_config(cfg_name, seed=0 if seed is None else seed % 1000)
    xb, rb = synth.make_tokens(lay.hidden, tk, seed, "normal")
    got, routing = _moe.run_layer(lay, xb, rb, numerics=2, repacked=repacked)
    pick = np.unique(np.linspace(0, tk - 1, 8).astype(int))
    ref = oracle.moe_forward(lay, xb[pick], rb[pick], mode=2, trace=False)
    g = synth.bf16_bits_to_f32(got[pick]).astype(np.float64)
    r = synth.bf16_bits_to_f32(ref.out).astype(np.float64)
    moe_part = r - synth.bf16_bits_to_f32(rb[pick]).astype(np.float64)
    return dict(ids_exact=bool(np.array_equal(routing["ids"][pick], ref.ids)),
                rel_l2_vs_reference_arithmetic=float(np.linalg.norm(g - r) / np.linalg.norm(r)),
                rel_l2_of_the_layer_term_alone=float(np.linalg.norm(g - r) / max(np.linalg.norm(moe_part), 1e-30)),
                sample=f"{len(pick)} tokens against the CPU checker (reference arithmetic); the mode's own arithmetic "
                       "(the same quantised operands in float64) is held to 1e-3 by the GPU tests")


def measure_layer(args, ctx, workload, steps, warmup, tokens=0, graph=True, with_norm=False, layers=0, sustained_s=0.0, numerics=0):
    """One workload on this rank's GPU (every rank runs the same layer on its own tokens): device-timed
    steps, per-kernel phase times, the end-to-end call with host buffers and, on request, a seconds-long
    loop with the SM clock sampled. Returns rank 0's record (other ranks: the timing fields only)."""
    torch, dist, world, rank, local = ctx
    from oco_b200 import moe
    cfg, default_tokens = WORKLOADS[workload]
    tokens = tokens or default_tokens
    layer = synth.make_config(cfg, seed=args.seed)
    decode = tokens == 1
    # Cold-cache protocol. Prefill reads every expert (hundreds of MB, more than the 126 MB L2) each
    # step, so the inputs themselves exceed L2. A single token touches only top_k experts (tens of
    # MB), so distinct weight copies are rotated step by step and never revisited within L2 reach.
    per_step_bytes = layer.top_k * layer.expert_bytes() if decode else layer.experts * layer.expert_bytes()
    copies = layers or (max(2, int(np.ceil(600e6 / per_step_bytes))) if decode else 1)
    weights = [moe._Weights.from_layer(layer) for _ in range(copies)]
    plans = []
    for w in weights:
        p = moe.plan_for(layer, numerics=numerics)
        p.reserve(tokens)
        p.bind(w)
        if getattr(args, "repacked", False) and layer.arch == synth.ARCH_GPT_OSS and (numerics == 2 or decode):
            # the optional second form of the expert tensors: the block-scaled tiles (numerics 2) and, with
            # OCO_MOE_REPACKED_TOKEN=1, the single-token kernels (any numerics) then get every operand by bulk copies
            p.repack()
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
        if with_norm:
            p.add_norm_forward(res, x, norm_w, 1e-5, layer.arch == synth.ARCH_GPT_OSS, tokens)   # x stands in for the mixer's output
        else:
            p.forward(x, res, tokens)
        return p

    for i in range(max(warmup, copies if decode else 0)):
        step(i)
    torch.cuda.synchronize()
    plans[0].poll()
    if decode and graph:
        # A single token is a handful of microsecond kernels: record each weight copy's step as a graph of the
        # library (oco_moe_graph_capture) so the timed region measures the GPU, not the host's launch rate.
        # (The fused add-norm entry point has no graph call of its own and is captured through torch.)
        if not with_norm:
            for c in range(copies):
                plans[c].set_profiling(False)
                graphs[c] = plans[c].capture(x, res, tokens)
        else:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for c in range(copies):
                    plans[c].set_profiling(False)
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=side):
                        plans[c].add_norm_forward(res, x, norm_w, 1e-5, layer.arch == synth.ARCH_GPT_OSS, tokens)
                    graphs[c] = g
            torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
    # routing of this batch (for the algorithmic byte count)
    routing = moe.Routing(); routing.plan, routing.rows = plans[(warmup - 1) % copies if warmup else 0], tokens
    if not warmup:
        step(0); torch.cuda.synchronize()
    ids = routing.read()["ids"]
    alg_bytes, alg_flops, touched = algorithmic(layer, tokens, ids)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.2)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    phase_acc = {}
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    launches = 0
    t_wall = time.perf_counter()
    for i in range(steps):
        starts[i].record(stream)
        p = step(warmup + i, profile=False)
        ends[i].record(stream)
        launches += p.launch_count()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    wall = time.perf_counter() - t_wall
    clocks = sampler.stop() if rank == 0 else {}
    clocks.pop("sm_mhz_all", None)
    # Per-kernel durations: the phase events of a plan hold its last call, so a few more steps are
    # run one at a time and read back (same kernels, same inputs, still rotating weight copies).
    for i in range(min(10, steps)):
        p = step(warmup + steps + i, profile=True)
        torch.cuda.synchronize()
        for k, v in p.phase_times().items():
            phase_acc.setdefault(k, []).append(v)
    for p in plans:
        p.set_profiling(False)
    step_ms = [s.elapsed_time(e) for s, e in zip(starts, ends)]
    total_ms = starts[0].elapsed_time(ends[-1])
    ms_per_step = total_ms / steps
    if world > 1:
        t = torch.tensor([ms_per_step], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_per_step = float(t.item())
    plans[0].poll()
    value = world * tokens / (ms_per_step / 1e3)

    # ---- a seconds-long run of the same step, the SM clock sampled every 50 ms -------------------------
    sustained = None
    if sustained_s > 0:
        n = max(steps, int(sustained_s * 1e3 / max(ms_per_step, 1e-3)) + 1)
        s2 = ClockSampler(local)
        if rank == 0:
            s2.start(); time.sleep(0.1)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record(stream)
        for i in range(n):
            step(i)
        b.record(stream)
        torch.cuda.synchronize()
        c2 = s2.stop() if rank == 0 else {}
        ms_long = a.elapsed_time(b) / n
        if rank == 0:
            mhz = np.array(c2.pop("sm_mhz_all", []) or [0.0])
            under = mhz[mhz >= np.median(mhz)] if len(mhz) else mhz
            hist = {str(int(k)): int(v) for k, v in zip(*np.unique((mhz // 100) * 100, return_counts=True))}
            sustained = dict(seconds=ms_long * n / 1e3, steps=n, ms_per_step=ms_long, tokens_per_s=tokens / (ms_long / 1e3),
                             sm_mhz_median_under_load=float(np.median(under)), sm_mhz_histogram_100mhz_bins=hist,
                             ms_times_median_mhz=ms_long * float(np.median(under)), reasons=c2.get("reasons"),
                             burst_ms_per_step=ms_per_step)

    # ---- end to end through the host-buffer entry point -----------------------------------------
    hx = torch.from_numpy(x_bits.view(np.int16)).pin_memory()
    hres = torch.from_numpy(res_bits.view(np.int16).copy()).pin_memory()
    hx_np, hres_np = hx.numpy().view(np.uint16), hres.numpy().view(np.uint16)
    e2e_steps = max(10, min(2 * steps, 60))       # enough steps that the two calls in flight fill their pipeline
    for i in range(max(2, copies)):      # every weight copy's plan once: its first call sets up its copy streams and events
        plans[i % copies].forward_host(hx_np, hres_np, tokens)
    row_bytes = tokens * layer.hidden * 2

    def timed_host_steps(in_flight):
        """ms per step of e2e_steps host-buffer calls, every step with its H2D of x and the residual rows and its
        D2H of the residual rows. in_flight 1: one call at a time (oco_moe_forward_host). 2: a call is ended
        only after the next one was begun, so its copies cross the bus beside the other call's kernels. Each
        call in flight has its own pinned residual buffer (the library writes the rows back into it)."""
        bufs = [hres_np] + [torch.from_numpy(res_bits.view(np.int16).copy()).pin_memory().numpy().view(np.uint16)
                            for _ in range(in_flight - 1)]
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        if in_flight == 1:
            for i in range(e2e_steps):
                plans[i % copies].forward_host(hx_np, bufs[0], tokens)
        else:
            for i in range(e2e_steps):
                plans[i % copies].forward_host_begin(hx_np, bufs[i % 2], tokens)
                if i >= 1:
                    plans[(i - 1) % copies].forward_host_end()
            plans[(e2e_steps - 1) % copies].forward_host_end()
        ms = 1e3 * (time.perf_counter() - t0) / e2e_steps
        if world > 1:
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    one_ms = timed_host_steps(1)
    if tokens > 64:
        # throughput workloads: two calls in flight. With one weight copy per plan rotation the two calls may
        # belong to different plans: each plan owns its staging slots and copy streams, and all share the stream.
        two_ms = timed_host_steps(2)
        # on a host whose memory or PCIe root is shared by many ranks the second call in flight can cost more than it
        # hides: the line carries the faster of the two ways of calling, and both figures
        if two_ms <= one_ms:
            e2e_ms = two_ms
            api = "oco_moe_forward_host_begin/_end, two calls in flight (pinned host buffers in, residual rows back, every step)"
        else:
            e2e_ms = one_ms
            api = "oco_moe_forward_host, one call at a time (pinned host buffers in, residual rows back); two calls in flight were slower here"
    else:
        # latency workloads: the whole host call (copies in, kernels, copy back) as one graph of the library per plan
        hgraphs = [plans[c].capture_host(hx_np, hres_np, tokens) for c in range(copies)]
        for c in range(copies):
            hgraphs[c].replay()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            hgraphs[i % copies].replay()
            stream.synchronize()                   # the rows are back in the host buffer
        e2e_ms = 1e3 * (time.perf_counter() - t0) / e2e_steps
        if world > 1:
            t = torch.tensor([e2e_ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t.item())
        del hgraphs
        api = "oco_moe_graph_capture_host + oco_moe_graph_launch + stream wait (pinned host buffers in, residual rows back, every step)"
    e2e = dict(value=world * tokens / (e2e_ms / 1e3), unit="tokens/s", ms_per_step=e2e_ms,
               h2d_bytes_per_step=2 * row_bytes, d2h_bytes_per_step=row_bytes, api=api,
               one_call_at_a_time=dict(ms_per_step=one_ms, tokens_per_s=world * tokens / (one_ms / 1e3),
                                       api="oco_moe_forward_host"))
    if tokens > 64:
        e2e["two_calls_in_flight"] = dict(ms_per_step=two_ms, tokens_per_s=world * tokens / (two_ms / 1e3),
                                          api="oco_moe_forward_host_begin/_end")
    del plans, weights, graphs
    torch.cuda.empty_cache()
    if rank != 0:
        return None

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
                            frac=achieved / peaks["hbm_gbs"], traffic=NCU_TRAFFIC.get((workload, dominant)),
                            peak_source=f"{peaks['source']} copy bandwidth",
                            algorithmic_bytes_per_launch=units, launch_ms=phases[dominant],
                            per_kernel={k: dict(gbs=per[k] / (v / 1e3) / 1e9, frac=per[k] / (v / 1e3) / 1e9 / peaks["hbm_gbs"])
                                        for k, v in expert_phases.items() if k in per},
                            whole_step=dict(bytes=alg_bytes, gbs=alg_bytes / (ms_per_step / 1e3) / 1e9,
                                            frac=alg_bytes / (ms_per_step / 1e3) / 1e9 / peaks["hbm_gbs"]))
        else:
            per = {"up_tiles": 2.0 * R * n_up * F * H, "down_tiles": 2.0 * R * H * F}
            units = per.get(dominant, alg_flops)
            achieved = units / dur_s / 1e12
            long_run = wall > 2.0 and peaks.get("tflops_sustained")
            peak = peaks["tflops_sustained"] if long_run else peaks["tflops"]
            source = f"{peaks['source']} dense bf16 cuBLAS, {'sustained' if long_run else 'burst'}"
            if numerics == 2:
                pk4 = tensor_peaks()["mxfp4_tcgen05_tflops"]
                peak, source = (pk4 or FP4_NOMINAL_TFLOPS), ("measured tcgen05 kind::mxf4 issue loop" if pk4 else "nominal FP4")
            roofline = dict(bound="tensor", kernel=dominant, achieved=achieved, peak=peak, unit="TFLOP/s",
                            frac=achieved / peak, traffic=(NCU_TRAFFIC.get((workload, dominant)) if tokens == default_tokens and numerics == 0 else None),
                            peak_source=source, frac_of_fp4_nominal=achieved / FP4_NOMINAL_TFLOPS,
                            algorithmic_flops_per_launch=units, launch_ms=phases[dominant],
                            whole_step=dict(flops=alg_flops, tflops=alg_flops / (ms_per_step / 1e3) / 1e12,
                                            bytes=alg_bytes, gbs=alg_bytes / (ms_per_step / 1e3) / 1e9))
    return dict(
        value=value, ms_per_step=ms_per_step, layer=layer, tokens=tokens,
        config=dict(workload=workload, tokens_per_gpu=tokens, hidden=layer.hidden, ffn=layer.ffn,
                    experts=layer.experts, top_k=layer.top_k, weight_format={39: "MXFP4", 12: "Q4_K", 2: "Q4_0"}[layer.fmt],
                    experts_touched=touched, weight_copies=copies,
                    cache="every step reads all expert weights (%.0f MB), more than the 126 MB L2" % (per_step_bytes / 1e6)
                    if not decode else "%d weight copies rotated per step (%.0f MB between reuses)" % (copies, copies * per_step_bytes / 1e6),
                    cuda_graph=bool(decode and graph), fused_add_norm=bool(with_norm), numerics=numerics,
                    repacked_weights=bool(getattr(args, "repacked", False) and layer.arch == synth.ARCH_GPT_OSS and (numerics == 2 or decode)),
                    parallelism="replicas" if world > 1 else "single"),
        clocks=clocks, e2e=e2e, gpu_launches=launches, phases_ms=phases, roofline=roofline, sustained=sustained,
        step_ms_min=min(step_ms), step_ms_max=max(step_ms))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gpt-oss-20b-prefill", choices=sorted(WORKLOADS) + sorted(DENSE_WORKLOADS))
    ap.add_argument("--tokens", type=int, default=0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--cpu-tokens", type=int, default=256, help="tokens in the CPU baseline's bounded sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="only the headline workload: no decode block, tensor peaks, sustained run, CPU full batch or expert-parallel block")
    ap.add_argument("--no-graph", action="store_true", help="single-token workloads: launch kernels directly instead of replaying CUDA graphs")
    ap.add_argument("--layers", type=int, default=0, help="distinct weight copies rotated per step (0 = auto)")
    ap.add_argument("--numerics", type=int, default=0, choices=[0, 2],
                    help="2: the opt-in block-scaled mode (MXFP4 activations on tcgen05 kind::mxf4); never the headline")
    ap.add_argument("--repacked", action="store_true",
                    help="bind the repacked form of the MXFP4 expert tensors (oco_moe_bind_repacked): read by the tiles of --numerics 2 "
                         "and by single-token workloads in the reference numerics")
    ap.add_argument("--with-norm", action="store_true",
                    help="time the fused entry point: residual add + RMS norm + layer (the step either side of the layer)")
    args = ap.parse_args()
    if args.impl == "reference":
        if args.workload in DENSE_WORKLOADS:
            print(json.dumps(dict(impl="reference", unavailable="the reference arm times the MoE layer workloads only")))
            return 0
        return run_reference(args)

    import torch
    import torch.distributed as dist
    from oco_b200 import build
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
    ctx = (torch, dist, world, rank, local)
    default = args.workload == "gpt-oss-20b-prefill" and not args.tokens and args.numerics == 0
    extras = default and not args.no_extras

    if args.workload in DENSE_WORKLOADS:
        rec = run_dense(args, ctx)
        if rank == 0:
            print(json.dumps(rec))
        if world > 1:
            dist.destroy_process_group()
        return 0

    if world > 1 and args.workload in EXPERT_PARALLEL:
        rec = run_expert_parallel(args, torch, dist, world, rank, local, args.workload, args.steps, args.warmup,
                                  with_cpu=not args.no_cpu_baseline)
        if rank == 0:
            print(json.dumps(dict(metric=METRIC, higher_is_better=True, vs_baseline=None, data="synthetic", **rec)))
        dist.destroy_process_group()
        return 0

    head = measure_layer(args, ctx, args.workload, args.steps, args.warmup, tokens=args.tokens, graph=not args.no_graph,
                         with_norm=args.with_norm, layers=args.layers, sustained_s=2.0 if extras else 0.0, numerics=args.numerics)
    line = None
    if rank == 0:
        layer, tokens = head.pop("layer"), head.pop("tokens")
        line = dict(metric=METRIC, value=head.pop("value"), unit="tokens/s", n_gpus=world, steps=args.steps, warmup=args.warmup,
                    ms_per_step=head.pop("ms_per_step"), higher_is_better=True, scaling="weak", vs_baseline=None,
                    dtype="f16" if args.numerics == 0 else "mxfp4 (opt-in numerics: not the reference's arithmetic)",
                    data="synthetic", **head)
        if not args.no_cpu_baseline:
            base, _ = cpu_baseline(layer, tokens, args.seed, args.cpu_tokens)
            base["note"] = "the port is the bit-exact checker, not a tuned CPU kernel"
            if extras:
                full, dt = cpu_baseline(layer, tokens, args.seed, tokens)
                base["full_batch"] = dict(value=full["value"], unit="tokens/s", tokens=tokens, seconds=dt, cores=full["cores"])
            line["cpu_baseline"] = base
        else:
            line["cpu_baseline"] = None
    if args.numerics == 2:
        par = block_scaled_distance(args.workload, args.tokens, args.seed + 1000 * rank, args.repacked)
        if rank == 0:
            line["parity"] = par
    if extras:
        # the HBM half of the metric: one token through the same layer (three launches replayed as a graph)
        dec = measure_layer(args, ctx, "gpt-oss-20b-decode", 200, 10)
        if rank == 0:
            rl = dec["roofline"] or {}
            line["decode"] = dict(workload="gpt-oss-20b-decode", us_per_token=1e3 * dec["ms_per_step"], tokens_per_s=dec["value"] / world,
                                  whole_step_hbm_frac=(rl.get("whole_step") or {}).get("frac"),
                                  per_kernel_hbm=rl.get("per_kernel"), phases_ms=dec["phases_ms"], gpu_launches=dec["gpu_launches"],
                                  e2e_us_per_token=1e3 * dec["e2e"]["ms_per_step"], config=dec["config"],
                                  hbm_peak_gbs=measured_peaks()["hbm_gbs"], hbm_nominal_gbs=8000.0)
        # the FP4 half of the metric's tensor roofline: the same workload in the opt-in block-scaled numerics (MXFP4
        # activations; NOT the reference's arithmetic, never the headline) over the repacked form of the expert tensors
        import copy as _copy
        bs_args = _copy.copy(args)
        bs_args.repacked = True
        bs = measure_layer(bs_args, ctx, "gpt-oss-20b-prefill", 20, 5, numerics=2)
        if rank == 0:
            bs_par = block_scaled_distance("gpt-oss-20b-prefill", 0, args.seed, True)
            brl = bs["roofline"] or {}
            line["block_scaled"] = dict(numerics=2, repacked_weights=True, ms_per_step=bs["ms_per_step"], tokens_per_s=bs["value"] / world,
                                        phases_ms=bs["phases_ms"], up_tiles_tflops=brl.get("achieved"),
                                        frac_of_fp4_tcgen05_measured=brl.get("frac"), frac_of_fp4_nominal=brl.get("frac_of_fp4_nominal"),
                                        parity=bs_par, gpu_launches=bs["gpu_launches"],
                                        note="opt-in numerics: MXFP4 activations on tcgen05 kind::mxf4; its own arithmetic is held to 1e-3 by "
                                             "the GPU tests, the distance to the reference's arithmetic is parity.rel_l2_vs_reference_arithmetic")
        if rank == 0:
            # every tensor fraction against the measured and the nominal ceilings
            pk = tensor_peaks()
            mp = measured_peaks()
            pk["bf16_cublas_tflops"] = mp["tflops"]
            pk["bf16_cublas_sustained_tflops"] = mp["tflops_sustained"]
            line["peaks"] = pk
            r = line.get("roofline")
            if r and r.get("bound") == "tensor":
                a = r["achieved"]
                r["frac_of"] = {k: (a / v if v else None) for k, v in
                                dict(bf16_cublas_measured=mp["tflops"], f16_tcgen05_measured=pk["f16_tcgen05_tflops"],
                                     fp4_tcgen05_measured=pk["mxfp4_tcgen05_tflops"], fp4_nominal=FP4_NOMINAL_TFLOPS).items()}
        if world > 1:
            # the configuration that shards: 128 experts over the ranks, rows through windows over peer memory; rank 0
            # also runs it alone first, for the strong-scaling reference on the same box
            n1 = None
            if rank == 0:
                solo = measure_layer(args, (torch, dist, 1, 0, local), "gpt-oss-120b-prefill", 10, 3)
                n1 = solo["ms_per_step"]
            dist.barrier()
            try:
                epr = run_expert_parallel(args, torch, dist, world, rank, local, "gpt-oss-120b-prefill", 10, 3)
            except Exception as e:      # the headline line is printed whatever happens to this block
                epr = dict(error=f"{type(e).__name__}: {e}"[:300])
            if rank == 0:
                epr["n1_ms_per_step_same_box"] = n1
                line["expert_parallel"] = epr
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
