#!/usr/bin/env python
"""Benchmark of the fp32 GEMM hot path (one JSON line on stdout, printed by rank 0).

    python bench.py --gpus N --steps K --warmup W            # this library (CUDA, sm_100a)
    python bench.py --impl reference --gpus N ...            # CPU baseline arm (rank 0 only)

Workloads (synthetic, seeded; shapes and distributions of the specification's configs):
  N = 1   "sgemm_4096_nn_nt_tn_tt": M=N=K=4096, alpha=1.5, beta=0.5, one step = the four
          transpose combinations NN, NT, TN, TT once each (A, B, C ~ U[-1,1)).
  N > 1   "sgemm_32768_nn_row_sharded": M=N=K=32768, NN, alpha=1, beta=0; A split by row
          block over the ranks, B replicated, C all-gathered (NCCL) -- strong scaling.
Metric: fp32 GEMM TFLOP/s = 2*M*N*K per GEMM / device time, whole job.
A step never re-uses cached results: every GEMM re-reads its operands from HBM (the
working set, operands + split planes, exceeds the 126 MB L2).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "fp32_gemm_tflops"
UNIT = "TFLOP/s"
SEED = 20240601

# DRAM bytes per launch of the dominant kernel from the committed ncu capture
# (profiles/sgemm_tc3x_4096_ncu.md, profiles/sgemm_tc3x_65536x256x4096_ncu.md: dram__bytes_read.sum +
# dram__bytes_write.sum); None where no capture exists.
NCU_TRAFFIC_BYTES = {"sgemm_4096_nn_nt_tn_tt": 588.9e6, "sgemm_65536x256x4096_nn_row_sharded": 1136.1e6}


def log(*a):
    print(*a, file=sys.stderr, flush=True)


def env_rank():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(hbm_gbs=d["hbm_gbs"], bf16=d["bf16_tflops"], bf16_sustained=d["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons of one GPU while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None
        self.tmp = None

    def start(self):
        try:
            self.tmp = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.idx), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=self.tmp, stderr=subprocess.DEVNULL)
        except Exception as e:  # nvidia-smi missing
            log("clock sampler unavailable:", e)
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if not self.proc:
            return out
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.tmp.flush()
        rows = []
        with open(self.tmp.name) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) >= 7:
                    rows.append(parts)
        os.unlink(self.tmp.name)
        if not rows:
            return out
        sm = [float(r[0]) for r in rows if r[0].replace(".", "").isdigit()]
        # "under load": samples in the upper half of the power range seen
        try:
            pw = [float(r[2]) for r in rows]
            thr = (max(pw) + min(pw)) / 2
            sm_load = [float(r[0]) for r in rows if float(r[2]) >= thr] or sm
        except ValueError:
            sm_load = sm
        reasons = []
        for name, col in (("hw_slowdown", 3), ("hw_thermal_slowdown", 4), ("sw_thermal_slowdown", 5), ("sw_power_cap", 6)):
            if any(r[col].lower().startswith("active") for r in rows):
                reasons.append(name)
        out.update(sm_mhz=statistics.median(sm_load) if sm_load else None,
                   sm_max_mhz=float(rows[0][1]) if rows[0][1].replace(".", "").isdigit() else None,
                   reasons=reasons, samples=len(rows))
        return out


# --------------------------------------------------------------------------- workloads
def workload_for(n_gpus: int, name: str | None):
    w = {
        "sgemm_4096_nn_nt_tn_tt": dict(m=4096, n=4096, k=4096, alpha=1.5, beta=0.5,
                                       cases=[(0, 0), (0, 1), (1, 0), (1, 1)], sharded=False),
        "sgemm_32768_nn_row_sharded": dict(m=32768, n=32768, k=32768, alpha=1.0, beta=0.0, cases=[(0, 0)], sharded=True),
        "sgemm_1024_nn": dict(m=1024, n=1024, k=1024, alpha=1.0, beta=0.0, cases=[(0, 0)], sharded=False),
        "sgemm_65536x256x4096_nn_row_sharded": dict(m=65536, n=256, k=4096, alpha=1.0, beta=0.0, cases=[(0, 0)],
                                                    sharded=True),
    }
    if name is None:
        name = "sgemm_4096_nn_nt_tn_tt" if n_gpus == 1 else "sgemm_32768_nn_row_sharded"
    if name not in w:
        raise SystemExit(f"unknown workload {name}; choose from {sorted(w)}")
    if n_gpus > 1 and not w[name]["sharded"]:
        raise SystemExit(f"workload {name} does not shard; run it with --gpus 1")
    return name, w[name]


def flops_per_step(w):
    return 2.0 * w["m"] * w["n"] * w["k"] * len(w["cases"])


# --------------------------------------------------------------------------- CPU arm
def cpu_gemm_rate(w, threads, budget_s, steps, warmup):
    """Times MKL sgemm (torch CPU) on a bounded sample of the workload.
    Returns (TFLOP/s, seconds per step, sample description, sample flops)."""
    import torch
    from oracle import ref_gemm as og

    torch.set_num_threads(threads)
    m, n, k = w["m"], w["n"], w["k"]
    g = torch.Generator().manual_seed(SEED)
    # probe the host's sgemm rate on a small problem to size the sample
    pa = torch.empty(1024, 2048).uniform_(-1, 1, generator=g)
    pb = torch.empty(2048, 2048).uniform_(-1, 1, generator=g)
    pc = torch.empty(1024, 2048)
    og.mkl_proxy_gemm(0, 0, 1.0, pa, pb, 0.0, pc)
    t0 = time.perf_counter()
    og.mkl_proxy_gemm(0, 0, 1.0, pa, pb, 0.0, pc)
    rate = 2.0 * 1024 * 2048 * 2048 / max(time.perf_counter() - t0, 1e-6)
    # rows of A (and C) per sampled GEMM so that warmup+steps fit the budget
    per_step_budget = budget_s / max(1, steps + warmup)
    rows = int(per_step_budget * rate / (2.0 * n * k * len(w["cases"])))
    rows = max(256, min(m, rows // 256 * 256))
    b = torch.empty(k, n).uniform_(-1, 1, generator=g)          # stored k x n or n x k: square or NN only
    results = []
    for (ta, tb) in w["cases"]:
        a = torch.empty((k, rows) if ta else (rows, k)).uniform_(-1, 1, generator=g)
        bb = b if not tb else b.t().contiguous() if n != k else b
        results.append((ta, tb, a, bb, torch.empty(rows, n).uniform_(-1, 1, generator=g)))
    flops = 2.0 * rows * n * k * len(w["cases"])

    def step():
        for (ta, tb, a, bb, c) in results:
            og.mkl_proxy_gemm(ta, tb, w["alpha"], a, bb, w["beta"], c)

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    sample = (f"MKL sgemm via torch CPU (oneMKL proxy for the reference's oneMKL call), {threads} threads, "
              f"{rows} of {m} rows of A/C per GEMM x {len(w['cases'])} GEMMs per step, full N={n} K={k}, "
              f"{steps} timed steps")
    return flops / dt / 1e12, dt, sample, flops


def run_reference(args):
    rank, world, _ = env_rank()
    if rank != 0:
        return
    name, w = workload_for(args.gpus, args.workload)
    threads = len(os.sched_getaffinity(0))
    tf, dt, sample, _ = cpu_gemm_rate(w, threads, budget_s=120.0, steps=args.steps, warmup=args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": round(tf, 4), "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": name, "m": w["m"], "n": w["n"], "k": w["k"], "alpha": w["alpha"], "beta": w["beta"],
                   "transposes": ["NT"[ta] + "NT"[tb] for ta, tb in w["cases"]],
                   "note": "the reference's SYCL/oneMKL build is unavailable on this box; MKL sgemm (torch CPU) stands in"},
        "cpu_baseline": {"value": round(tf, 4), "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": round(tf, 4), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU arm
def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from sushiblas_b200 import SushiCuda, load_library
    from sushiblas_b200.capi import partition, workspace_bytes

    rank, world, local_rank = env_rank()
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    if not torch.cuda.is_available():
        raise SystemExit("no CUDA device: this library has no CPU fallback")
    load_library()                       # fails loudly if the CUDA extension was not built
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    name, w = workload_for(args.gpus, args.workload)
    m, n, k, alpha, beta = w["m"], w["n"], w["k"], w["alpha"], w["beta"]

    ctx = SushiCuda([local_rank])
    # one explicit stream for torch's events/copies and the library's kernels (torch's default
    # stream has handle 0, which the C ABI reads as "use the context's own stream")
    stream = torch.cuda.Stream(device)
    torch.cuda.set_stream(stream)
    ctx.set_stream(stream.cuda_stream)
    if world > 1:
        ids = [ctx.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        ctx.comm_init_rank(ids[0], world, rank)

    first, count = partition(m, world, rank)

    def barrier():
        if world > 1:
            dist.barrier()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident inputs (rows [first, first+count) of the global A, all of B)
    a = torch.empty(count, k, device=device) if w["sharded"] else torch.empty(m, k, device=device)
    b = torch.empty(k, n, device=device)
    gather_mode = 1
    c_raw = None
    if world > 1 and args.gather == "fused":
        # C lives in a plain cudaMalloc block so that it can be mapped into the peers (CUDA IPC):
        # the GEMM epilogue then stores finished tiles straight into every rank's C over NVLink
        c_raw = ctx.malloc(m * n * 4)
        handles = [None] * world
        dist.all_gather_object(handles, ctx.ipc_export(c_raw))
        opened = [ctx.ipc_open(handles[r]) if r != rank else None for r in range(world)]
        ctx.comm_set_peer_buffers([c_raw if r == rank else opened[r] for r in range(world)], m * n * 4)
        c = c_raw
        gather_mode = 2
    else:
        c = torch.empty(m, n, device=device)
    ctx.fill_uniform(a, a.numel(), SEED, first_index=first * k if w["sharded"] else 0)
    ctx.fill_uniform(b, b.numel(), SEED + 1)
    ctx.fill_uniform(c, m * n, SEED + 2)
    ctx.reserve_workspace(workspace_bytes(count if w["sharded"] else m, n, k))
    ctx.sync()

    def step():
        if w["sharded"]:
            ctx.sgemm_row_sharded(0, 0, m, n, k, alpha, a, k, b, n, beta, c, n, gather=gather_mode)
        else:
            for (ta, tb) in w["cases"]:
                ctx.sgemm(ta, tb, m, n, k, alpha, a, m if ta else k, b, k if tb else n, beta, c, n)

    for _ in range(args.warmup):
        step()
    ctx.sync()

    # ---- timed region: K steps, CUDA events on the launching stream, max over ranks
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.25)
    ctx.kernel_timing_enable(True)
    launches0 = ctx.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    torch.cuda.synchronize()
    wall0 = time.perf_counter()
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    torch.cuda.synchronize()
    barrier()
    wall = time.perf_counter() - wall0
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    gemm_ms, gemm_launches, prepass_ms, prepass_launches = ctx.kernel_timing_read()
    ctx.kernel_timing_enable(False)
    launches = ctx.launch_count() - launches0
    clocks = sampler.stop() if sampler else None
    ctx.sync()

    ms_per_step = ms_total / args.steps
    value = flops_per_step(w) / (ms_per_step * 1e-3) / 1e12

    # ---- roofline of the dominant kernel (tcgen05 3xTF32 GEMM): algorithmic flops per launch
    peaks = measured_peaks()
    long_region = ms_total > 1000.0
    bf16_peak = peaks["bf16_sustained"] if long_region else peaks["bf16"]
    peak_3x = bf16_peak / 2.0 / 3.0       # TF32 runs at half the bf16 rate; 3 MMAs per fp32 product
    flops_per_launch = 2.0 * (count if w["sharded"] else m) * n * k
    if w["sharded"] and gemm_launches:
        flops_per_launch = 2.0 * count * n * k * args.steps / gemm_launches     # slabs
    avg_gemm_ms = gemm_ms / max(1, gemm_launches)
    achieved = flops_per_launch / (avg_gemm_ms * 1e-3) / 1e12 if avg_gemm_ms > 0 else 0.0
    alg_bytes = 4.0 * ((count if w["sharded"] else m) * k + k * n + m * n * (2 if beta != 0 else 1))
    traffic = NCU_TRAFFIC_BYTES.get(name)
    roofline = {
        "bound": "tensor", "kernel": "sgemm_tc3x_kernel", "achieved": round(achieved, 2), "peak": round(peak_3x, 2),
        "unit": UNIT, "frac": round(achieved / peak_3x, 4), "traffic": traffic,
        "peak_source": f"{peaks['source']} bf16 {'sustained' if long_region else 'burst'} {bf16_peak} TFLOP/s / 2 (TF32 rate) / 3 (3xTF32)",
        "frac_of_nominal": round(achieved / (2250.0 / 6.0), 4),
        "avg_launch_ms": round(avg_gemm_ms, 4), "launches": gemm_launches,
        "prepass_avg_ms_per_gemm": round(prepass_ms / max(1, gemm_launches), 4),
        "algorithmic_flops_per_launch": flops_per_launch, "algorithmic_bytes_per_gemm": alg_bytes,
        "hbm_gbs_at_algorithmic_bytes": round(alg_bytes / (avg_gemm_ms * 1e-3 + prepass_ms / max(1, gemm_launches) * 1e-3) / 1e9, 1)
        if avg_gemm_ms > 0 else None,
        "frac_of_fp32_simt_peak": round(achieved / 75.0, 3),
    }

    # ---- end to end through the C ABI with pinned HOST buffers (copies inside the timed region)
    e2e = None
    if not args.no_e2e:
        e2e = measure_e2e(ctx, torch, np, w, world, rank, first, count, barrier, max_over_ranks, stream, a, b, c,
                          gather_mode)

    extras = {}
    if world == 1 and not args.no_extras and name == "sgemm_4096_nn_nt_tn_tt":
        del a, b, c
        torch.cuda.empty_cache()
        extras = strong_scaling_base(ctx, torch, stream)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        threads = len(os.sched_getaffinity(0))
        tf, dt, sample, _ = cpu_gemm_rate(w, threads, budget_s=20.0, steps=2, warmup=1)
        cpu = {"value": round(tf, 4), "unit": UNIT, "cores": threads, "kind": "port", "sample": sample}

    if rank == 0:
        line = {
            "metric": METRIC, "value": round(value, 3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": name, "m": m, "n": n, "k": k, "alpha": alpha, "beta": beta,
                       "transposes": ["NT"[ta] + "NT"[tb] for ta, tb in w["cases"]],
                       "arithmetic": "3xTF32 on tcgen05 (hi/lo split), fp32 accumulate in TMEM",
                       "partition": (f"row blocks of A over {world} GPU(s), B replicated, C all-gathered "
                                     + ("by peer stores fused into the GEMM epilogue (NVLink) + NCCL barrier"
                                        if gather_mode == 2 else "with NCCL, slab-pipelined"))
                       if w["sharded"] else "single GPU",
                       "l2": "no flush needed: operands + split planes per GEMM exceed the 126 MB L2 "
                             f"({alg_bytes / 2**20:.0f} MiB operands, {workspace_bytes(count if w['sharded'] else m, n, k) / 2**20:.0f} MiB planes)"},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches),
            "clocks": clocks, "wall_s_timed_region": round(wall, 4),
        }
        line.update(extras)
        print(json.dumps(line), flush=True)
    if gather_mode == 2:
        # unmap the peers' buffers only after every rank has finished using them
        ctx.sync()
        barrier()
        ctx.comm_set_peer_buffers([], 0)
        for r in range(world):
            if r != rank:
                ctx.ipc_close(opened[r])
        barrier()
        ctx.free(c_raw)
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


def measure_e2e(ctx, torch, np, w, world, rank, first, count, barrier, max_over_ranks, stream, a, b, c, gather_mode=1):
    """Same metric through the C ABI with HOST buffers: every step copies its inputs from
    pinned host memory to the device and the step's result back."""
    m, n, k, alpha, beta = w["m"], w["n"], w["k"], w["alpha"], w["beta"]
    rows = count if w["sharded"] else m

    def pinned(nfloats):
        ptr = ctx.host_alloc(nfloats * 4)
        arr = np.frombuffer((ctypes.c_float * nfloats).from_address(ptr), dtype=np.float32)
        return ptr, arr

    pa, ha = pinned(rows * k)
    pb, hb = pinned(k * n)
    pc, hc = pinned(rows * n)
    # host images of the same synthetic operands (device -> host once, outside the timed region)
    ctx.memcpy_d2h(ha, a, ha.nbytes); ctx.memcpy_d2h(hb, b, hb.nbytes)
    from sushiblas_b200.capi import _addr
    c_block = _addr(c) + first * n * 4 if w["sharded"] else _addr(c)      # this rank's rows of C
    ctx.memcpy_d2h(hc, c_block, hc.nbytes)
    ctx.sync()
    steps, warm = (3, 1) if w["sharded"] else (5, 2)

    if w["sharded"]:
        def step():
            ctx.memcpy_h2d(a, ha, ha.nbytes)
            ctx.memcpy_h2d(b, hb, hb.nbytes)
            ctx.sgemm_row_sharded(0, 0, m, n, k, alpha, a, k, b, n, beta, c, n, gather=gather_mode)
            ctx.memcpy_d2h(hc, c_block, hc.nbytes)
        h2d, d2h = ha.nbytes + hb.nbytes, hc.nbytes
    else:
        def step():
            for (ta, tb) in w["cases"]:
                ctx.sgemm_strided_batched_host(ta, tb, m, n, k, alpha, ha, m if ta else k, 0, hb, k if tb else n, 0,
                                               beta, hc, n, 0, 1)
        per = ha.nbytes + hb.nbytes + (hc.nbytes if beta != 0 else 0)
        h2d, d2h = per * len(w["cases"]), hc.nbytes * len(w["cases"])

    for _ in range(warm):
        step()
    ctx.sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e0.record(stream)
    for _ in range(steps):
        step()
    e1.record(stream)
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    barrier()
    ms = max_over_ranks(max(e0.elapsed_time(e1), wall * 1e3)) / steps
    for p in (pa, pb, pc):
        ctx.host_free(p)
    return {"value": round(flops_per_step(w) / (ms * 1e-3) / 1e12, 3), "unit": UNIT,
            "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "ms_per_step": round(ms, 3),
            "steps": steps, "api": "sushi_cuda_sgemm_strided_batched_host" if not w["sharded"]
            else "sushi_cuda_memcpy_h2d + sushi_cuda_sgemm_row_sharded + sushi_cuda_memcpy_d2h"}


def strong_scaling_base(ctx, torch, stream):
    """The 32768^3 NN problem of the multi-GPU runs on one GPU (3 timed steps): the base the
    N > 1 lines are compared with."""
    from sushiblas_b200.capi import workspace_bytes
    n = 32768
    try:
        a = torch.empty(n, n, device="cuda"); b = torch.empty(n, n, device="cuda"); c = torch.empty(n, n, device="cuda")
        ctx.fill_uniform(a, n * n, SEED); ctx.fill_uniform(b, n * n, SEED + 1)
        ctx.reserve_workspace(workspace_bytes(n, n, n))
        ctx.kernel_timing_enable(True)
        ctx.sgemm_row_sharded(0, 0, n, n, n, 1.0, a, n, b, n, 0.0, c, n, gather=True)
        ctx.sync()
        ctx.kernel_timing_read()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(3):
            ctx.sgemm_row_sharded(0, 0, n, n, n, 1.0, a, n, b, n, 0.0, c, n, gather=True)
        e1.record(stream)
        torch.cuda.synchronize()
        gemm_ms, gl, pre_ms, _ = ctx.kernel_timing_read()
        ctx.kernel_timing_enable(False)
        ms = e0.elapsed_time(e1) / 3
        fl = 2.0 * n ** 3
        return {"strong_scaling_base": {"workload": "sgemm_32768_nn_row_sharded", "n_gpus": 1,
                                        "value": round(fl / (ms * 1e-3) / 1e12, 3), "unit": UNIT,
                                        "ms_per_step": round(ms, 3),
                                        "gemm_kernel_tflops": round(fl * 3 / (gemm_ms * 1e-3) / 1e12, 3) if gemm_ms else None,
                                        "prepass_ms_per_step": round(pre_ms / 3, 3)}}
    except Exception as e:   # reported, never hidden
        return {"strong_scaling_base": {"error": str(e)}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None)
    ap.add_argument("--no-extras", action="store_true", help="skip the 32768^3 single-GPU base measurement")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl"],
                    help="multi-GPU exchange of C: peer stores fused into the GEMM epilogue, or slab-pipelined NCCL")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg (profiling runs)")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        log("note: fewer than 3 warm-up steps were requested")
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
