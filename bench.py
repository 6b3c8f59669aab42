#!/usr/bin/env python
"""Benchmark of the fp32 GEMM hot path (one JSON line on stdout, printed by rank 0).

    python bench.py --gpus N --steps K --warmup W            # this library (CUDA, sm_100a)
    python bench.py --impl reference --gpus N ...            # CPU baseline arm (rank 0 only)
    python bench.py --workload NAME ...                      # any workload of the table below

Workloads (synthetic, seeded; shapes and distributions of the specification's five configs):
  sgemm_1024_nn                           M=N=K=1024, alpha=1, beta=0, A, B ~ U[-1,1)
  sgemm_4096_nn_nt_tn_tt   (default N=1)  M=N=K=4096, alpha=1.5, beta=0.5, one step = NN, NT, TN, TT once
                                          each; A, B, C ~ U[-1,1)
  sgemm_batched_256x512_nn_batch_sharded  256 x (512 x 512 x 512), alpha=1, beta=0, A, B ~ N(0,1); batch index
                                          sharded over the ranks, C batches all-gathered
  sgemm_65536x256x4096_nn_row_sharded     A ~ U[-1,1), B ~ N(0, 0.02); row blocks of A over the ranks
  sgemm_32768_nn_row_sharded (default N>1) M=N=K=32768, A, B ~ U[-1,1); row blocks of A over the ranks,
                                          B replicated, C gathered on every rank -- strong scaling
  sgemm_skinny_65536x16x256               deliberately bandwidth-bound shape (tall-and-skinny kernel)
  dgemm_N / ssyrk_N / strsm_N             timing of the widened Level-3 rows (N = matrix order)
Metric: fp32 GEMM TFLOP/s = 2*M*N*K*batch per GEMM / device time, whole job.

After the timed region (never inside it) every rank checks the result it holds: sampled entries and
whole rows of C against float64 dot products of the same inputs, within the stated tolerance
|dC| <= 4*K*2^-24*(|A||B|) + 2^-24*|beta*C| (half of the specification's K budget), and a checksum
of the full C compared across ranks.  A failed check makes the run exit non-zero.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import re
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "fp32_gemm_tflops"
UNIT = "TFLOP/s"
SEED = 20240601
U24 = 2.0 ** -24

# DRAM bytes per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum of one ncu
# capture of that kernel on that workload).  A constant: the bench cannot read DRAM counters itself.
NCU_TRAFFIC_BYTES = {
    # tensor kernel, one launch of 4096^3 with beta != 0: 552.6 MB read + 51.9 MB written (ncu --set full, 2 launches)
    "sgemm_4096_nn_nt_tn_tt": 604.5e6,
}


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
        return self

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
GEMM_WORKLOADS = {
    "sgemm_1024_nn": dict(m=1024, n=1024, k=1024, batch=1, alpha=1.0, beta=0.0, cases=[(0, 0)], shard=None,
                          dist_a=("uniform",), dist_b=("uniform",)),
    "sgemm_4096_nn_nt_tn_tt": dict(m=4096, n=4096, k=4096, batch=1, alpha=1.5, beta=0.5,
                                   cases=[(0, 0), (0, 1), (1, 0), (1, 1)], shard=None,
                                   dist_a=("uniform",), dist_b=("uniform",)),
    "sgemm_batched_256x512_nn_batch_sharded": dict(m=512, n=512, k=512, batch=256, alpha=1.0, beta=0.0, cases=[(0, 0)],
                                                   shard="batch", dist_a=("normal", 1.0), dist_b=("normal", 1.0)),
    "sgemm_65536x256x4096_nn_row_sharded": dict(m=65536, n=256, k=4096, batch=1, alpha=1.0, beta=0.0, cases=[(0, 0)],
                                                shard="rows", dist_a=("uniform",), dist_b=("normal", 0.02)),
    "sgemm_32768_nn_row_sharded": dict(m=32768, n=32768, k=32768, batch=1, alpha=1.0, beta=0.0, cases=[(0, 0)],
                                       shard="rows", dist_a=("uniform",), dist_b=("uniform",)),
    "sgemm_skinny_65536x16x256": dict(m=65536, n=16, k=256, batch=1, alpha=1.0, beta=0.0, cases=[(0, 0)], shard=None,
                                      dist_a=("uniform",), dist_b=("uniform",)),
}
LEVEL3_RE = re.compile(r"^(dgemm|ssyrk|strsm)_(\d+)$")


def workload_for(n_gpus: int, name: str | None):
    if name is None:
        name = "sgemm_4096_nn_nt_tn_tt" if n_gpus == 1 else "sgemm_32768_nn_row_sharded"
    if name not in GEMM_WORKLOADS:
        raise SystemExit(f"unknown workload {name}; choose from {sorted(GEMM_WORKLOADS)} or dgemm_N / ssyrk_N / strsm_N")
    if n_gpus > 1 and not GEMM_WORKLOADS[name]["shard"]:
        raise SystemExit(f"workload {name} does not shard; run it with --gpus 1")
    return name, GEMM_WORKLOADS[name]


def flops_per_step(w):
    return 2.0 * w["m"] * w["n"] * w["k"] * w["batch"] * len(w["cases"])


def config_of(name, w):
    """The `config` object: identical in both arms."""
    return {"workload": name, "m": w["m"], "n": w["n"], "k": w["k"], "batch": w["batch"], "alpha": w["alpha"],
            "beta": w["beta"], "transposes": ["NT"[ta] + "NT"[tb] for ta, tb in w["cases"]]}


# --------------------------------------------------------------------------- seeded generator (host twin)
def _splitmix64(x):
    import numpy as np
    with np.errstate(over="ignore"):
        z = x + np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def uniform_at(seed: int, idx):
    """float64 values of the library's counter-based U[-1,1) generator (sushi_cuda_fill_uniform) at the
    global element indices `idx`: a pure function of (seed, index), so any row or column of a matrix
    can be rebuilt on the host without the matrix."""
    import numpy as np
    idx = np.asarray(idx, dtype=np.uint64)
    key = _splitmix64(np.full(1, seed, dtype=np.uint64))[0]
    u = (_splitmix64(idx ^ key) >> np.uint64(32)).astype(np.uint32) >> np.uint32(8)
    return (u.astype(np.float64) - 8388608.0) * 2.0 ** -23


class GenMatrix:
    """Row-major matrix whose element (r, c) is generator element first_index + r*ld + c."""

    def __init__(self, seed, ld, first_index=0):
        self.seed, self.ld, self.first = seed, ld, first_index

    def block(self, rows, cols):
        import numpy as np
        rows = np.asarray(rows, dtype=np.uint64)[:, None]
        cols = np.asarray(cols, dtype=np.uint64)[None, :]
        return uniform_at(self.seed, np.uint64(self.first) + rows * np.uint64(self.ld) + cols)


class TensorMatrix:
    """Row-major matrix held in a torch tensor (device or host); blocks are read back as float64."""

    def __init__(self, tensor2d, row0=0):
        self.t, self.row0 = tensor2d, row0

    def block(self, rows, cols):
        import numpy as np
        import torch
        r = torch.as_tensor(np.asarray(rows, dtype=np.int64) - self.row0, device=self.t.device)
        sub = self.t.index_select(0, r)
        if not (len(cols) == self.t.shape[1] and int(cols[0]) == 0 and int(cols[-1]) == self.t.shape[1] - 1):
            sub = sub.index_select(1, torch.as_tensor(np.asarray(cols, dtype=np.int64), device=self.t.device))
        return sub.cpu().numpy().astype(np.float64)


def check_gemm(ta, tb, m, n, k, alpha, beta, a_mat, b_mat, c_in_mat, read_c_rows, rng, n_points=64, n_rows=4,
               row_lo=0, row_hi=None, k_chunk=2048):
    """Checks C = alpha*op(A)*op(B) + beta*C_in at `n_points` random entries and `n_rows` whole rows
    (rows drawn from [row_lo, row_hi)) against float64 dot products of the same inputs.
    a_mat / b_mat / c_in_mat: objects with .block(rows, cols) giving the STORED matrices in float64;
    read_c_rows(rows) -> float64 array (len(rows), n) of the result under test.
    Returns (max_ratio, samples): max |dC| / (4*K*2^-24*(|A||B|) + 2^-24*|beta*C_in|), number of entries checked."""
    import numpy as np
    row_hi = m if row_hi is None else row_hi
    if row_hi <= row_lo or n <= 0:
        return 0.0, 0
    ks = np.arange(k)
    al, be = float(np.float32(alpha)), float(np.float32(beta))

    def op_a(rows, kk):          # (len(rows), len(kk))
        return a_mat.block(kk, rows).T if ta else a_mat.block(rows, kk)

    def op_b(kk, cols):          # (len(kk), len(cols))
        return b_mat.block(cols, kk).T if tb else b_mat.block(kk, cols)

    def ratio(got, ref, absab, cin):
        bound = 4.0 * max(k, 1) * U24 * absab + (U24 * np.abs(be * cin) if be != 0.0 else 0.0)
        err = np.abs(got - ref)
        if not np.all(np.isfinite(got)):
            return float("inf")
        with np.errstate(divide="ignore", invalid="ignore"):
            r = np.where(bound > 0, err / bound, np.where(err == 0, 0.0, np.inf))
        return float(r.max(initial=0.0))

    worst, samples = 0.0, 0
    # ---- random entries
    pi = rng.integers(row_lo, row_hi, size=n_points)
    pj = rng.integers(0, n, size=n_points)
    ar = op_a(pi, ks)                                    # points x k
    bc = op_b(ks, pj)                                    # k x points
    ref = al * np.einsum("pk,kp->p", ar, bc)
    absab = np.einsum("pk,kp->p", np.abs(ar), np.abs(bc))
    cin = np.zeros(n_points)
    if be != 0.0:
        cin = np.array([c_in_mat.block([i], [j])[0, 0] for i, j in zip(pi, pj)])
        ref = ref + be * cin
    got_rows = read_c_rows(pi)
    got = got_rows[np.arange(n_points), pj]
    worst = max(worst, ratio(got, ref, absab, cin))
    samples += n_points
    # ---- whole rows (all of op(B), streamed in k chunks)
    if n_rows > 0:
        ri = np.sort(rng.choice(row_hi - row_lo, size=min(n_rows, row_hi - row_lo), replace=False)) + row_lo
        ref = np.zeros((len(ri), n))
        absab = np.zeros((len(ri), n))
        cols = np.arange(n)
        for k0 in range(0, k, k_chunk):
            kk = ks[k0:k0 + k_chunk]
            a_blk, b_blk = op_a(ri, kk), op_b(kk, cols)
            ref += a_blk @ b_blk
            absab += np.abs(a_blk) @ np.abs(b_blk)
        ref *= al
        cin = np.zeros((len(ri), n))
        if be != 0.0:
            cin = c_in_mat.block(ri, cols)
            ref = ref + be * cin
        worst = max(worst, ratio(read_c_rows(ri), ref, absab, cin))
        samples += len(ri) * n
    return worst, samples


def device_checksum(torch, ctx, ptr_or_tensor, nfloats, device):
    """Order-dependent 128-bit checksum of `nfloats` floats in device memory (bit patterns), computed on
    the device in 64 Mi-element chunks: (sum of words, sum of words * position weight), both mod 2^64."""
    from sushiblas_b200.capi import _addr
    base = _addr(ptr_or_tensor)
    chunk = 1 << 26
    scratch = torch.empty(min(chunk, nfloats), dtype=torch.int32, device=device)
    weights = (torch.arange(min(chunk, nfloats), device=device, dtype=torch.int64) % 65521) + 1
    s0 = s1 = 0
    for off in range(0, nfloats, chunk):
        cnt = min(chunk, nfloats - off)
        ctx.memcpy_d2d(scratch, base + off * 4, cnt * 4)
        w = scratch[:cnt].to(torch.int64)
        s0 = (s0 + int(w.sum().item())) & 0xFFFFFFFFFFFFFFFF
        s1 = (s1 * 31 + int((w * weights[:cnt]).sum().item())) & 0xFFFFFFFFFFFFFFFF
    return f"{s0:016x}{s1:016x}"


# --------------------------------------------------------------------------- CPU arm
def cpu_gemm_rate(w, threads, budget_s, steps, warmup):
    """Times MKL sgemm (torch CPU) on a bounded sample of the workload.
    Returns (TFLOP/s, seconds per step, sample description, sample flops)."""
    import torch
    from oracle import ref_gemm as og

    torch.set_num_threads(threads)
    m, n, k, batch = w["m"], w["n"], w["k"], w["batch"]
    g = torch.Generator().manual_seed(SEED)
    # probe the host's sgemm rate on a small problem to size the sample
    pa = torch.empty(1024, 2048).uniform_(-1, 1, generator=g)
    pb = torch.empty(2048, 2048).uniform_(-1, 1, generator=g)
    pc = torch.empty(1024, 2048)
    og.mkl_proxy_gemm(0, 0, 1.0, pa, pb, 0.0, pc)
    t0 = time.perf_counter()
    og.mkl_proxy_gemm(0, 0, 1.0, pa, pb, 0.0, pc)
    rate = 2.0 * 1024 * 2048 * 2048 / max(time.perf_counter() - t0, 1e-6)
    per_step_budget = budget_s / max(1, steps + warmup)
    if batch > 1:
        # a bounded number of batch entries, each a full m x n x k product
        nb = int(per_step_budget * rate / (2.0 * m * n * k))
        nb = max(1, min(batch, nb))
        a = torch.empty(nb, m, k).normal_(0, 1, generator=g)
        b = torch.empty(nb, k, n).normal_(0, 1, generator=g)
        c = torch.empty(nb, m, n)
        flops = 2.0 * m * n * k * nb

        def step():
            for i in range(nb):
                og.mkl_proxy_gemm(0, 0, w["alpha"], a[i], b[i], w["beta"], c[i])
        what = f"{nb} of {batch} batch entries per step"
    else:
        # rows of A (and C) per sampled GEMM so that warmup+steps fit the budget
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
        what = f"{rows} of {m} rows of A/C per GEMM x {len(w['cases'])} GEMMs per step, full N={n} K={k}"

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    sample = (f"MKL sgemm via torch CPU (oneMKL proxy for the reference's oneMKL call), {threads} threads, "
              f"{what}, {steps} timed steps")
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
        "config": config_of(name, w),
        "notes": {"stand_in": "the reference's SYCL/oneMKL build is unavailable on this box; MKL sgemm (torch CPU) stands in"},
        "cpu_baseline": {"value": round(tf, 4), "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": round(tf, 4), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU arm
class Harness:
    """Process-wide set-up shared by every measurement of one bench run."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        from sushiblas_b200 import SushiCuda, load_library
        self.torch, self.dist = torch, dist
        self.rank, self.world, self.local_rank = env_rank()
        if self.world != args.gpus:
            raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={self.world}: launch with torch.distributed.run")
        if not torch.cuda.is_available():
            raise SystemExit("no CUDA device: this library has no CPU fallback")
        load_library()                       # fails loudly if the CUDA extension was not built
        torch.cuda.set_device(self.local_rank)
        self.device = torch.device("cuda", self.local_rank)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.device)
        self.ctx = SushiCuda([self.local_rank])
        # one explicit stream for torch's events/copies and the library's kernels (torch's default
        # stream has handle 0, which the C ABI reads as "use the context's own stream")
        self.stream = torch.cuda.Stream(self.device)
        torch.cuda.set_stream(self.stream)
        self.ctx.set_stream(self.stream.cuda_stream)
        if self.world > 1:
            ids = [self.ctx.comm_unique_id() if self.rank == 0 else None]
            dist.broadcast_object_list(ids, src=0)
            self.ctx.comm_init_rank(ids[0], self.world, self.rank)
        self._scrub = None

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()

    def max_over_ranks(self, x: float) -> float:
        if self.world == 1:
            return x
        t = self.torch.tensor([x], device=self.device, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def flush_l2(self):
        """Write a buffer twice the size of L2, then read it back: the write displaces the operands, the
        read leaves L2 full of clean lines, so the next call does not pay for write-backs."""
        if self._scrub is None:
            self._scrub = self.torch.empty(256 << 20, dtype=self.torch.uint8, device=self.device)
        self._scrub.fill_(1)
        self._scrub.max()

    def close(self):
        self.ctx.close()
        if self.world > 1:
            self.dist.destroy_process_group()


class GemmProblem:
    """Device-resident operands of one GEMM workload on this rank, the step that multiplies them, and
    the check of the result."""

    def __init__(self, h: Harness, name, w, gather="fused"):
        from sushiblas_b200.capi import partition
        torch, ctx = h.torch, h.ctx
        self.h, self.name, self.w = h, name, w
        m, n, k, batch = w["m"], w["n"], w["k"], w["batch"]
        self.shard = w["shard"]
        self.opened = []
        self.c_raw = None
        self.gather_mode = 1
        dev = h.device
        if self.shard == "batch":
            self.first, self.count = partition(batch, h.world, h.rank)
            self.a = torch.empty(max(self.count, 1), m, k, device=dev)
            self.b = torch.empty(max(self.count, 1), k, n, device=dev)
            if h.world > 1 and gather == "fused":
                self._register_peer_c(batch * m * n * 4)
            else:
                self.c = torch.empty(batch, m, n, device=dev)
        else:
            self.first, self.count = partition(m, h.world, h.rank) if self.shard == "rows" else (0, m)
            self.a = torch.empty(self.count, k, device=dev)          # square when transposed cases exist
            self.b = torch.empty(k, n, device=dev)
            if h.world > 1 and gather == "fused":
                self._register_peer_c(m * n * 4)
            else:
                self.c = torch.empty(m, n, device=dev)
        self.fill_inputs()
        self.fill_c()
        ctx.sync()

    def _register_peer_c(self, nbytes):
        """C lives in a plain cudaMalloc block so that it can be mapped into the peers (CUDA IPC): the GEMM
        epilogue then stores finished tiles straight into every rank's C over NVLink."""
        h, ctx = self.h, self.h.ctx
        self.c_raw = ctx.malloc(nbytes)
        handles = [None] * h.world
        h.dist.all_gather_object(handles, ctx.ipc_export(self.c_raw))
        self.opened = [ctx.ipc_open(handles[r]) if r != h.rank else None for r in range(h.world)]
        ctx.comm_set_peer_buffers([self.c_raw if r == h.rank else self.opened[r] for r in range(h.world)], nbytes)
        self.c = self.c_raw
        self.gather_mode = 2

    # ---- inputs
    def _fill(self, t, dist_spec, seed, first_index):
        torch = self.h.torch
        if dist_spec[0] == "uniform":
            self.h.ctx.fill_uniform(t, t.numel(), seed, first_index=first_index)
        else:
            # normal(0, std): torch's device generator, seeded per (tensor, first element) so that a shard
            # holds the same values whatever the number of ranks is not required -- the check reads the
            # operands back from the device
            g = torch.Generator(device=self.h.device).manual_seed(seed * 1000003 + first_index % 1000003)
            with torch.cuda.stream(self.h.stream):
                t.normal_(0.0, dist_spec[1], generator=g)

    def fill_inputs(self):
        w = self.w
        if self.shard == "batch":
            self._fill(self.a, w["dist_a"], SEED, self.first * w["m"] * w["k"])
            self._fill(self.b, w["dist_b"], SEED + 1, self.first * w["k"] * w["n"])
        else:
            self._fill(self.a, w["dist_a"], SEED, self.first * w["k"])
            self._fill(self.b, w["dist_b"], SEED + 1, 0)

    def fill_c(self):
        w = self.w
        self.h.ctx.fill_uniform(self.c, w["m"] * w["n"] * w["batch"], SEED + 2)

    # ---- the step
    def run_case(self, ta, tb):
        w, ctx = self.w, self.h.ctx
        m, n, k = w["m"], w["n"], w["k"]
        if self.shard == "batch":
            ctx.sgemm_batch_sharded(ta, tb, m, n, k, w["alpha"], self.a, k, m * k, self.b, n, k * n, w["beta"], self.c, n,
                                    m * n, w["batch"], gather=self.gather_mode if self.h.world > 1 else 0)
        elif self.shard == "rows":
            ctx.sgemm_row_sharded(ta, tb, m, n, k, w["alpha"], self.a, k, self.b, n, w["beta"], self.c, n,
                                  gather=self.gather_mode)
        else:
            ctx.sgemm(ta, tb, m, n, k, w["alpha"], self.a, m if ta else k, self.b, k if tb else n, w["beta"], self.c, n)

    def step(self):
        for (ta, tb) in self.w["cases"]:
            self.run_case(ta, tb)

    # ---- the check (outside every timed region)
    def read_c_rows(self, rows):
        """Rows of the (batch*m) x n result matrix as float64."""
        import numpy as np
        from sushiblas_b200.capi import _addr
        n = self.w["n"]
        out = np.empty((len(rows), n), dtype=np.float32)
        base = _addr(self.c)
        for i, r in enumerate(rows):
            self.h.ctx.memcpy_d2h(out[i], base + int(r) * n * 4, n * 4)
        self.h.ctx.sync()
        return out.astype(np.float64)

    def check(self):
        """Runs every case once more on freshly filled C and checks the result this rank holds."""
        import numpy as np
        w, h = self.w, self.h
        m, n, k, batch = w["m"], w["n"], w["k"], w["batch"]
        rng = np.random.default_rng(SEED + 17 * h.rank)
        worst, samples, sums = 0.0, 0, []
        for (ta, tb) in w["cases"]:
            self.fill_c()
            h.ctx.sync()
            h.barrier()
            self.run_case(ta, tb)
            h.ctx.sync()
            h.barrier()
            if self.shard == "batch":
                # this rank's operands cover its own batch entries; the others' results are covered by the checksum
                for bi in rng.integers(0, max(self.count, 1), size=min(4, self.count)):
                    g = self.first + int(bi)
                    r, s = check_gemm(ta, tb, m, n, k, w["alpha"], w["beta"], TensorMatrix(self.a[bi]), TensorMatrix(self.b[bi]),
                                      GenMatrix(SEED + 2, n, g * m * n), lambda rows, g=g: self.read_c_rows(np.asarray(rows) + g * m),
                                      rng, n_points=32, n_rows=2)
                    worst, samples = max(worst, r), samples + s
            else:
                a_mat = (GenMatrix(SEED, k) if w["dist_a"][0] == "uniform" and not ta
                         else GenMatrix(SEED, m) if w["dist_a"][0] == "uniform" else TensorMatrix(self.a, self.first))
                b_mat = TensorMatrix(self.b)
                lo, hi = (0, m) if w["dist_a"][0] == "uniform" else (self.first, self.first + self.count)
                r, s = check_gemm(ta, tb, m, n, k, w["alpha"], w["beta"], a_mat, b_mat, GenMatrix(SEED + 2, n),
                                  self.read_c_rows, rng, n_points=64, n_rows=4 if h.world == 1 else 1, row_lo=lo, row_hi=hi)
                worst, samples = max(worst, r), samples + s
            sums.append(device_checksum(h.torch, h.ctx, self.c, m * n * batch, h.device))
        gathered = [None] * h.world
        if h.world > 1:
            h.dist.all_gather_object(gathered, (worst, samples, sums))
        else:
            gathered = [(worst, samples, sums)]
        identical = all(g[2] == gathered[0][2] for g in gathered)
        max_ratio = max(g[0] for g in gathered)
        ok = bool(identical and max_ratio <= 1.0)
        return {"ok": ok, "max_ratio": round(max_ratio, 4), "samples": int(sum(g[1] for g in gathered)),
                "ranks_identical": identical, "checksum": gathered[0][2][-1],
                "tolerance": "|dC| <= 4*K*2^-24*(|A||B|) + 2^-24*|beta*C_in| against float64 dot products "
                             "(half of the specification's K budget)",
                "what": "per rank and case: 64 random entries + whole rows of the C the rank holds after one more run "
                        "on freshly filled C; checksum of the full C compared across ranks"}

    def release(self):
        h = self.h
        if self.gather_mode == 2:
            # unmap the peers' buffers only after every rank has finished using them
            h.ctx.sync()
            h.barrier()
            h.ctx.comm_set_peer_buffers([], 0)
            for r in range(h.world):
                if r != h.rank:
                    h.ctx.ipc_close(self.opened[r])
            h.barrier()
            h.ctx.free(self.c_raw)
        self.a = self.b = self.c = None
        h.torch.cuda.empty_cache()


def time_steps(h: Harness, step, steps, warmup, sample_clocks=True):
    """W warm-up steps, then K steps between CUDA events on the launching stream, barrier + synchronize on
    both sides, maximum over ranks.  Returns a dict with the timing and what the library recorded."""
    torch, ctx = h.torch, h.ctx
    for _ in range(warmup):
        step()
    ctx.sync()
    sampler = ClockSampler(h.local_rank).start() if (sample_clocks and h.rank == 0) else None
    if sampler:
        time.sleep(0.25)
    ctx.kernel_timing_enable(True)
    launches0 = ctx.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    h.barrier()
    torch.cuda.synchronize()
    wall0 = time.perf_counter()
    e0.record(h.stream)
    for _ in range(steps):
        step()
    e1.record(h.stream)
    torch.cuda.synchronize()
    h.barrier()
    wall = time.perf_counter() - wall0
    ms_total = h.max_over_ranks(e0.elapsed_time(e1))
    gemm_ms, gemm_launches, prepass_ms, prepass_launches = ctx.kernel_timing_read()
    ctx.kernel_timing_enable(False)
    launches = ctx.launch_count() - launches0
    clocks = sampler.stop() if sampler else None
    ctx.sync()
    return dict(ms_total=ms_total, ms_per_step=ms_total / steps, wall=wall, gemm_ms=gemm_ms, gemm_launches=gemm_launches,
                prepass_ms=prepass_ms, prepass_launches=prepass_launches, launches=launches, clocks=clocks)


def time_calls_flushed(h: Harness, fn, steps, warmup):
    """Per-call CUDA-event times with L2 flushed before every call (for problems that fit in L2)."""
    torch = h.torch
    times = []
    for i in range(warmup + steps):
        h.flush_l2()
        h.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(h.stream)
        fn()
        e1.record(h.stream)
        e1.synchronize()
        if i >= warmup:
            times.append(h.max_over_ranks(e0.elapsed_time(e1)))
    return statistics.median(times), min(times)


def roofline_of(name, w, count_rows, t, peaks, steps):
    """Roofline object of the dominant kernel from the library's own CUDA-event records."""
    m, n, k, batch, beta = w["m"], w["n"], w["k"], w["batch"], w["beta"]
    long_region = t["ms_total"] > 1000.0
    bf16_peak = peaks["bf16_sustained"] if long_region else peaks["bf16"]
    peak_3x = bf16_peak / 2.0 / 3.0       # TF32 runs at half the bf16 rate; 3 MMAs per fp32 product
    gl = max(1, t["gemm_launches"])
    flops_per_launch = 2.0 * count_rows * n * k * batch * len(w["cases"]) * steps / gl
    avg_gemm_ms = t["gemm_ms"] / gl
    achieved = flops_per_launch / (avg_gemm_ms * 1e-3) / 1e12 if avg_gemm_ms > 0 else 0.0
    alg_bytes = 4.0 * batch * (count_rows * k + k * n + count_rows * n * (2 if beta != 0 else 1))
    prepass_per_gemm = t["prepass_ms"] / gl
    traffic = NCU_TRAFFIC_BYTES.get(name)
    return {
        "bound": "tensor", "kernel": "sgemm_tc3x_kernel", "achieved": round(achieved, 2), "peak": round(peak_3x, 2),
        "unit": UNIT, "frac": round(achieved / peak_3x, 4), "traffic": traffic,
        "traffic_source": "constant typed into bench.py from an ncu capture of this kernel on this workload (dram__bytes_read.sum + dram__bytes_write.sum per launch); not measured by this run" if traffic else None,
        "peak_source": f"{peaks['source']} bf16 {'sustained' if long_region else 'burst'} {bf16_peak} TFLOP/s / 2 (TF32 rate) / 3 (3xTF32)",
        "frac_of_nominal": round(achieved / (2250.0 / 6.0), 4),
        "avg_launch_ms": round(avg_gemm_ms, 4), "launches": t["gemm_launches"],
        "prepass_avg_ms_per_gemm": round(prepass_per_gemm, 4),
        "algorithmic_flops_per_launch": flops_per_launch, "algorithmic_bytes_per_gemm": alg_bytes,
        "hbm_gbs_at_algorithmic_bytes": round(alg_bytes / ((avg_gemm_ms + prepass_per_gemm) * 1e-3) / 1e9, 1) if avg_gemm_ms > 0 else None,
        "frac_of_hbm_peak": round(alg_bytes / ((avg_gemm_ms + prepass_per_gemm) * 1e-3) / 1e9 / peaks["hbm_gbs"], 4) if avg_gemm_ms > 0 else None,
        "frac_of_fp32_simt_peak": round(achieved / 75.0, 3),
    }


def run_ours(args):
    import numpy as np
    h = Harness(args)
    torch, ctx = h.torch, h.ctx
    name, w = workload_for(args.gpus, args.workload)
    prob = GemmProblem(h, name, w, gather=args.gather)
    t = time_steps(h, prob.step, args.steps, args.warmup)
    value = flops_per_step(w) / (t["ms_per_step"] * 1e-3) / 1e12
    peaks = measured_peaks()
    count_rows = prob.count if prob.shard == "rows" else w["m"]
    if prob.shard == "batch":
        w_local = dict(w, batch=prob.count)
        roofline = roofline_of(name, w_local, w["m"], t, peaks, args.steps)
    else:
        roofline = roofline_of(name, w, count_rows, t, peaks, args.steps)
    if name == "sgemm_skinny_65536x16x256":
        roofline.update(bound="hbm", kernel="sgemm_skinny_kernel", unit="GB/s", peak=peaks["hbm_gbs"],
                        achieved=roofline["hbm_gbs_at_algorithmic_bytes"], frac=roofline["frac_of_hbm_peak"],
                        peak_source=f"{peaks['source']} copy bandwidth")

    check = None if args.no_check else prob.check()

    # ---- end to end through the C ABI with pinned HOST buffers (copies inside the timed region)
    e2e = None
    if not args.no_e2e:
        e2e = measure_e2e(h, prob, np)

    extras = {}
    if h.world == 1 and not args.no_extras and name == "sgemm_4096_nn_nt_tn_tt":
        prob.release()
        extras["configs"] = other_configs(h, peaks)
        extras["tf32_ceiling"] = tf32_ceiling(h)
        extras.update(strong_scaling_base(h))
        prob = None

    cpu = None
    if h.rank == 0 and h.world == 1 and not args.no_cpu:
        threads = len(os.sched_getaffinity(0))
        tf, dt, sample, _ = cpu_gemm_rate(w, threads, budget_s=20.0, steps=2, warmup=1)
        cpu = {"value": round(tf, 4), "unit": UNIT, "cores": threads, "kind": "port", "sample": sample}

    if h.rank == 0:
        gathered_by = ("peer stores fused into the GEMM epilogue (NVLink) + NCCL barrier" if args.gather == "fused"
                       else "NCCL, slab-pipelined")
        line = {
            "metric": METRIC, "value": round(value, 3), "unit": UNIT, "n_gpus": h.world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(t["ms_per_step"], 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_of(name, w),
            "notes": {"arithmetic": "3xTF32 on tcgen05 (hi/lo split), fp32 accumulate in TMEM",
                      "partition": (f"row blocks of A over {h.world} GPU(s), B replicated, C gathered by {gathered_by}"
                                    if w["shard"] == "rows" else
                                    f"batch index over {h.world} GPU(s), C batches gathered with NCCL" if w["shard"] == "batch"
                                    else "single GPU"),
                      "l2": ("operands of one GEMM exceed the 126 MB L2, no flush between steps"
                             if 4.0 * w["batch"] * (w["m"] * w["k"] + w["k"] * w["n"] + w["m"] * w["n"]) > 126e6 * 1.5
                             else "working set fits in L2 and steps run back to back: see the flushed per-call time in `flushed`"),
                      "n1_vs_n": "the default N = 1 workload (4096^3) differs from the default N > 1 workload (32768^3): "
                                 "compare N > 1 values with `strong_scaling_base` of the N = 1 line"},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "check": check, "gpu_launches": int(t["launches"]),
            "clocks": t["clocks"], "wall_s_timed_region": round(t["wall"], 4),
        }
        line.update(extras)
        print(json.dumps(line), flush=True)
    if prob is not None:
        prob.release()
    h.close()
    if check is not None and not check["ok"]:
        log("CHECK FAILED:", check)
        sys.exit(3)


def measure_e2e(h: Harness, prob: GemmProblem, np):
    """Same metric through the C ABI with HOST buffers: every step copies its inputs from pinned host
    memory to the device and the step's result back, inside the timed region."""
    from sushiblas_b200.capi import _addr, partition
    torch, ctx, w = h.torch, h.ctx, prob.w
    m, n, k, batch, alpha, beta = w["m"], w["n"], w["k"], w["batch"], w["alpha"], w["beta"]

    def pinned(nfloats):
        ptr = ctx.host_alloc(nfloats * 4)
        arr = np.frombuffer((ctypes.c_float * nfloats).from_address(ptr), dtype=np.float32)
        return ptr, arr

    if prob.shard == "batch":
        # each rank stages its own batch entries and reads its own results back
        cnt = prob.count
        pa, ha = pinned(max(cnt, 1) * m * k); pb, hb = pinned(max(cnt, 1) * k * n); pc, hc = pinned(max(cnt, 1) * m * n)
        ctx.memcpy_d2h(ha, prob.a, ha.nbytes); ctx.memcpy_d2h(hb, prob.b, hb.nbytes)
        ctx.sync()

        def step():
            if cnt:
                ctx.sgemm_strided_batched_host(0, 0, m, n, k, alpha, ha, k, m * k, hb, n, k * n, beta, hc, n, m * n, cnt)
        h2d, d2h = ha.nbytes + hb.nbytes, hc.nbytes
        api = "sushi_cuda_sgemm_strided_batched_host on this rank's batch entries"
        steps, warm = 5, 2
    elif prob.shard == "rows":
        rows = prob.count
        # every rank uploads its rows of A and its share of B's k rows (the rest of B arrives over NVLink) and
        # reads its rows of C back; the device buffers of the device-timed run serve as the call's scratch.  Only
        # the rank's share of B exists on its host: the call is given the address the whole B would start at.
        b_first, b_rows = partition(k, h.world, h.rank)
        pa, ha = pinned(max(rows, 1) * k); pb, hb = pinned(max(b_rows, 1) * n); pc, hc = pinned(max(rows, 1) * n)
        ctx.memcpy_d2h(ha, prob.a, ha.nbytes)
        ctx.memcpy_d2h(hb, _addr(prob.b) + b_first * n * 4, b_rows * n * 4)
        ctx.sync()
        c_block = _addr(prob.c) + prob.first * n * 4
        b_host = pb - b_first * n * 4

        def step():
            ctx.sgemm_row_sharded_host(0, 0, m, n, k, alpha, ha, k, b_host, n, beta, hc, n, prob.a, prob.b, c_block)
        h2d, d2h = ha.nbytes + b_rows * n * 4 + (hc.nbytes if beta != 0 else 0), hc.nbytes
        api = "sushi_cuda_sgemm_row_sharded_host (each rank's host receives its rows of C)"
        steps, warm = (3, 1) if m * n * k > 1e12 else (5, 2)
    else:
        pa, ha = pinned(m * k); pb, hb = pinned(k * n); pc, hc = pinned(m * n)
        ctx.memcpy_d2h(ha, prob.a, ha.nbytes); ctx.memcpy_d2h(hb, prob.b, hb.nbytes); ctx.memcpy_d2h(hc, prob.c, hc.nbytes)
        ctx.sync()

        def step():
            for (ta, tb) in w["cases"]:
                ctx.sgemm_strided_batched_host(ta, tb, m, n, k, alpha, ha, m if ta else k, 0, hb, k if tb else n, 0,
                                               beta, hc, n, 0, 1)
        per = ha.nbytes + hb.nbytes + (hc.nbytes if beta != 0 else 0)
        h2d, d2h = per * len(w["cases"]), hc.nbytes * len(w["cases"])
        api = "sushi_cuda_sgemm_strided_batched_host"
        steps, warm = 5, 2

    for _ in range(warm):
        step()
    ctx.sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    h.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e0.record(h.stream)
    for _ in range(steps):
        step()
    e1.record(h.stream)
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    h.barrier()
    ms = h.max_over_ranks(max(e0.elapsed_time(e1), wall * 1e3)) / steps
    for p in (pa, pb, pc):
        ctx.host_free(p)
    return {"value": round(flops_per_step(w) / (ms * 1e-3) / 1e12, 3), "unit": UNIT,
            "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "ms_per_step": round(ms, 3),
            "steps": steps, "api": api}


def other_configs(h: Harness, peaks):
    """The specification's other single-GPU configs (and the bandwidth-bound shape), each timed per call
    with L2 flushed before the call, plus its check: what the driver's default run would otherwise not see."""
    out = {}
    for name in ("sgemm_1024_nn", "sgemm_batched_256x512_nn_batch_sharded", "sgemm_65536x256x4096_nn_row_sharded",
                 "sgemm_skinny_65536x16x256"):
        w = GEMM_WORKLOADS[name]
        try:
            prob = GemmProblem(h, name, w)
            h.ctx.kernel_timing_enable(True)
            med, best = time_calls_flushed(h, prob.step, steps=20, warmup=3)
            gemm_ms, gl, pre_ms, _ = h.ctx.kernel_timing_read()
            h.ctx.kernel_timing_enable(False)
            fl = flops_per_step(w)
            alg_bytes = 4.0 * w["batch"] * (w["m"] * w["k"] + w["k"] * w["n"] + w["m"] * w["n"])
            kernel_ms = gemm_ms / max(1, gl)
            entry = {"config": config_of(name, w), "ms_median": round(med, 4), "ms_best": round(best, 4),
                     "value": round(fl / (med * 1e-3) / 1e12, 2), "unit": UNIT, "kernel_ms": round(kernel_ms, 4),
                     "prepass_ms": round(pre_ms / max(1, gl), 4), "steps": 20, "l2": "flushed before every call",
                     "frac_of_3xtf32_peak": round(fl / (med * 1e-3) / 1e12 / (peaks["bf16"] / 6.0), 4),
                     "hbm_gbs_at_algorithmic_bytes": round(alg_bytes / (med * 1e-3) / 1e9, 1),
                     "frac_of_hbm_peak": round(alg_bytes / (med * 1e-3) / 1e9 / peaks["hbm_gbs"], 4),
                     "check": prob.check()}
            prob.release()
        except Exception as e:   # reported, never hidden
            entry = {"error": repr(e)}
        out[name] = entry
    return out


def tf32_ceiling(h: Harness):
    """MMA rate of the same tensor-core kernel when it issues ONE TF32 MMA per product (the hi*hi term alone; a
    TF32-accurate result, used for nothing else) and when it issues the regular three: what the tensor pipe is seen to
    sustain on this GPU, to set beside the "bf16 peak / 2" assumed for the TF32 rate in the roofline denominator."""
    torch, ctx = h.torch, h.ctx
    if not hasattr(ctx, "sgemm_tf32_probe"):
        return None
    n = 8192
    try:
        a = torch.empty(n, n, device=h.device); b = torch.empty(n, n, device=h.device); c = torch.empty(n, n, device=h.device)
        ctx.fill_uniform(a, n * n, SEED); ctx.fill_uniform(b, n * n, SEED + 1)
        out = {}
        for label, products in (("tf32_x1", 1), ("tf32_x3", 3)):
            # the library's own CUDA events around the GEMM kernel alone (the operands' pre-pass is not part of the rate)
            for _ in range(3):
                ctx.sgemm_tf32_probe(0, 1, n, n, n, a, n, b, n, c, n, products)
            ctx.sync()
            ctx.kernel_timing_enable(True)
            for _ in range(10):
                ctx.sgemm_tf32_probe(0, 1, n, n, n, a, n, b, n, c, n, products)
            ctx.sync()
            gemm_ms, gemm_launches, _, _ = ctx.kernel_timing_read()
            ctx.kernel_timing_enable(False)
            ms = gemm_ms / max(1, gemm_launches)
            out[label] = {"kernel_ms": round(ms, 4), "mma_tflops": round(2.0 * n ** 3 * products / (ms * 1e-3) / 1e12, 1)}
        out["shape"] = f"{n}^3 NT"
        out["tf32_mma_tflops_sustained"] = out["tf32_x3"]["mma_tflops"]
        out["note"] = ("MMA work per second of the same kernel with one and with three MMAs per product; with one the kernel is "
                       "bound by feeding its stages (same bytes per stage), so the three-product run is the measured lower bound of the "
                       "TF32 tensor rate: compare it with the bf16 / 2 assumed by roofline.peak_source")
        del a, b, c
        torch.cuda.empty_cache()
        return out
    except Exception as e:
        return {"error": repr(e)}


def strong_scaling_base(h: Harness):
    """The 32768^3 NN problem of the multi-GPU runs on one GPU (10 timed steps, own clock sample): the base
    the N > 1 lines are compared with."""
    name = "sgemm_32768_nn_row_sharded"
    w = GEMM_WORKLOADS[name]
    try:
        prob = GemmProblem(h, name, w)
        t = time_steps(h, prob.step, steps=10, warmup=1)
        fl = flops_per_step(w)
        check = prob.check()
        prob.release()
        return {"strong_scaling_base": {"workload": name, "n_gpus": 1, "value": round(fl / (t["ms_per_step"] * 1e-3) / 1e12, 3),
                                        "unit": UNIT, "ms_per_step": round(t["ms_per_step"], 3), "steps": 10,
                                        "gemm_kernel_tflops": round(fl * 10 / (t["gemm_ms"] * 1e-3) / 1e12, 3) if t["gemm_ms"] else None,
                                        "prepass_ms_per_step": round(t["prepass_ms"] / 10, 3), "clocks": t["clocks"],
                                        "check": check}}
    except Exception as e:   # reported, never hidden
        return {"strong_scaling_base": {"error": repr(e)}}


# --------------------------------------------------------------------------- Level-3 rows next to the GEMM
def run_level3(args, op, n):
    """Timing of fp64 GEMM / SYRK / TRSM of order n (one JSON line; CUDA events per call, L2 flushed)."""
    h = Harness(args)
    torch, ctx = h.torch, h.ctx
    dev = h.device
    lines = {}
    if op == "dgemm":
        a = torch.rand(n, n, device=dev, dtype=torch.float64); b = torch.rand(n, n, device=dev, dtype=torch.float64)
        c = torch.zeros(n, n, device=dev, dtype=torch.float64)
        for (ta, tb) in ((0, 0), (0, 1), (1, 0), (1, 1)):
            med, best = time_calls_flushed(h, lambda: ctx.dgemm(ta, tb, n, n, n, 1.0, a, n, b, n, 0.0, c, n), args.steps, args.warmup)
            lines["NT"[ta] + "NT"[tb]] = {"ms_median": round(med, 4), "ms_best": round(best, 4),
                                          "tflops": round(2.0 * n ** 3 / (med * 1e-3) / 1e12, 2)}
        flops = 2.0 * n ** 3
    elif op == "ssyrk":
        a = torch.rand(n, n, device=dev); c = torch.zeros(n, n, device=dev)
        for trans in (0, 1):
            med, best = time_calls_flushed(h, lambda: ctx.ssyrk(0, trans, n, n, 1.0, a, n, 0.0, c, n), args.steps, args.warmup)
            lines["trans" if trans else "notrans"] = {"ms_median": round(med, 4), "ms_best": round(best, 4),
                                                      "tflops": round(1.0 * n ** 3 / (med * 1e-3) / 1e12, 2)}
        flops = 1.0 * n ** 3
    else:
        a = torch.rand(n, n, device=dev) * 0.5 / n + torch.eye(n, device=dev) * 4.0
        b0 = torch.rand(n, n, device=dev); b = b0.clone()
        for (left, upper, trans) in ((1, 0, 0), (1, 1, 0), (0, 0, 0), (1, 0, 1)):
            def call():
                b.copy_(b0)
                ctx.strsm(left, upper, trans, 0, n, n, 1.0, a, n, b, n)
            med, best = time_calls_flushed(h, call, args.steps, args.warmup)
            lines[f"left{left}_upper{upper}_trans{trans}"] = {"ms_median": round(med, 4), "ms_best": round(best, 4),
                                                              "tflops": round(1.0 * n ** 3 / (med * 1e-3) / 1e12, 2),
                                                              "note": "includes a device copy of B (n^2 floats) per call"}
        flops = 1.0 * n ** 3
    first = next(iter(lines.values()))
    line = {"metric": f"{op}_tflops", "value": first["tflops"], "unit": UNIT, "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": first["ms_median"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f64" if op == "dgemm" else "f32", "data": "synthetic",
            "config": {"workload": f"{op}_{n}", "n": n}, "cases": lines, "flops_per_call": flops,
            "notes": {"l2": "flushed before every call"}, "gpu_launches": int(ctx.launch_count())}
    print(json.dumps(line), flush=True)
    h.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None)
    ap.add_argument("--no-extras", action="store_true", help="skip the other configs and the 32768^3 single-GPU base")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-check", action="store_true", help="skip the post-timing result check (profiling runs)")
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl"],
                    help="multi-GPU exchange of C: peer stores fused into the GEMM epilogue, or slab-pipelined NCCL")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg (profiling runs)")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        log("note: fewer than 3 warm-up steps were requested")
    lv3 = LEVEL3_RE.match(args.workload or "")
    if args.impl == "reference":
        run_reference(args)
    elif lv3:
        run_level3(args, lv3.group(1), int(lv3.group(2)))
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
