"""Timing of the Level-3 rows next to the fp32 GEMM: fp64 GEMM, TRSM, SYRK, and of a deliberately
bandwidth-bound fp32 GEMM shape (65536 x 16 x 256, served by the FFMA kernel).

    python -m sushiblas_b200.level3_bench [--op dgemm|strsm|ssyrk|skinny|activation|all] [--size N] [--steps K] [--warmup W] [--library]

One JSON line per (op, case): CUDA-event time of each call on the launching stream (median and
best of K calls after W warm-up calls), inputs resident in HBM, L2 flushed between calls by
writing and re-reading a 256 MiB buffer.  `--library` adds the time of torch's own routine for the same problem
(cuBLAS) on the same GPU as context; it is not part of the product path.  Needs a CUDA device:
there is no CPU fallback.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics


def _hbm_peak_gbs():
    """Measured copy bandwidth of this pool's GPUs when the file is present, else the documented fallback."""
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def _time_calls(torch, stream, fn, reset, flush, steps, warmup):
    times = []
    for i in range(warmup + steps):
        reset()
        flush()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        fn()
        e1.record(stream)
        e1.synchronize()
        if i >= warmup:
            times.append(e0.elapsed_time(e1))
    return statistics.median(times), min(times)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="all", choices=["dgemm", "strsm", "ssyrk", "skinny", "activation", "all"])
    ap.add_argument("--size", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--library", action="store_true")
    args = ap.parse_args(argv)

    import torch
    from sushiblas_b200 import SushiCuda, load_library
    if not torch.cuda.is_available():
        raise SystemExit("no CUDA device: this library has no CPU fallback")
    load_library()
    ctx = SushiCuda([0])
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    ctx.set_stream(stream.cuda_stream)
    n = args.size
    scrub = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def flush():
        # write a buffer twice the size of L2, then read it back: the write displaces the operands,
        # the read leaves L2 full of clean lines, so the timed call does not pay for write-backs
        scrub.fill_(1)
        scrub.max()

    def emit(op, case, flops, med, best, lib_ms, extra=None):
        line = {"op": op, "case": case, "size": n, "ms_median": round(med, 4), "ms_best": round(best, 4),
                "tflops_median": round(flops / med / 1e9, 2), "steps": args.steps, "warmup": args.warmup,
                "library_ms": None if lib_ms is None else round(lib_ms, 4), "l2": "flushed between calls"}
        line.update(extra or {})
        print(json.dumps(line), flush=True)

    if args.op in ("dgemm", "all"):
        a = torch.rand(n, n, device="cuda", dtype=torch.float64)
        b = torch.rand(n, n, device="cuda", dtype=torch.float64)
        c = torch.zeros(n, n, device="cuda", dtype=torch.float64)
        for ta, tb in [(0, 0), (0, 1), (1, 0), (1, 1)]:
            med, best = _time_calls(torch, stream, lambda: ctx.dgemm(ta, tb, n, n, n, 1.5, a, n, b, n, 0.5, c, n),
                                    lambda: None, flush, args.steps, args.warmup)
            lib = None
            if args.library:
                aa, bb = (a.t() if ta else a), (b.t() if tb else b)
                lib, _ = _time_calls(torch, stream, lambda: torch.addmm(c, aa, bb, beta=0.5, alpha=1.5, out=c),
                                     lambda: None, flush, args.steps, args.warmup)
            emit("dgemm", "NT"[ta] + "NT"[tb], 2.0 * n * n * n, med, best, lib,
                 {"dtype": "f64", "kernel": "dgemm_mma_kernel", "peak_note": "DMMA register-only microbenchmark: 35.6 TFLOP/s"})
        del a, b, c

    if args.op in ("strsm", "all"):
        a = (torch.rand(n, n, device="cuda") * (2.0 / n)) + torch.eye(n, device="cuda") * 4.0
        b0 = torch.rand(n, n, device="cuda")
        b = b0.clone()
        for (left, upper, trans) in [(1, 0, 0), (1, 1, 1), (0, 1, 0), (0, 0, 1)]:
            med, best = _time_calls(torch, stream, lambda: ctx.strsm(left, upper, trans, 0, n, n, 1.0, a, n, b, n),
                                    lambda: b.copy_(b0), flush, args.steps, args.warmup)
            lib = None
            if args.library:
                tri = a.triu() if upper else a.tril()
                op_a = tri.t() if trans else tri
                lib, _ = _time_calls(torch, stream,
                                     lambda: torch.linalg.solve_triangular(op_a, b0, upper=bool(upper) != bool(trans), left=bool(left)),
                                     lambda: None, flush, args.steps, args.warmup)
            emit("strsm", f"{'left' if left else 'right'}/{'upper' if upper else 'lower'}/{'T' if trans else 'N'}",
                 1.0 * n * n * n, med, best, lib, {"dtype": "f32"})
        del a, b, b0

    if args.op in ("skinny", "all"):
        # AI = 7.5 flop / byte: far below the ridge of either roofline, so HBM bounds it
        m_, n_, k_ = 65536, 16, 256
        a = torch.rand(m_, k_, device="cuda")
        b = torch.rand(k_, n_, device="cuda")
        c = torch.zeros(m_, n_, device="cuda")
        med, best = _time_calls(torch, stream, lambda: ctx.sgemm(0, 0, m_, n_, k_, 1.0, a, k_, b, n_, 0.0, c, n_),
                                lambda: None, flush, args.steps, args.warmup)
        lib = None
        if args.library:
            lib, _ = _time_calls(torch, stream, lambda: torch.mm(a, b, out=c), lambda: None, flush, args.steps, args.warmup)
        alg_bytes = 4.0 * (m_ * k_ + k_ * n_ + m_ * n_)
        peak, src = _hbm_peak_gbs()
        gbs = alg_bytes / (med * 1e-3) / 1e9
        emit("sgemm", "65536x16x256 NN", 2.0 * m_ * n_ * k_, med, best, lib,
             {"dtype": "f32", "size": None, "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peak, "unit": "GB/s",
                                                         "frac": round(gbs / peak, 4), "peak_source": src,
                                                         "algorithmic_bytes": alg_bytes}})
        del a, b, c

    if args.op in ("activation", "all"):
        # element-wise, in place: 4 B read + 4 B written per element; 1 GiB of floats
        count = 1 << 28
        x = torch.rand(count, device="cuda") * 4 - 2
        dy = torch.rand(count, device="cuda")
        dx = torch.empty(count, device="cuda")
        peak, src = _hbm_peak_gbs()
        for kind, label in [(1, "relu"), (7, "gelu"), (3, "sigmoid")]:
            med, best = _time_calls(torch, stream, lambda: ctx.activation(kind, x, count, 0.0), lambda: None, flush,
                                    args.steps, args.warmup)
            gbs = 8.0 * count / (med * 1e-3) / 1e9
            emit("activation", label, 0.0, med, best, None,
                 {"dtype": "f32", "size": count, "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peak, "unit": "GB/s",
                                                               "frac": round(gbs / peak, 4), "peak_source": src,
                                                               "algorithmic_bytes": 8.0 * count}})
            x.uniform_(-2, 2)
        med, best = _time_calls(torch, stream, lambda: ctx.activation_backward(7, dy, x, dx, count, 0.0), lambda: None, flush,
                                args.steps, args.warmup)
        gbs = 12.0 * count / (med * 1e-3) / 1e9
        emit("activation_backward", "gelu", 0.0, med, best, None,
             {"dtype": "f32", "size": count, "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peak, "unit": "GB/s",
                                                           "frac": round(gbs / peak, 4), "peak_source": src,
                                                           "algorithmic_bytes": 12.0 * count}})
        del x, dy, dx

    if args.op in ("ssyrk", "all"):
        a = torch.rand(n, n, device="cuda")
        c = torch.zeros(n, n, device="cuda")
        for (upper, trans) in [(0, 0), (1, 1)]:
            med, best = _time_calls(torch, stream, lambda: ctx.ssyrk(upper, trans, n, n, 1.0, a, n, 0.0, c, n),
                                    lambda: None, flush, args.steps, args.warmup)
            emit("ssyrk", f"{'upper' if upper else 'lower'}/{'T' if trans else 'N'}", 1.0 * n * n * n, med, best, None,
                 {"dtype": "f32", "flops_note": "n*n*k: the triangle only"})
    ctx.close()


if __name__ == "__main__":
    main()
