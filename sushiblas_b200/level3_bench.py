"""Timing of the Level-3 rows next to the fp32 GEMM: fp64 GEMM, TRSM, SYRK.

    python -m sushiblas_b200.level3_bench [--op dgemm|strsm|ssyrk|all] [--size N] [--steps K] [--warmup W] [--library]

One JSON line per (op, case): CUDA-event time of each call on the launching stream (median and
best of K calls after W warm-up calls), inputs resident in HBM, L2 flushed between calls by
writing a 256 MiB buffer.  `--library` adds the time of torch's own routine for the same problem
(cuBLAS) on the same GPU as context; it is not part of the product path.  Needs a CUDA device:
there is no CPU fallback.
"""
from __future__ import annotations

import argparse
import json
import statistics


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
    ap.add_argument("--op", default="all", choices=["dgemm", "strsm", "ssyrk", "all"])
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
        scrub.fill_(1)

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
