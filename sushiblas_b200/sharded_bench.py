"""Multi-GPU timing of the two sharded shapes next to the headline one: the batched GEMM sharded by
batch index (256 x 512^3) with and without the all-gather of C, and the tall GEMM sharded by row
blocks (65536 x 256 x 4096) without exchange, with the NCCL slab exchange and with the exchange
fused into the GEMM epilogue.  One process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \\
        -m sushiblas_b200.sharded_bench [--steps K] [--warmup W]

Rank 0 prints one JSON line per case: device time per call (CUDA events on the launching stream,
maximum over ranks, median of K calls after W warm-up calls); L2 is flushed before every call by
writing and re-reading a 256 MiB buffer.  Needs CUDA devices: there is no CPU fallback.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args(argv)

    import torch
    import torch.distributed as dist
    from sushiblas_b200 import SushiCuda, load_library
    from sushiblas_b200.capi import partition

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if not torch.cuda.is_available():
        raise SystemExit("no CUDA device: this library has no CPU fallback")
    load_library()
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    ctx = SushiCuda([local])
    stream = torch.cuda.Stream(device)
    torch.cuda.set_stream(stream)
    ctx.set_stream(stream.cuda_stream)
    if world > 1:
        ids = [ctx.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        ctx.comm_init_rank(ids[0], world, rank)
    scrub = torch.empty(256 << 20, dtype=torch.uint8, device=device)

    def timed(fn):
        times = []
        for i in range(args.warmup + args.steps):
            scrub.fill_(1)
            scrub.max()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            fn()
            e1.record(stream)
            e1.synchronize()
            t = torch.tensor([e0.elapsed_time(e1)], device=device, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            if i >= args.warmup:
                times.append(float(t.item()))
        return statistics.median(times), min(times)

    def emit(case, flops, med, best, extra):
        if rank == 0:
            line = {"case": case, "n_gpus": world, "ms_median": round(med, 4), "ms_best": round(best, 4),
                    "tflops_whole_job": round(flops / med / 1e9, 2), "steps": args.steps, "warmup": args.warmup,
                    "l2": "flushed before every call", "timing": "CUDA events, max over ranks"}
            line.update(extra)
            print(json.dumps(line), flush=True)

    # ---- batched GEMM, sharded by batch index (256 x 512^3)
    batch, n = 256, 512
    first, count = partition(batch, world, rank)
    a = torch.rand(max(count, 1), n, n, device=device) * 2 - 1
    b = torch.rand(max(count, 1), n, n, device=device) * 2 - 1
    c = torch.zeros(batch, n, n, device=device)
    for gather in (0, 1):
        med, best = timed(lambda: ctx.sgemm_batch_sharded(0, 0, n, n, n, 1.0, a, n, n * n, b, n, n * n, 0.0, c, n, n * n, batch,
                                                          gather=bool(gather)))
        emit("sgemm_256x512^3_batch_sharded", 2.0 * n * n * n * batch, med, best,
             {"exchange": "ncclAllGather of the C batches" if gather and world > 1 else "none (each rank keeps its batches)",
              "batches_per_rank": count})
    del a, b, c

    # ---- tall GEMM, sharded by row blocks (65536 x 256 x 4096)
    m, n, k = 65536, 256, 4096
    first, count = partition(m, world, rank)
    a = torch.rand(count, k, device=device) * 2 - 1
    b = torch.rand(k, n, device=device) * 0.04 - 0.02
    c_raw = ctx.malloc(m * n * 4)
    modes = [(0, "none (each rank keeps its row block)")]
    if world > 1:
        handles = [None] * world
        dist.all_gather_object(handles, ctx.ipc_export(c_raw))
        opened = [ctx.ipc_open(handles[r]) if r != rank else None for r in range(world)]
        ctx.comm_set_peer_buffers([c_raw if r == rank else opened[r] for r in range(world)], m * n * 4)
        modes += [(1, "NCCL, slab-pipelined"), (2, "peer stores fused into the GEMM epilogue (NVLink)")]
    for gather, label in modes:
        med, best = timed(lambda: ctx.sgemm_row_sharded(0, 0, m, n, k, 1.0, a, k, b, n, 0.0, c_raw, n, gather=gather))
        emit("sgemm_65536x256x4096_row_sharded", 2.0 * m * n * k, med, best, {"exchange": label, "rows_per_rank": count})
    ctx.sync()
    if world > 1:
        dist.barrier()
        ctx.comm_set_peer_buffers([], 0)
        for r in range(world):
            if r != rank:
                ctx.ipc_close(opened[r])
        dist.barrier()
    ctx.free(c_raw)
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
