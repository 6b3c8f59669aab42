"""Worker of the multi-GPU tests; run one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29511 tests/multi_gpu_worker.py

Each rank multiplies its row block (or batch block) through the sharded C-ABI entry points with
the NCCL exchange, then compares the gathered result with the same problem computed by this
rank alone through sushi_cuda_sgemm: the tiles are the same kernels in the same order, so the
results must be bit-identical.  Exits non-zero on any mismatch.
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from sushiblas_b200 import SushiCuda
from sushiblas_b200.capi import partition


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    ctx = SushiCuda([local])
    stream = torch.cuda.Stream(dev)
    torch.cuda.set_stream(stream)
    ctx.set_stream(stream.cuda_stream)
    ids = [ctx.comm_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    ctx.comm_init_rank(ids[0], world, rank)
    failures = []

    def full(seed, rows, cols):
        t = torch.empty(rows, cols, device=dev)
        ctx.fill_uniform(t, t.numel(), seed)
        return t

    # ---- row-sharded GEMM: even blocks with slabs, uneven blocks, beta != 0, transposed A
    for (m, n, k, ta, alpha, beta) in [(8192, 512, 384, 0, 1.0, 0.0), (4100, 256, 300, 0, 1.5, 0.5),
                                       (2048, 384, 256, 1, 1.0, 1.0), (30, 20, 10, 0, 1.0, 0.0)]:
        a = full(11, k, m) if ta else full(11, m, k)
        b = full(12, k, n)
        c_in = full(13, m, n)
        first, count = partition(m, world, rank)
        a_local = (a[:, first:first + count] if ta else a[first:first + count]).contiguous()
        c_shard = c_in.clone()
        torch.cuda.synchronize()
        # same kernel family on both sides (the automatic choice depends on the block size)
        ctx.set_gemm_variant(2 if m >= 1024 else 1)
        ctx.sgemm_row_sharded(ta, 0, m, n, k, alpha, a_local, count if ta else k, b, n, beta, c_shard, n, gather=True)
        c_one = c_in.clone()
        ctx.sgemm(ta, 0, m, n, k, alpha, a, m if ta else k, b, n, beta, c_one, n)
        ctx.sync()
        torch.cuda.synchronize()
        if not torch.equal(c_shard, c_one):
            bad = int((c_shard != c_one).sum())
            failures.append(f"row_sharded m={m} n={n} k={k} ta={ta}: {bad} elements differ on rank {rank}")

    # ---- batch-sharded strided-batched GEMM
    for (batch, m, n, k) in [(16, 256, 256, 192), (5, 64, 48, 32)]:
        a = full(21, batch * m, k).view(batch, m, k)
        b = full(22, batch * k, n).view(batch, k, n)
        first, count = partition(batch, world, rank)
        c_shard = torch.full((batch, m, n), float("nan"), device=dev)
        ctx.set_gemm_variant(2 if m >= 256 else 1)
        ctx.sgemm_batch_sharded(0, 0, m, n, k, 1.0, a[first:first + count].contiguous() if count else a, k, m * k,
                                b[first:first + count].contiguous() if count else b, n, k * n, 0.0, c_shard, n, m * n,
                                batch, gather=True)
        c_one = torch.empty(batch, m, n, device=dev)
        ctx.sgemm_strided_batched(0, 0, m, n, k, 1.0, a, k, m * k, b, n, k * n, 0.0, c_one, n, m * n, batch)
        ctx.sync()
        torch.cuda.synchronize()
        if not torch.equal(c_shard, c_one):
            failures.append(f"batch_sharded batch={batch} m={m}: mismatch on rank {rank}")

    flag = torch.tensor([len(failures)], device=dev)
    dist.all_reduce(flag)
    for f in failures:
        print("FAIL:", f, flush=True)
    if rank == 0:
        print(f"multi_gpu_worker: world={world} total failures={int(flag.item())}", flush=True)
    ctx.close()
    dist.destroy_process_group()
    sys.exit(1 if int(flag.item()) else 0)


if __name__ == "__main__":
    main()
