"""Worker of the multi-GPU tests; run one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29511 tests/multi_gpu_worker.py

Each rank multiplies its row block (or batch block) through the sharded C-ABI entry points --
NCCL slab exchange, the exchange fused into the GEMM epilogue (peer stores over NVLink) and the host-buffer form --
then compares the gathered result with the same problem computed by this rank alone through
sushi_cuda_sgemm.  Where both sides run the same tiles in the same order the results must be
bit-identical; the fused case checks that all ranks hold identical bits and that they agree
with the single-GPU result to fp32 summation order.  Exits non-zero on any mismatch.
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

    import zlib
    import numpy as np

    def compare(got, want, k, alpha, beta, label, absab=None, c_in=None):
        """got / want: numpy arrays.  (1) every rank holds identical bits (the exchange is exact);
        (2) agreement with one GPU computing everything, up to fp32 summation order (a block with
        fewer tiles than SMs is cut along K, the full problem may be cut differently): both sides lie
        within 4*K*2^-24*(|A||B|) + 2^-24*|beta*C| of the exact result, so they differ by at most twice that."""
        sums = [None] * world
        dist.all_gather_object(sums, zlib.crc32(np.ascontiguousarray(got).tobytes()))
        if len(set(sums)) != 1:
            failures.append(f"{label}: ranks hold different results ({sums})")
        diff = np.abs(got.astype(np.float64) - want)
        if absab is None:
            bound = np.full_like(diff, 64 * 2.0 ** -24 * (abs(alpha) * k * 0.5 + abs(beta)))
        else:
            bound = 8.0 * k * 2.0 ** -24 * absab.astype(np.float64)
            if beta != 0.0 and c_in is not None:
                bound = bound + 2.0 ** -23 * np.abs(beta * c_in.astype(np.float64))
        if not np.all(diff <= bound):
            failures.append(f"{label}: max |diff| {float(diff.max())}, worst ratio to the bound "
                            f"{float((diff / np.maximum(bound, 1e-300)).max())} vs single GPU on rank {rank}")

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
        compare(c_shard.cpu().numpy(), c_one.cpu().numpy(), k, alpha, beta, f"row_sharded m={m} n={n} k={k} ta={ta}")

    # ---- fused GEMM + all-gather: the epilogue stores finished tiles into the peers' buffers.  Even blocks,
    # uneven blocks, the automatic kernel choice on an uneven partition (every rank must choose the same exchange)
    # and a problem with fewer rows than ranks (trailing ranks own nothing but still take part).
    for (m, n, k, alpha, beta, variant) in [(4096, 1024, 512, 1.0, 0.0, 2), (2048 * world, 768, 640, 1.5, 0.5, 2),
                                            (1000, 512, 256, 1.0, 0.0, 2), (4099, 512, 512, 1.0, 0.5, 0),
                                            (1017, 512, 512, 1.0, 0.0, 0), (world - 1, 256, 128, 2.0, 0.0, 2)]:
        nbytes = m * n * 4
        c_mine = ctx.malloc(nbytes)                      # base of a cudaMalloc block: exportable
        handles = [None] * world
        dist.all_gather_object(handles, ctx.ipc_export(c_mine))
        opened = [ctx.ipc_open(handles[r]) if r != rank else None for r in range(world)]
        ctx.comm_set_peer_buffers([c_mine if r == rank else opened[r] for r in range(world)], nbytes)
        a = full(31, m, k); b = full(32, k, n); c_in = full(33, m, n)
        first, count = partition(m, world, rank)
        ctx.memcpy_d2d(c_mine, c_in, nbytes)
        ctx.set_gemm_variant(variant)
        a_local = a[first:first + count].contiguous() if count else a[:1].contiguous()
        for _ in range(2):                               # twice: the second call overwrites the first's C
            ctx.memcpy_d2d(c_mine, c_in, nbytes)
            ctx.sync(); dist.barrier()
            ctx.sgemm_row_sharded(0, 0, m, n, k, alpha, a_local, k, b, n, beta, c_mine, n, gather=2)
        c_one = c_in.clone()
        ctx.sgemm(0, 0, m, n, k, alpha, a, k, b, n, beta, c_one, n)
        got = np.empty((m, n), dtype=np.float32)
        ctx.memcpy_d2h(got, c_mine, nbytes)
        ctx.sync()
        torch.cuda.synchronize()
        want = c_one.cpu().numpy()
        absab = (a.abs().double() @ b.abs().double()).cpu().numpy()
        compare(got, want, k, alpha, beta, f"fused gather m={m} n={n} k={k} variant={variant}", absab=absab,
                c_in=c_in.cpu().numpy())
        dist.barrier()
        ctx.comm_set_peer_buffers([], 0)
        for r in range(world):
            if r != rank:
                ctx.ipc_close(opened[r])
        dist.barrier()
        ctx.free(c_mine)

    # ---- host-buffer form: every rank uploads its rows of A and its share of B's k rows, the shares are exchanged
    # device to device, C's rows come back to the rank's host.  Even and uneven partitions of m and of k, beta != 0,
    # transposed A, and a transposed B (no exchange: every rank uploads all of it).
    # Shares of 4096 k rows or more travel in pieces of ~2048 rows and the first row chunk is accumulated piece by piece.
    for (m, n, k, ta, tb, alpha, beta) in [(8192, 512, 1024, 0, 0, 1.0, 0.0), (4100, 256, 301, 0, 0, 1.5, 0.5),
                                           (2048 * world, 384, 512, 1, 0, 1.0, 1.0), (3000, 320, 256, 0, 1, 1.0, 0.0),
                                           (2304 * world, 256, 4200 * world, 0, 0, 1.5, 0.5),
                                           (2050 * world, 256, 6144 * world + 5, 1, 0, 1.0, 0.0),
                                           (world - 1, 64, 48, 0, 0, 2.0, 0.0)]:      # fewer rows than ranks: the last rank owns none
        a = full(41, k, m) if ta else full(41, m, k)
        b = full(42, n, k) if tb else full(42, k, n)
        c_in = full(43, m, n)
        first, count = partition(m, world, rank)
        rows = max(count, 1)
        lo = first if count else 0                          # a rank without rows still passes valid (unused) buffers
        a_local = (a[:, lo:lo + rows] if ta else a[lo:lo + rows]).contiguous()
        ha = a_local.cpu().pin_memory()
        hb = torch.empty_like(b, device="cpu").pin_memory()
        k0, kc = partition(k, world, rank)
        if tb:
            hb.copy_(b)                                      # stored n x k: goes up whole
        else:
            hb.fill_(float("nan"))                           # only this rank's share of the k rows is valid on its host
            hb[k0:k0 + kc].copy_(b[k0:k0 + kc])
        hc = c_in[lo:lo + rows].cpu().pin_memory()
        da = torch.empty_like(a_local); db = torch.full_like(b, float("nan")); dc = torch.empty(rows, n, device=dev)
        ctx.set_gemm_variant(2 if m >= 1024 else 1)
        torch.cuda.synchronize(); dist.barrier()
        ctx.sgemm_row_sharded_host(ta, tb, m, n, k, alpha, ha, rows if ta else k, hb, k if tb else n, beta, hc, n, da, db, dc)
        c_one = c_in.clone()
        ctx.sgemm(ta, tb, m, n, k, alpha, a, m if ta else k, b, k if tb else n, beta, c_one, n)
        ctx.sync()
        torch.cuda.synchronize()
        if count:
            want = c_one[first:first + count].cpu().numpy()
            got = hc[:count].numpy()
            diff = np.abs(got.astype(np.float64) - want)
            opa = (a.t() if ta else a)[first:first + count]
            opb = b.t() if tb else b
            absab = (opa.abs().double() @ opb.abs().double()).cpu().numpy()
            bound = 8.0 * k * 2.0 ** -24 * absab + 2.0 ** -23 * np.abs(beta * c_in[first:first + count].cpu().numpy().astype(np.float64))
            if not np.all(diff <= bound):
                failures.append(f"row_sharded_host m={m} n={n} k={k} ta={ta} tb={tb}: worst ratio to the bound "
                                f"{float((diff / np.maximum(bound, 1e-300)).max())} on rank {rank}")
        if not tb and not torch.equal(db, b):
            failures.append(f"row_sharded_host m={m} k={k}: the exchanged B differs from the original on rank {rank}")
        dist.barrier()

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
        compare(c_shard.cpu().numpy(), c_one.cpu().numpy(), k, 1.0, 0.0, f"batch_sharded batch={batch} m={m}")

    # ---- batch-sharded GEMM with the exchange fused into the epilogue (peer stores): even and uneven batch counts,
    # fewer batches than ranks, beta != 0
    for (batch, m, n, k, alpha, beta) in [(4 * world, 512, 512, 256, 1.0, 0.0), (4 * world + 1, 256, 512, 384, 1.5, 0.5),
                                          (world - 1, 512, 256, 128, 1.0, 0.0)]:
        nbytes = batch * m * n * 4
        c_mine = ctx.malloc(nbytes)
        handles = [None] * world
        dist.all_gather_object(handles, ctx.ipc_export(c_mine))
        opened = [ctx.ipc_open(handles[r]) if r != rank else None for r in range(world)]
        ctx.comm_set_peer_buffers([c_mine if r == rank else opened[r] for r in range(world)], nbytes)
        a = full(51, batch * m, k).view(batch, m, k); b = full(52, batch * k, n).view(batch, k, n); c_in = full(53, batch * m, n)
        first, count = partition(batch, world, rank)
        ctx.set_gemm_variant(2)
        a_local = a[first:first + count].contiguous() if count else a[:1].contiguous()
        b_local = b[first:first + count].contiguous() if count else b[:1].contiguous()
        for _ in range(2):
            ctx.memcpy_d2d(c_mine, c_in, nbytes)
            ctx.sync(); dist.barrier()
            ctx.sgemm_batch_sharded(0, 0, m, n, k, alpha, a_local, k, m * k, b_local, n, k * n, beta, c_mine, n, m * n, batch, gather=2)
        c_one = c_in.clone()
        ctx.sgemm_strided_batched(0, 0, m, n, k, alpha, a, k, m * k, b, n, k * n, beta, c_one, n, m * n, batch)
        got = np.empty((batch * m, n), dtype=np.float32)
        ctx.memcpy_d2h(got, c_mine, nbytes)
        ctx.sync()
        torch.cuda.synchronize()
        absab = torch.bmm(a.abs().double(), b.abs().double()).reshape(batch * m, n).cpu().numpy()
        compare(got, c_one.cpu().numpy(), k, alpha, beta, f"fused batch gather batch={batch} m={m} n={n} k={k}", absab=absab,
                c_in=c_in.cpu().numpy())
        dist.barrier()
        ctx.comm_set_peer_buffers([], 0)
        for r in range(world):
            if r != rank:
                ctx.ipc_close(opened[r])
        dist.barrier()
        ctx.free(c_mine)

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
