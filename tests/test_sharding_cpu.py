"""Multi-rank logic of the row-block / batch-index partition on CPU: world_size-2 gloo ranks
compute their blocks with the oracle, exchange them the way the library does (every rank is
the root of its own piece) and must reproduce the single-process result exactly."""
import os
import socket

import numpy as np
import pytest

torch = pytest.importorskip("torch")


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, m, n, k, batch, result_dir):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import torch.distributed as dist
    from oracle import ref_gemm as og
    from sushiblas_b200.capi import partition

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    a = og.uniform_pm1(1, batch * m * k).reshape(batch, m, k)
    b = og.uniform_pm1(2, batch * k * n).reshape(batch, k, n)
    c0 = og.uniform_pm1(3, batch * m * n).reshape(batch, m, n)

    # ---- row-block partition of a single GEMM (batch entry 0), B replicated, beta != 0
    first, count = partition(m, world, rank)
    c_full = torch.from_numpy(c0[0].copy())
    if count:
        ref, _ = og.gemm_f64_np(0, 0, count, n, k, 1.5, a[0, first:first + count], k, 0, b[0], n, 0, 0.5,
                                c0[0, first:first + count], n, 0, 1)
        c_full[first:first + count] = torch.from_numpy(ref[0].astype(np.float32))
    for r in range(world):                     # the exchange: rank r broadcasts its own block in place
        f, cnt = partition(m, world, r)
        if cnt:
            piece = c_full[f:f + cnt].contiguous()
            dist.broadcast(piece, src=r)
            c_full[f:f + cnt] = piece
    np.save(os.path.join(result_dir, f"rows_{rank}.npy"), c_full.numpy())

    # ---- batch-index partition of the strided-batched GEMM, beta == 0
    first, count = partition(batch, world, rank)
    out = torch.full((batch, m, n), float("nan"))
    if count:
        ref, _ = og.gemm_f64_np(0, 0, m, n, k, 1.0, a[first:first + count], k, m * k, b[first:first + count], n, k * n,
                                0.0, None, n, m * n, count)
        out[first:first + count] = torch.from_numpy(ref.astype(np.float32))
    for r in range(world):
        f, cnt = partition(batch, world, r)
        if cnt:
            piece = out[f:f + cnt].contiguous()
            dist.broadcast(piece, src=r)
            out[f:f + cnt] = piece
    np.save(os.path.join(result_dir, f"batch_{rank}.npy"), out.numpy())
    dist.destroy_process_group()


@pytest.mark.parametrize("m,batch", [(64, 4), (37, 3)])       # even and uneven blocks
def test_two_rank_partition_reproduces_single_process(tmp_path, lib_path, m, batch):
    import torch.multiprocessing as mp
    from oracle import ref_gemm as og

    n, k, world = 24, 40, 2
    port = _free_port()
    mp.spawn(_worker, args=(world, port, m, n, k, batch, str(tmp_path)), nprocs=world, join=True)

    a = og.uniform_pm1(1, batch * m * k).reshape(batch, m, k)
    b = og.uniform_pm1(2, batch * k * n).reshape(batch, k, n)
    c0 = og.uniform_pm1(3, batch * m * n).reshape(batch, m, n)
    ref_rows, _ = og.gemm_f64_np(0, 0, m, n, k, 1.5, a[0], k, 0, b[0], n, 0, 0.5, c0[0], n, 0, 1)
    ref_batch, _ = og.gemm_f64_np(0, 0, m, n, k, 1.0, a, k, m * k, b, n, k * n, 0.0, None, n, m * n, batch)
    for rank in range(world):
        rows = np.load(tmp_path / f"rows_{rank}.npy")
        bat = np.load(tmp_path / f"batch_{rank}.npy")
        assert np.array_equal(rows, ref_rows[0].astype(np.float32)), f"rank {rank} row-sharded result differs"
        assert np.array_equal(bat, ref_batch.astype(np.float32)), f"rank {rank} batch-sharded result differs"
