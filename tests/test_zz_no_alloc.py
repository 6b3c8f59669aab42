"""The allocation-free entry point (sushi_cuda_sgemm_static_scratch) against the regular one.

Collected last on purpose: a run that stops at the first failure has then already exercised
every other test.  The entry point serves callers that cannot let the library allocate at
call time (a host pool that owns the GPU, a graph capture in progress elsewhere in the
process, a loop that cannot take an allocation's device-wide synchronisation); its operand
planes live in a fixed 32 MiB array inside the library, shared by all calls on a device.
"""
import numpy as np
import pytest

from oracle import ref_gemm as og

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

TC3X = 2


def _case(ctx, stream, ta, tb, m, n, k, alpha, beta, seed):
    from sushiblas_b200.capi import sgemm_static_scratch
    ar, ac = (k, m) if ta else (m, k)
    br, bc = (n, k) if tb else (k, n)
    ha = og.uniform_pm1(seed, ar * ac).reshape(ar, ac)
    hb = og.uniform_pm1(seed + 1, br * bc).reshape(br, bc)
    hc = og.uniform_pm1(seed + 2, m * n).reshape(m, n)
    da, db = torch.from_numpy(ha).cuda(), torch.from_numpy(hb).cuda()
    c_new, c_old = torch.from_numpy(hc.copy()).cuda(), torch.from_numpy(hc.copy()).cuda()
    status = torch.full((1,), 77, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    # new entry point: no context, caller's stream, caller's status word
    sgemm_static_scratch(stream.cuda_stream, ta, tb, m, n, k, alpha, da, ac, db, bc, beta, c_new, n, status)
    # existing entry point on the tensor-core path
    ctx.set_gemm_variant(TC3X)
    ctx.sgemm(ta, tb, m, n, k, alpha, da, ac, db, bc, beta, c_old, n)
    ctx.set_gemm_variant(0)
    ctx.sync()
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    got, want = c_new.cpu().numpy(), c_old.cpu().numpy()
    # Same pre-pass and the same tensor-core kernel; only the work distribution may differ (the
    # regular entry point can cut few-tile problems along K through its context-owned exchange
    # area, which reorders the fp32 summation).  So: both inside the tolerance the parity tests use
    # against the fp64 oracle, and within a few fp32 roundings of each other.
    ref, absab = og.gemm_f64_np(ta, tb, m, n, k, alpha, ha, ac, 0, hb, bc, 0, beta, hc, n, 0, 1)
    for name, out in (("static_scratch", got), ("regular", want)):
        r, _ = og.tolerance_ratio(out[None], ref, absab, k, beta=beta, c_in=hc[None], budget=0.5)
        assert r <= 1.0, (name, r)
    scale = 2.0 ** -24 * (np.abs(alpha) * absab[0] + np.abs(beta * hc))
    assert np.all(np.abs(got.astype(np.float64) - want) <= 64.0 * scale + 1e-30), \
        f"max difference {np.abs(got - want).max()} between the two entry points"


def test_static_scratch_matches_regular_entry_point_twice_in_a_row(ctx):
    stream = torch.cuda.current_stream()
    # two calls back to back: the second is smaller and ragged, so stale planes of the first
    # remain in the shared array around it
    _case(ctx, stream, 1, 0, 512, 384, 256, 1.5, 0.5, seed=900)
    _case(ctx, stream, 0, 0, 300, 260, 100, 1.0, 0.0, seed=910)
    # and the largest square problem the 32 MiB array admits, after the small one
    _case(ctx, stream, 0, 1, 1024, 1024, 2048, -1.0, 1.0, seed=920)
    # K below 4: both entry points hand the product to the exact FFMA kernel
    _case(ctx, stream, 0, 0, 200, 136, 3, 1.0, 0.5, seed=930)


def test_static_scratch_rejects_sizes_beyond_its_array(ctx):
    from sushiblas_b200.capi import SushiCudaError, sgemm_static_scratch, workspace_bytes, STATIC_SCRATCH_BYTES
    assert workspace_bytes(1024, 1024, 2048) <= STATIC_SCRATCH_BYTES < workspace_bytes(2048, 2048, 2048)
    x = torch.zeros(16, device="cuda")          # never dereferenced: the size check comes first
    with pytest.raises(SushiCudaError) as e:
        sgemm_static_scratch(torch.cuda.current_stream().cuda_stream, 0, 0, 2048, 2048, 2048, 1.0, x, 2048, x, 2048,
                             0.0, x, 2048)
    assert e.value.code == -7 and "static scratch" in str(e.value)
    with pytest.raises(SushiCudaError) as e:
        sgemm_static_scratch(None, 0, 0, 64, 64, 64, 1.0, x, 8, x, 64, 0.0, x, 64)      # lda < k
    assert e.value.code == -1
