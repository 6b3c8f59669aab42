"""GPU parity tests of the fp64 GEMM (C ABI sushi_cuda_dgemm*) against the extended-precision oracle.

Tolerance (floating point): the fp64 form of the GEMM bound,
    |dC_ij| <= 8*K*2^-53*(|A||B|)_ij + 2^-53*|beta*C_ij| ,
tested with the K term at HALF budget against a reference accumulated in x87 extended precision
(oracle_dgemm_f80acc).  The integer-valued golden vectors of the fp32 path, widened to double,
must match bit for bit.
"""
import os

import numpy as np
import pytest

from oracle import ref_gemm as og

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "gemm_integer_kat.npz")
BUDGET = 0.5


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def run(ctx, ta, tb, m, n, k, alpha, a, lda, sa, b, ldb, sb, beta, c, ldc, sc, batch):
    dc = dev(c)
    ctx.dgemm(ta, tb, m, n, k, alpha, dev(a), lda, dev(b), ldb, beta, dc, ldc, sa, sb, sc, batch)
    ctx.sync()
    return dc.cpu().numpy()


def check(ctx, ta, tb, m, n, k, alpha, beta, batch=1, pad=(0, 0, 0), seed=900, poison_c=False):
    ar, ac = (k, m) if ta else (m, k)
    br, bc = (n, k) if tb else (k, n)
    lda, ldb, ldc = ac + pad[0], bc + pad[1], n + pad[2]
    sa, sb, sc = ar * lda, br * ldb, m * ldc
    rng = np.random.default_rng(seed)
    a = rng.uniform(-1, 1, max(1, batch * sa))
    b = rng.uniform(-1, 1, max(1, batch * sb))
    c0 = rng.uniform(-1, 1, max(1, batch * sc))
    c_in = np.full_like(c0, np.nan) if poison_c else c0.copy()
    out = run(ctx, ta, tb, m, n, k, alpha, a, lda, sa, b, ldb, sb, beta, c_in, ldc, sc, batch)
    ref, absab = og.dgemm_f80_c(ta, tb, m, n, k, alpha, a, lda, sa, b, ldb, sb, beta, c0, ldc, sc, batch)
    idx = (np.arange(batch)[:, None, None] * sc + np.arange(m)[None, :, None] * ldc + np.arange(n)[None, None, :]).ravel()
    r = og.tolerance_ratio_f64(out[idx], ref[idx], absab[idx], k, beta=beta, c_in=c0[idx], budget=BUDGET)
    assert r <= 1.0, f"ta={ta} tb={tb} m={m} n={n} k={k} batch={batch} pad={pad}: ratio {r:.3g}"
    if pad[2] and not poison_c:
        keep = np.ones(out.shape, dtype=bool)
        keep[idx] = False
        assert np.array_equal(out[keep], c0[keep]), "C padding was overwritten"
    return r


def test_reference_known_answers_in_double(ctx):
    # tests/blas/level3/test_gemm.cpp:39-62 (3 x 3 times identity) and :64-88 (column-major 2 x 2 by operand swap)
    g = np.load(GOLDEN)
    out = run(ctx, 0, 0, 3, 3, 3, 1.0, g["ref_simple3x3.a"].astype(np.float64), 3, 0, g["ref_simple3x3.b"].astype(np.float64),
              3, 0, 0.0, np.zeros(9), 3, 0, 1)
    assert np.array_equal(out, g["ref_simple3x3.c_out"].astype(np.float64))
    out = run(ctx, 0, 0, 2, 2, 2, 1.0, g["ref_colmajor2x2.b"].astype(np.float64), 2, 0,
              g["ref_colmajor2x2.a"].astype(np.float64), 2, 0, 0.0, np.zeros(4), 2, 0, 1)
    assert np.array_equal(out, g["ref_colmajor2x2.c_out"].astype(np.float64))


def test_integer_golden_bit_exact_in_double(ctx):
    g = np.load(GOLDEN)
    for name in g["names"]:
        ta, tb, m, n, k, alpha, beta, batch, lda, ldb, ldc, sa, sb, sc = [int(v) for v in g[f"{name}.meta"]]
        out = run(ctx, ta, tb, m, n, k, float(alpha), g[f"{name}.a"].astype(np.float64), lda, sa,
                  g[f"{name}.b"].astype(np.float64), ldb, sb, float(beta), g[f"{name}.c_in"].astype(np.float64), ldc, sc, batch)
        exp = g[f"{name}.c_out"].astype(np.float64)
        assert np.array_equal(out, exp), name


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_dgemm_shape_sweep(ctx, ta, tb):
    worst = 0.0
    for (m, n, k) in [(1, 1, 1), (2, 3, 4), (7, 5, 3), (8, 8, 8), (17, 33, 9), (64, 64, 16), (65, 63, 17), (100, 1, 50),
                      (1, 100, 50), (129, 127, 130), (200, 300, 70)]:
        for (alpha, beta) in [(1.0, 0.0), (1.5, 0.5), (-1.0, 1.0)]:
            worst = max(worst, check(ctx, ta, tb, m, n, k, alpha, beta, seed=901 + m + n + k))
    # padded / odd leading dimensions (scalar load path), batches, both tile sizes
    check(ctx, ta, tb, 130, 70, 90, 1.5, 0.5, batch=3, pad=(1, 3, 5), seed=950)
    check(ctx, ta, tb, 130, 70, 90, 1.5, 0.5, batch=2, pad=(2, 4, 6), seed=951)
    check(ctx, ta, tb, 1536, 1664, 200, 1.0, 0.5, seed=952)          # 128 x 128 tiles, more than one wave of CTAs
    check(ctx, ta, tb, 1500, 1700, 77, 1.0, 0.0, pad=(0, 0, 2), seed=953, poison_c=False)
    assert worst <= 1.0


def test_dgemm_beta_zero_ignores_nan_c_and_degenerate_sizes(ctx):
    check(ctx, 0, 0, 96, 80, 64, 1.0, 0.0, poison_c=True)
    check(ctx, 1, 1, 1300, 1300, 40, 2.0, 0.0, poison_c=True)
    c = torch.ones(16, dtype=torch.float64, device="cuda")
    x = torch.zeros(16, dtype=torch.float64, device="cuda")
    ctx.dgemm(0, 0, 4, 4, 0, 1.0, x, 1, x, 4, 0.5, c, 4)              # k == 0: C <- beta C
    ctx.sync()
    assert torch.equal(c, torch.full((16,), 0.5, dtype=torch.float64, device="cuda"))
    ctx.dgemm(0, 0, 4, 4, 4, 0.0, x, 4, x, 4, 0.0, c, 4)              # alpha == 0, beta == 0: C <- 0
    ctx.sync()
    assert torch.count_nonzero(c).item() == 0
    c = torch.ones(16, dtype=torch.float64, device="cuda")
    ctx.dgemm(0, 0, 0, 4, 4, 1.0, x, 4, x, 4, 0.0, c, 4)
    ctx.dgemm(0, 0, 4, 0, 4, 1.0, x, 4, x, 1, 0.0, c, 1)
    ctx.dgemm(0, 0, 4, 4, 4, 1.0, x, 4, x, 4, 0.0, c, 4, batch=0)
    ctx.sync()
    assert torch.equal(c, torch.ones(16, dtype=torch.float64, device="cuda"))


def test_dgemm_invalid_arguments_are_rejected(ctx):
    from sushiblas_b200 import SushiCudaError
    x = torch.zeros(64, dtype=torch.float64, device="cuda")
    with pytest.raises(SushiCudaError) as e:
        ctx.dgemm(0, 0, 4, 4, 4, 1.0, x, 3, x, 4, 0.0, x, 4)         # lda < k
    assert e.value.code == -1
    with pytest.raises(SushiCudaError):
        ctx.dgemm(0, 0, 4, 4, 4, 1.0, x, 4, x, 4, 0.0, x, 2)         # ldc < n
    with pytest.raises(SushiCudaError):
        ctx.dgemm(0, 0, 4, 4, 4, 1.0, None, 4, x, 4, 0.0, x, 4)


def test_dgemm_2048_sampled_rows(ctx):
    """2048^3 in all four transposes; sampled rows against numpy extended-precision dot products."""
    m = n = k = 2048
    rng = np.random.default_rng(77)
    a = rng.uniform(-1, 1, (m, k)); b = rng.uniform(-1, 1, (k, n)); c0 = rng.uniform(-1, 1, (m, n))
    rows = np.array([0, 1, 127, 128, 1023, 1500, 2047])
    for ta, tb in [(0, 0), (0, 1), (1, 0), (1, 1)]:
        a_st = np.ascontiguousarray(a.T) if ta else a
        b_st = np.ascontiguousarray(b.T) if tb else b
        dc = dev(c0)
        ctx.dgemm(ta, tb, m, n, k, 1.5, dev(a_st), a_st.shape[1], dev(b_st), b_st.shape[1], 0.5, dc, n)
        ctx.sync()
        got = dc.cpu().numpy()[rows]
        al = a[rows].astype(np.longdouble); bl = b.astype(np.longdouble)
        ref = np.longdouble(1.5) * (al @ bl) + np.longdouble(0.5) * c0[rows].astype(np.longdouble)
        absab = (np.abs(a[rows]) @ np.abs(b))
        r = og.tolerance_ratio_f64(got, ref, absab, k, beta=0.5, c_in=c0[rows], budget=BUDGET)
        assert r <= 1.0, (ta, tb, r)
