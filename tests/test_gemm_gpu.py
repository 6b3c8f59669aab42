"""GPU parity tests: the CUDA path through the C ABI against the fp64 oracle.

Tolerance (floating point): the bound of the specification,
    |dC_ij| <= 8*K*2^-24*(|A||B|)_ij + 2^-24*|beta*C_ij| ,
tested against the fp64 oracle with the K term at HALF budget, so that, by the triangle
inequality, the result is within the full K term of any conforming reference sgemm (the
beta term is a single fp32 rounding of the output and is kept whole).  Integer-valued golden
vectors must match bit for bit.
"""
import os

import numpy as np
import pytest

from oracle import ref_gemm as og
from sushiblas_b200 import SushiCuda, SushiCudaError

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "gemm_integer_kat.npz")
AUTO, SIMT, TC3X = 0, 1, 2
BUDGET = 0.5


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def run_gemm(ctx, variant, ta, tb, m, n, k, alpha, a, lda, sa, b, ldb, sb, beta, c, ldc, sc, batch):
    """a, b, c: flat float32 numpy buffers.  Returns the flat C buffer after the call."""
    ctx.set_gemm_variant(variant)
    da, db, dc = dev(a), dev(b), dev(c)
    if batch == 1 and sa == 0 and sb == 0 and sc == 0:
        ctx.sgemm(ta, tb, m, n, k, alpha, da, lda, db, ldb, beta, dc, ldc)
    else:
        ctx.sgemm_strided_batched(ta, tb, m, n, k, alpha, da, lda, sa, db, ldb, sb, beta, dc, ldc, sc, batch)
    ctx.sync()
    ctx.set_gemm_variant(AUTO)
    return dc.cpu().numpy()


def make_case(seed, ta, tb, m, n, k, batch=1, pad=(0, 0, 0), dist="uniform"):
    ar, ac = (k, m) if ta else (m, k)
    br, bc = (n, k) if tb else (k, n)
    lda, ldb, ldc = ac + pad[0], bc + pad[1], n + pad[2]
    sa, sb, sc = ar * lda, br * ldb, m * ldc
    gen = og.uniform_pm1 if dist == "uniform" else (lambda s, cnt: og.normal(s, cnt, 1.0))
    a = gen(seed, max(1, batch * sa))
    b = gen(seed + 1, max(1, batch * sb))
    c = og.uniform_pm1(seed + 2, max(1, batch * sc))
    return dict(a=a, b=b, c=c, lda=lda, ldb=ldb, ldc=ldc, sa=sa, sb=sb, sc=sc)


def check(ctx, variant, ta, tb, m, n, k, alpha, beta, batch=1, pad=(0, 0, 0), seed=100, dist="uniform",
          poison_c=False, budget=BUDGET):
    cs = make_case(seed, ta, tb, m, n, k, batch, pad, dist)
    c_in = cs["c"].copy()
    if poison_c:
        assert beta == 0.0
        c_in[:] = np.nan
    out = run_gemm(ctx, variant, ta, tb, m, n, k, alpha, cs["a"], cs["lda"], cs["sa"], cs["b"], cs["ldb"], cs["sb"],
                   beta, c_in, cs["ldc"], cs["sc"], batch)
    ref, absab = og.gemm_f64_np(ta, tb, m, n, k, alpha, cs["a"], cs["lda"], cs["sa"], cs["b"], cs["ldb"], cs["sb"],
                                beta, cs["c"], cs["ldc"], cs["sc"], batch)
    got = og._view(out, m, n, cs["ldc"], cs["sc"], batch)
    cin_v = og._view(cs["c"], m, n, cs["ldc"], cs["sc"], batch)
    r, q = og.tolerance_ratio(got, ref, absab, k, beta=beta, c_in=cin_v, budget=budget)
    assert r <= 1.0, f"variant={variant} ta={ta} tb={tb} m={m} n={n} k={k} batch={batch}: ratio {r:.3g} (noK {q:.3g})"
    # padding between rows / batches of C must be untouched
    if pad[2] and not poison_c:
        mask = np.ones(out.shape, dtype=bool)
        idx = (np.arange(batch)[:, None, None] * cs["sc"] + np.arange(m)[None, :, None] * cs["ldc"]
               + np.arange(n)[None, None, :]).ravel()
        mask[idx] = False
        assert np.array_equal(out[mask], cs["c"][mask]), "C padding was overwritten"
    return r, q


# ------------------------------------------------------------------ known answers
def test_reference_kat_3x3(ctx):
    g = np.load(GOLDEN)
    out = run_gemm(ctx, AUTO, 0, 0, 3, 3, 3, 1.0, g["ref_simple3x3.a"], 3, 0, g["ref_simple3x3.b"], 3, 0, 0.0,
                   g["ref_simple3x3.c_in"], 3, 0, 1)
    assert np.array_equal(out, g["ref_simple3x3.c_out"])


def test_reference_kat_column_major_via_operand_swap(ctx):
    # column-major C = A*B is the row-major product C^T = B^T * A^T on the same memory images
    g = np.load(GOLDEN)
    out = run_gemm(ctx, AUTO, 0, 0, 2, 2, 2, 1.0, g["ref_colmajor2x2.b"], 2, 0, g["ref_colmajor2x2.a"], 2, 0, 0.0,
                   np.zeros(4, np.float32), 2, 0, 1)
    assert np.array_equal(out, g["ref_colmajor2x2.c_out"])


@pytest.mark.parametrize("variant", [SIMT, TC3X])
def test_integer_golden_bit_exact(ctx, variant):
    g = np.load(GOLDEN)
    for name in g["names"]:
        ta, tb, m, n, k, alpha, beta, batch, lda, ldb, ldc, sa, sb, sc = [int(v) for v in g[f"{name}.meta"]]
        out = run_gemm(ctx, variant, ta, tb, m, n, k, float(alpha), g[f"{name}.a"], lda, sa, g[f"{name}.b"], ldb, sb,
                       float(beta), g[f"{name}.c_in"], ldc, sc, batch)
        exp = g[f"{name}.c_out"]
        bad = np.flatnonzero(out != exp)
        assert bad.size == 0, f"{name} variant={variant}: {bad.size} mismatches, first at {bad[:5]}, " \
                              f"got {out[bad[:5]]} want {exp[bad[:5]]}"


# ------------------------------------------------------------------ SIMT kernel
@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_simt_small_shape_sweep(ctx, ta, tb):
    sizes = [1, 2, 3, 8, 17, 32, 33, 64, 65, 127, 129]
    rng = np.random.default_rng(5 + 2 * ta + tb)
    for _ in range(24):
        m, n, k = (int(rng.choice(sizes)) for _ in range(3))
        alpha, beta = float(rng.choice([1.0, 1.5, -0.5])), float(rng.choice([0.0, 0.5, 1.0, -1.0]))
        pad = tuple(int(v) for v in rng.choice([0, 1, 3, 4], 3))
        check(ctx, SIMT, ta, tb, m, n, k, alpha, beta, batch=int(rng.choice([1, 2, 5])), pad=pad,
              seed=int(rng.integers(1, 1 << 30)))


def test_simt_beta_zero_ignores_nan_c(ctx):
    check(ctx, SIMT, 0, 0, 70, 50, 33, 1.0, 0.0, poison_c=True)
    check(ctx, SIMT, 1, 1, 128, 128, 64, 2.0, 0.0, batch=2, poison_c=True)


def test_simt_mid_sizes(ctx):
    check(ctx, SIMT, 0, 0, 512, 384, 256, 1.0, 0.0)
    check(ctx, SIMT, 0, 1, 1000, 300, 200, 1.5, 0.5, pad=(0, 0, 4))
    check(ctx, SIMT, 1, 0, 256, 1024, 96, 1.0, 1.0, batch=3)


def test_degenerate_sizes(ctx):
    # k == 0: C <- beta*C ; alpha == 0 likewise; m or n == 0: no-op
    c = og.uniform_pm1(9, 12)
    out = run_gemm(ctx, AUTO, 0, 0, 3, 4, 0, 1.0, np.zeros(1, np.float32), 1, 0, np.zeros(4, np.float32), 4, 0, 0.5,
                   c.copy(), 4, 0, 1)
    assert np.array_equal(out, np.float32(0.5) * c)
    out = run_gemm(ctx, AUTO, 0, 0, 3, 4, 0, 1.0, np.zeros(1, np.float32), 1, 0, np.zeros(4, np.float32), 4, 0, 0.0,
                   np.full(12, np.nan, np.float32), 4, 0, 1)
    assert np.array_equal(out, np.zeros(12, np.float32))
    out = run_gemm(ctx, AUTO, 0, 0, 0, 4, 5, 1.0, np.zeros(1, np.float32), 5, 0, np.zeros(20, np.float32), 4, 0, 0.0,
                   c.copy(), 4, 0, 1)
    assert np.array_equal(out, c)


def test_invalid_arguments_are_rejected(ctx):
    from sushiblas_b200 import SushiCudaError
    x = torch.zeros(64, device="cuda")
    with pytest.raises(SushiCudaError) as e:
        ctx.sgemm(0, 0, 4, 4, 4, 1.0, x, 3, x, 4, 0.0, x, 4)      # lda < k
    assert e.value.code == -1
    with pytest.raises(SushiCudaError):
        ctx.sgemm(0, 0, 4, 4, 4, 1.0, x, 4, x, 4, 0.0, x, 2)      # ldc < n
    with pytest.raises(SushiCudaError):
        ctx.sgemm(0, 0, -1, 4, 4, 1.0, x, 4, x, 4, 0.0, x, 4)
    with pytest.raises(SushiCudaError):
        ctx.sgemm(0, 0, 4, 4, 4, 1.0, None, 4, x, 4, 0.0, x, 4)
    with pytest.raises(SushiCudaError):
        ctx.sgemm(0, 0, 4, 4, 4, 1.0, x, 4, x, 4, 0.0, x, 4, dev=3)


# ------------------------------------------------------------------ tcgen05 3xTF32 kernel
@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_tc3x_transposes_alpha_beta(ctx, ta, tb):
    check(ctx, TC3X, ta, tb, 256, 256, 64, 1.0, 0.0)
    check(ctx, TC3X, ta, tb, 512, 768, 320, 1.5, 0.5)
    r, q = check(ctx, TC3X, ta, tb, 1024, 1024, 1024, 1.5, 0.5)
    assert q < 64.0, q      # 3xTF32 keeps the error at the fp32 level, independent of K's bound


def test_tc3x_ragged_and_padded(ctx):
    check(ctx, TC3X, 0, 0, 300, 260, 100, 1.0, 0.0)
    check(ctx, TC3X, 1, 0, 257, 255, 77, 2.0, -1.0, pad=(4, 0, 4))
    check(ctx, TC3X, 0, 1, 129, 513, 130, 1.0, 1.0, pad=(1, 3, 5))      # unaligned leading dims: scalar epilogue
    # k < 4 asked of the tensor-core path is served by the exact FFMA kernel (see the worst-case test below)
    check(ctx, TC3X, 1, 1, 640, 130, 1, 1.0, 0.5)
    check(ctx, TC3X, 1, 1, 640, 130, 4, 1.0, 0.5)
    check(ctx, TC3X, 0, 0, 1, 1, 4096, 1.0, 0.0)                         # one element of C


@pytest.mark.parametrize("k", [1, 2, 3])
def test_k_below_4_with_worst_case_split_residues_is_exact_fp32(ctx, k):
    """Inputs whose low 13 mantissa bits are all set leave the largest possible residue after the hi/lo
    split: a 3xTF32 product of two such numbers is off by up to ~12 * 2^-24 |a b|, more than the
    half-budget bound 4*K*2^-24 allows for K < 4.  A forced tensor-path request below K = 4 therefore runs
    on the FFMA kernel, whose K <= 3 products and sums are within one fp32 rounding each."""
    m, n = 256, 256
    rng = np.random.default_rng(5)
    def worst(shape):
        x = rng.uniform(1.0, 2.0, size=shape).astype(np.float32)
        bits = x.view(np.uint32) | np.uint32(0x1FFF)          # maximal lo residue, lo*lo term maximal too
        return (bits.view(np.float32) * rng.choice([-1.0, 1.0], size=shape)).astype(np.float32)
    a, b = worst((m, k)), worst((k, n))
    c0 = np.zeros((m, n), np.float32)
    out = run_gemm(ctx, TC3X, 0, 0, m, n, k, 1.0, a.ravel(), k, 0, b.ravel(), n, 0, 0.0, c0.ravel(), n, 0, 1)
    ref, absab = og.gemm_f64_np(0, 0, m, n, k, 1.0, a, k, 0, b, n, 0, 0.0, c0, n, 0, 1)
    r, q = og.tolerance_ratio(out.reshape(1, m, n), ref, absab, k, budget=BUDGET)
    assert r <= 1.0, (r, q)
    assert q <= k + 1.0, q        # fp32 products summed in fp32: about one rounding per term


def test_tc3x_beta_zero_ignores_nan_c(ctx):
    check(ctx, TC3X, 0, 0, 512, 512, 128, 1.0, 0.0, poison_c=True)


def test_tc3x_batched(ctx):
    check(ctx, TC3X, 0, 0, 512, 512, 512, 1.0, 0.0, batch=8, dist="normal")
    check(ctx, TC3X, 1, 0, 200, 300, 150, 0.5, 2.0, batch=5)
    check(ctx, TC3X, 0, 1, 256, 256, 256, 1.0, 1.0, batch=3, pad=(4, 4, 4))


def test_tc3x_many_tiles_persistent(ctx):
    # more tiles than SMs: exercises the persistent loop, the ring phases and TMEM hand-over
    check(ctx, TC3X, 0, 0, 4096, 3072, 96, 1.0, 0.5)
    check(ctx, TC3X, 0, 0, 256, 256, 48, 1.0, 0.0, batch=400)


def test_tc3x_split_k_tail_integer_exact(ctx):
    """Problems with fewer tiles than SMs are cut along K; partial accumulators travel through
    global scratch and are added by the owning CTA.  Integer inputs make the result exact under
    any summation order, so every element must match."""
    rng = np.random.default_rng(99)
    for (batch, m, n, k, ta, tb, alpha, beta) in [(1, 1024, 768, 512, 0, 0, 1.0, 0.0), (1, 512, 512, 2048, 1, 0, 2.0, 1.0),
                                                   (3, 512, 256, 384, 0, 1, 1.0, -1.0), (1, 2048, 2048, 1024, 0, 0, 1.0, 0.0),
                                                   (1, 300, 700, 1000, 1, 1, -1.0, 1.0),
                                                   # one tile cut 16 ways, every CTA finishing 16 of its rows; ragged single tile
                                                   (1, 256, 256, 4096, 0, 0, 1.0, 1.0), (1, 200, 250, 2100, 0, 1, 2.0, -1.0),
                                                   (1, 1024, 1024, 1024, 0, 0, 1.0, 0.0), (2, 512, 768, 2048, 1, 0, 1.0, 1.0)]:
        ar, ac = (k, m) if ta else (m, k)
        br, bc = (n, k) if tb else (k, n)
        a = rng.integers(-3, 4, size=(batch, ar, ac)).astype(np.float32)
        b = rng.integers(-3, 4, size=(batch, br, bc)).astype(np.float32)
        c = rng.integers(-8, 9, size=(batch, m, n)).astype(np.float32)
        opa = a.transpose(0, 2, 1) if ta else a
        opb = b.transpose(0, 2, 1) if tb else b
        want = (alpha * np.matmul(opa.astype(np.int64), opb.astype(np.int64)) + beta * c).astype(np.float32)
        got = run_gemm(ctx, TC3X, ta, tb, m, n, k, alpha, a.ravel(), ac, ar * ac, b.ravel(), bc, br * bc, beta, c.ravel(),
                       n, m * n, batch).reshape(batch, m, n)
        assert np.array_equal(got, want), (m, n, k, int(np.count_nonzero(got != want)))
    # repeated launches reuse the exchange area with a new epoch each time
    for _ in range(5):
        check(ctx, TC3X, 0, 0, 1024, 1024, 640, 1.5, 0.5)
    # the ReLU epilogue on a cut tile
    m, n, k = 512, 512, 3000
    a = rng.integers(-3, 4, size=(m, k)).astype(np.float32)
    b = rng.integers(-3, 4, size=(k, n)).astype(np.float32)
    c = rng.integers(-8, 9, size=(m, n)).astype(np.float32)
    dc = dev(c)
    ctx.set_gemm_variant(TC3X)
    ctx.sgemm_strided_batched_ex(0, 0, m, n, k, 1.0, dev(a), k, 0, dev(b), n, 0, 1.0, dc, n, 0, 1, epilogue=1)
    ctx.sync()
    ctx.set_gemm_variant(AUTO)
    want = np.maximum(a.astype(np.int64) @ b.astype(np.int64) + c, 0).astype(np.float32)
    assert np.array_equal(dc.cpu().numpy(), want)


def test_tc3x_in_kernel_split_paths(ctx):
    """Operands whose k index is contiguous are fetched raw by TMA and split inside the kernel
    (NT: both operands, NN: A, TT: B); unaligned leading dimensions fall back to the pre-pass.
    Ragged M, N, K rely on TMA zero fill."""
    for (ta, tb) in [(0, 1), (0, 0), (1, 1), (1, 0)]:
        check(ctx, TC3X, ta, tb, 300, 260, 100, 1.5, 0.5)                 # ragged everything, aligned ld
        check(ctx, TC3X, ta, tb, 1024, 512, 1000, 1.0, 0.0, pad=(4, 8, 0))  # padded but aligned ld
        check(ctx, TC3X, ta, tb, 257, 129, 77, 1.0, 1.0, pad=(1, 3, 0))     # ld % 4 != 0: pre-pass fallback
        check(ctx, TC3X, ta, tb, 512, 256, 333, 1.0, 0.0, batch=5)
    # row-contiguous operands are transposed by the converters: integer-exact in every storage order, ragged tiles
    rng = np.random.default_rng(6)
    for (ta, tb) in [(1, 0), (0, 0), (1, 1)]:
        m, n, k = 1000, 520, 328
        a = rng.integers(-3, 4, size=(k, m) if ta else (m, k)).astype(np.float32)
        b = rng.integers(-3, 4, size=(n, k) if tb else (k, n)).astype(np.float32)
        opa = (a.T if ta else a).astype(np.int64)
        opb = (b.T if tb else b).astype(np.int64)
        got = run_gemm(ctx, TC3X, ta, tb, m, n, k, 1.0, a.ravel(), a.shape[1], 0, b.ravel(), b.shape[1], 0, 0.0,
                       np.zeros(m * n, np.float32), n, 0, 1).reshape(m, n)
        assert np.array_equal(got, (opa @ opb).astype(np.float32)), (ta, tb)
    # integer-exact on the fully in-kernel path (NT) with split-K on top
    rng = np.random.default_rng(5)
    m, n, k = 1024, 768, 520
    a = rng.integers(-3, 4, size=(m, k)).astype(np.float32)
    b = rng.integers(-3, 4, size=(n, k)).astype(np.float32)
    got = run_gemm(ctx, TC3X, 0, 1, m, n, k, 1.0, a.ravel(), k, 0, b.ravel(), k, 0, 0.0, np.zeros(m * n, np.float32),
                   n, 0, 1).reshape(m, n)
    assert np.array_equal(got, (a.astype(np.int64) @ b.astype(np.int64).T).astype(np.float32))


def test_auto_matches_explicit_variants(ctx):
    # AUTO picks SIMT for small problems and TC3X for large ones; both are within tolerance
    check(ctx, AUTO, 0, 0, 96, 80, 40, 1.0, 0.0)
    check(ctx, AUTO, 0, 0, 2048, 2048, 512, 1.0, 0.0)


# ------------------------------------------------------------------ benchmark configurations
def test_config1_1024_cubed(ctx):
    # M=N=K=1024, NN, alpha=1, beta=0, A,B ~ U[-1,1), C zero-initialised
    for variant in (SIMT, TC3X, AUTO):
        check(ctx, variant, 0, 0, 1024, 1024, 1024, 1.0, 0.0, seed=20240601)


def _sampled_check(ctx, ta, tb, m, n, k, alpha, beta, a_t, b_t, c_in_t, c_out_t, rows, ldc=None):
    """fp64 check of selected rows of a large result (device tensors, row-major dense)."""
    rows_t = torch.as_tensor(rows, device="cuda")
    a_rows = (a_t[:, rows_t].T if ta else a_t[rows_t, :]).double().cpu().numpy()     # len(rows) x k
    opb = (b_t.T if tb else b_t).double().cpu().numpy()                               # k x n
    ref = float(np.float32(alpha)) * (a_rows @ opb)
    absab = np.abs(a_rows) @ np.abs(opb)
    cin = None
    if beta != 0.0:
        cin = c_in_t[rows_t, :].double().cpu().numpy()
        ref = ref + float(np.float32(beta)) * cin
    got = c_out_t[rows_t, :].cpu().numpy()
    return og.tolerance_ratio(got, ref, absab, k, beta=beta, c_in=cin, budget=BUDGET)


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_config2_4096_cubed(ctx, ta, tb):
    # M=N=K=4096, alpha=1.5, beta=0.5, A,B,C ~ U[-1,1); 256 sampled rows checked in fp64
    n = 4096
    a = torch.empty(n, n, device="cuda"); b = torch.empty_like(a); c = torch.empty_like(a)
    ctx.fill_uniform(a, n * n, 20240601); ctx.fill_uniform(b, n * n, 20240602); ctx.fill_uniform(c, n * n, 20240603)
    ctx.sync()
    # the device generator is bit-identical to the host one
    assert np.array_equal(a[0, :1000].cpu().numpy(), og.uniform_pm1(20240601, 1000))
    c_in = c.clone()
    ctx.sgemm(ta, tb, n, n, n, 1.5, a, n, b, n, 0.5, c, n)
    ctx.sync()
    rows = np.random.default_rng(7).choice(n, 256, replace=False)
    r, q = _sampled_check(ctx, ta, tb, n, n, n, 1.5, 0.5, a, b, c_in, c, rows)
    assert r <= 1.0 and q < 128.0, (r, q)
    # linearity property over the full matrix: GEMM(2A, B, beta=0) == 2 * GEMM(A, B, beta=0) exactly
    c1 = torch.empty_like(a); c2 = torch.empty_like(a)
    ctx.sgemm(ta, tb, n, n, n, 1.0, a, n, b, n, 0.0, c1, n)
    a2 = a * 2
    ctx.sgemm(ta, tb, n, n, n, 1.0, a2, n, b, n, 0.0, c2, n)
    ctx.sync()
    assert torch.equal(c2, c1 * 2)


def test_config3_batched_512(ctx):
    # batch of 512^3 NN, alpha=1, beta=0, A,B ~ N(0,1): 32 batches checked fully in fp64, and the
    # full 256-batch call must equal per-batch calls bit for bit (batch entries are independent)
    m = 512; batch = 256
    g = torch.Generator(device="cuda"); g.manual_seed(20240601)
    a = torch.randn(batch, m, m, device="cuda", generator=g)
    b = torch.randn(batch, m, m, device="cuda", generator=g)
    c = torch.full((batch, m, m), float("nan"), device="cuda")
    ctx.sgemm_strided_batched(0, 0, m, m, m, 1.0, a, m, m * m, b, m, m * m, 0.0, c, m, m * m, batch)
    ctx.sync()
    idx = list(range(0, batch, 8))
    a64 = a[idx].double().cpu().numpy(); b64 = b[idx].double().cpu().numpy()
    ref = a64 @ b64; absab = np.abs(a64) @ np.abs(b64)
    r, q = og.tolerance_ratio(c[idx].cpu().numpy(), ref, absab, m, budget=BUDGET)
    assert r <= 1.0 and q < 64.0, (r, q)
    # batch entries are independent: a single-entry call agrees with the batched one (to rounding:
    # a lone 512^3 problem is cut along K over more CTAs, which reorders the fp32 summation)
    single = torch.empty(m, m, device="cuda")
    ctx.set_gemm_variant(TC3X)
    for i in (0, 37, 255):
        ctx.sgemm(0, 0, m, m, m, 1.0, a[i], m, b[i], m, 0.0, single, m)
        ctx.sync()
        a64 = a[i].double().cpu().numpy(); b64 = b[i].double().cpu().numpy()
        r1, _ = og.tolerance_ratio(single.cpu().numpy(), a64 @ b64, np.abs(a64) @ np.abs(b64), m, budget=BUDGET)
        assert r1 <= 1.0
        assert float((single - c[i]).abs().max()) <= 2.0 ** -18 * float(c[i].abs().max())
    ctx.set_gemm_variant(AUTO)


def test_config4_tall_skinny(ctx):
    # M=65536, N=256, K=4096, NN, A ~ U[-1,1), B ~ N(0, 0.02); 512 sampled rows in fp64
    m, n, k = 65536, 256, 4096
    a = torch.empty(m, k, device="cuda")
    ctx.fill_uniform(a, m * k, 20240601); ctx.sync()
    b = dev(og.normal(20240602, k * n, std=0.02).reshape(k, n))
    c = torch.full((m, n), float("nan"), device="cuda")
    ctx.sgemm(0, 0, m, n, k, 1.0, a, k, b, n, 0.0, c, n)
    ctx.sync()
    rows = np.random.default_rng(8).choice(m, 512, replace=False)
    r, q = _sampled_check(ctx, 0, 0, m, n, k, 1.0, 0.0, a, b, None, c, rows)
    assert r <= 1.0 and q < 128.0, (r, q)
    assert bool(torch.isfinite(c).all())


# ------------------------------------------------------------------ fused activation epilogue
@pytest.mark.parametrize("variant", [SIMT, TC3X])
def test_relu_epilogue_and_standalone_relu(ctx, variant):
    """C <- relu(alpha*op(A)*op(B) + beta*C) in the GEMM epilogue equals GEMM followed by the
    standalone in-place ReLU bit for bit, and lies within the GEMM tolerance of relu(oracle)
    (|relu(x) - relu(y)| <= |x - y|)."""
    for (ta, tb, m, n, k, alpha, beta, batch) in [(0, 0, 300, 260, 100, 1.0, 0.0, 1), (1, 0, 512, 256, 384, 1.5, 0.5, 2),
                                                   (0, 1, 129, 65, 33, -1.0, 1.0, 1)]:
        cs = make_case(321, ta, tb, m, n, k, batch)
        ctx.set_gemm_variant(variant)
        da, db = dev(cs["a"]), dev(cs["b"])
        c_fused, c_two = dev(cs["c"].copy()), dev(cs["c"].copy())
        ctx.sgemm_strided_batched_ex(ta, tb, m, n, k, alpha, da, cs["lda"], cs["sa"], db, cs["ldb"], cs["sb"], beta,
                                     c_fused, cs["ldc"], cs["sc"], batch, 1)
        ctx.sgemm_strided_batched_ex(ta, tb, m, n, k, alpha, da, cs["lda"], cs["sa"], db, cs["ldb"], cs["sb"], beta,
                                     c_two, cs["ldc"], cs["sc"], batch, 0)
        ctx.relu(c_two, c_two.numel())
        ctx.sync()
        ctx.set_gemm_variant(AUTO)
        assert torch.equal(c_fused, c_two)
        ref, absab = og.gemm_f64_np(ta, tb, m, n, k, alpha, cs["a"], cs["lda"], cs["sa"], cs["b"], cs["ldb"], cs["sb"],
                                    beta, cs["c"], cs["ldc"], cs["sc"], batch)
        got = c_fused.cpu().numpy().reshape(batch, m, n)
        assert got.min() >= 0.0
        r, _ = og.tolerance_ratio(got, np.maximum(ref, 0.0), absab, k, beta=beta, c_in=cs["c"].reshape(batch, m, n),
                                  budget=BUDGET)
        assert r <= 1.0, r
    x = torch.tensor([-2.0, -0.5, 0.0, 3.5, float("nan")], device="cuda")     # reference's ReLU vector + NaN -> 0
    ctx.relu(x, 5); ctx.sync()
    assert x.tolist() == [0.0, 0.0, 0.0, 3.5, 0.0]
    from sushiblas_b200 import SushiCudaError
    with pytest.raises(SushiCudaError):
        ctx.sgemm_strided_batched_ex(0, 0, 4, 4, 4, 1.0, x, 4, 0, x, 4, 0, 0.0, x, 4, 0, 1, 7)   # unknown epilogue


# ------------------------------------------------------------------ SYRK on the GEMM main loop
def test_reference_kat_syrk(ctx):
    g = np.load(GOLDEN)
    # tests/blas/level3/test_syrk.cpp:39-63: row-major, lower, A 3x2
    c = torch.zeros(9, device="cuda")
    ctx.ssyrk(False, False, 3, 2, 1.0, dev(g["ref_syrk_lower3.a"]), 2, 0.0, c, 3)
    ctx.sync()
    assert np.array_equal(c.cpu().numpy(), g["ref_syrk_lower3.c_out"])
    # tests/blas/level3/test_syrk.cpp:65-88: column-major lower with transA == row-major upper without
    c = torch.zeros(4, device="cuda")
    ctx.ssyrk(True, False, 2, 3, 1.0, dev(g["ref_syrk_colmajor_trans.a"]), 3, 0.0, c, 2)
    ctx.sync()
    assert np.array_equal(c.cpu().numpy(), g["ref_syrk_colmajor_trans.c_out"])


@pytest.mark.parametrize("variant", [SIMT, TC3X])
def test_syrk_matches_oracle_and_leaves_the_other_triangle(ctx, variant):
    rng = np.random.default_rng(23)
    ctx.set_gemm_variant(variant)
    # (2304, 136): 45 tiles of the triangle in a 9 x 9 tile grid -- the tensor kernel numbers only those
    for (n, k, batch, pad) in [(7, 5, 1, 0), (65, 33, 2, 3), (300, 260, 1, 4), (512, 384, 3, 0), (1024, 200, 1, 0),
                                (257, 1000, 1, 1), (2304, 136, 2, 0)]:
        for upper in (0, 1):
            for trans in (0, 1):
                alpha, beta = float(rng.choice([1.0, 1.5])), float(rng.choice([0.0, 0.5, 1.0]))
                ar, ac = (k, n) if trans else (n, k)
                lda, ldc = ac + pad, n + pad
                sa, sc = ar * lda, n * ldc
                a = og.uniform_pm1(int(rng.integers(1 << 30)), batch * sa)
                c0 = og.uniform_pm1(int(rng.integers(1 << 30)), batch * sc)
                c_in = c0.copy()
                if beta == 0.0:
                    # the written triangle is not read when beta == 0: poison it
                    v = og._view(c_in, n, ldc, ldc, sc, batch).copy()
                    i, j = np.indices((n, n))
                    tri = (j >= i) if upper else (j <= i)
                    v[:, :, :n][np.broadcast_to(tri, (batch, n, n))] = np.nan
                    c_in = v.reshape(batch, n * ldc)[:, :sc].ravel().copy()
                dc = dev(c_in)
                ctx.ssyrk(upper, trans, n, k, alpha, dev(a), lda, beta, dc, ldc, sa, sc, batch)
                ctx.sync()
                out = dc.cpu().numpy()
                ref, absaa, mask = og.syrk_f64_np(upper, trans, n, k, alpha, a, lda, sa, beta, c0, ldc, sc, batch)
                got = og._view(out, n, n, ldc, sc, batch)
                cin = og._view(c0, n, n, ldc, sc, batch)
                r, _ = og.tolerance_ratio(np.where(mask[None], got, 0.0), np.where(mask[None], ref, 0.0), absaa, k,
                                          beta=beta, c_in=np.where(mask[None], cin, 0.0), budget=BUDGET)
                assert r <= 1.0, (variant, n, k, batch, upper, trans, alpha, beta, r)
                # everything outside the triangle (other triangle and row padding) keeps its bits
                keep = np.ones(out.shape, dtype=bool)
                idx = (np.arange(batch)[:, None, None] * sc + np.arange(n)[None, :, None] * ldc + np.arange(n)[None, None, :])
                keep[idx[np.broadcast_to(mask, (batch, n, n))]] = False
                assert np.array_equal(out[keep], c_in[keep]), (variant, n, k, upper, trans)
    ctx.set_gemm_variant(AUTO)
    # k == 0: only beta * C on the triangle
    c = torch.ones(16, device="cuda")
    ctx.ssyrk(False, False, 4, 0, 1.0, c, 1, 0.5, c, 4)
    ctx.sync()
    assert c.view(4, 4).cpu().numpy().tolist() == [[0.5, 1, 1, 1], [0.5, 0.5, 1, 1], [0.5, 0.5, 0.5, 1], [0.5] * 4]


# ------------------------------------------------------------------ grouped launch of small GEMMs
def test_grouped_small_gemms(ctx):
    """Independent small problems of mixed shapes, transposes, alpha/beta and epilogues in one
    call equal the same problems run one by one (same FFMA kernel body) bit for bit; a large
    problem in the list takes the tensor-core path and stays within tolerance."""
    rng = np.random.default_rng(17)
    probs, singles = [], []
    for i in range(200):
        m, n, k = (int(rng.choice([1, 3, 8, 17, 32, 64, 65, 100])) for _ in range(3))
        ta, tb = int(rng.integers(2)), int(rng.integers(2))
        batch = int(rng.choice([1, 1, 2]))
        cs = make_case(1000 + i, ta, tb, m, n, k, batch, pad=(int(rng.integers(3)), 0, int(rng.integers(3))))
        alpha, beta = float(rng.choice([1.0, -0.5])), float(rng.choice([0.0, 1.0, 0.5]))
        epi = int(rng.integers(2))
        da, db = dev(cs["a"]), dev(cs["b"])
        c_grp, c_one = dev(cs["c"].copy()), dev(cs["c"].copy())
        probs.append(dict(trans_a=ta, trans_b=tb, m=m, n=n, k=k, alpha=alpha, beta=beta, a=da, lda=cs["lda"],
                          stride_a=cs["sa"], b=db, ldb=cs["ldb"], stride_b=cs["sb"], c=c_grp, ldc=cs["ldc"],
                          stride_c=cs["sc"], batch=batch, epilogue=epi))
        singles.append((c_one, c_grp))
    before = ctx.launch_count()
    ctx.sgemm_grouped(probs)
    assert ctx.launch_count() - before == 1          # one kernel for all 200 problems
    ctx.set_gemm_variant(SIMT)
    for q, (c_one, _) in zip(probs, singles):
        ctx.sgemm_strided_batched_ex(q["trans_a"], q["trans_b"], q["m"], q["n"], q["k"], q["alpha"], q["a"], q["lda"],
                                     q["stride_a"], q["b"], q["ldb"], q["stride_b"], q["beta"], c_one, q["ldc"],
                                     q["stride_c"], q["batch"], q["epilogue"])
    ctx.sync()
    ctx.set_gemm_variant(AUTO)
    for i, (c_one, c_grp) in enumerate(singles):
        assert torch.equal(c_one, c_grp), i
    # a list mixing a big problem (tensor-core path) with small ones
    big = make_case(5, 0, 0, 1024, 1024, 512)
    dA, dB, dC = dev(big["a"]), dev(big["b"]), dev(big["c"].copy())
    small = probs[:3]
    ctx.sgemm_grouped([dict(m=1024, n=1024, k=512, a=dA, lda=512, b=dB, ldb=1024, c=dC, ldc=1024)] + small)
    ctx.sync()
    ref, absab = og.gemm_f64_np(0, 0, 1024, 1024, 512, 1.0, big["a"], 512, 0, big["b"], 1024, 0, 0.0, None, 1024, 0, 1)
    r, _ = og.tolerance_ratio(dC.cpu().numpy().reshape(1, 1024, 1024), ref, absab, 512, budget=BUDGET)
    assert r <= 1.0
    ctx.sgemm_grouped([])                            # empty list: no-op


# ------------------------------------------------------------------ host-buffer entry point and storage calls
def test_host_entry_point_matches_device_path(ctx):
    m, n, k, batch = 300, 200, 150, 2
    cs = make_case(55, 0, 1, m, n, k, batch, pad=(0, 0, 4))
    c_host = cs["c"].copy()
    ctx.sgemm_strided_batched_host(0, 1, m, n, k, 1.5, cs["a"], cs["lda"], cs["sa"], cs["b"], cs["ldb"], cs["sb"],
                                   0.5, c_host, cs["ldc"], cs["sc"], batch)
    ctx.sync()
    out = run_gemm(ctx, AUTO, 0, 1, m, n, k, 1.5, cs["a"], cs["lda"], cs["sa"], cs["b"], cs["ldb"], cs["sb"], 0.5,
                   cs["c"].copy(), cs["ldc"], cs["sc"], batch)
    assert np.array_equal(c_host, out)
    # beta == 0 with a padded C: the gaps between rows survive the copy back
    c_host = cs["c"].copy()
    ctx.sgemm_strided_batched_host(0, 1, m, n, k, 1.0, cs["a"], cs["lda"], cs["sa"], cs["b"], cs["ldb"], cs["sb"],
                                   0.0, c_host, cs["ldc"], cs["sc"], batch)
    ctx.sync()
    v = og._view(c_host, m, cs["ldc"], cs["ldc"], cs["sc"], batch)
    assert np.array_equal(v[:, :, n:], og._view(cs["c"], m, cs["ldc"], cs["ldc"], cs["sc"], batch)[:, :, n:])


@pytest.mark.parametrize("ta,tb", [(0, 0), (1, 0), (0, 1), (1, 1)])
def test_host_entry_point_chunked_pipeline(ctx, ta, tb):
    """Above 32 MiB the host-buffer call uploads, multiplies and downloads in four chunks on
    separate copy streams; the result must equal the device path on the same data."""
    m, n, k = 2304, 2048, 1800                       # 2304 rows: chunks of 768 (last one shorter after rounding)
    cs = make_case(77, ta, tb, m, n, k)
    ctx.set_gemm_variant(TC3X)
    for beta in (0.5, 0.0):
        c_host = cs["c"].copy()
        ctx.sgemm_strided_batched_host(ta, tb, m, n, k, 1.5, cs["a"], cs["lda"], 0, cs["b"], cs["ldb"], 0, beta, c_host,
                                       cs["ldc"], 0, 1)
        # a second call right behind the first reuses the staging buffers
        c_host2 = cs["c"].copy()
        ctx.sgemm_strided_batched_host(ta, tb, m, n, k, 1.5, cs["a"], cs["lda"], 0, cs["b"], cs["ldb"], 0, beta, c_host2,
                                       cs["ldc"], 0, 1)
        ctx.sync()
        ref, absab = og.gemm_f64_np(ta, tb, m, n, k, 1.5, cs["a"], cs["lda"], 0, cs["b"], cs["ldb"], 0, beta, cs["c"],
                                    cs["ldc"], 0, 1)
        r, _ = og.tolerance_ratio(c_host.reshape(1, m, n), ref, absab, k, beta=beta, c_in=cs["c"].reshape(1, m, n),
                                  budget=BUDGET)
        assert r <= 1.0, (ta, tb, beta, r)
        assert np.array_equal(c_host, c_host2)
    ctx.set_gemm_variant(AUTO)
    # batched: chunks of batch entries
    batch, m, n, k = 10, 512, 384, 640
    cs = make_case(78, ta, tb, m, n, k, batch)
    c_host = cs["c"].copy()
    ctx.sgemm_strided_batched_host(ta, tb, m, n, k, 1.0, cs["a"], cs["lda"], cs["sa"], cs["b"], cs["ldb"], cs["sb"], 1.0,
                                   c_host, cs["ldc"], cs["sc"], batch)
    ctx.sync()
    ref, absab = og.gemm_f64_np(ta, tb, m, n, k, 1.0, cs["a"], cs["lda"], cs["sa"], cs["b"], cs["ldb"], cs["sb"], 1.0,
                                cs["c"], cs["ldc"], cs["sc"], batch)
    r, _ = og.tolerance_ratio(c_host.reshape(batch, m, n), ref, absab, k, beta=1.0, c_in=cs["c"].reshape(batch, m, n),
                              budget=BUDGET)
    assert r <= 1.0, (ta, tb, r)


def test_row_sharded_host_entry_on_one_rank(ctx):
    """The host-buffer form of the row-sharded GEMM without a communicator (one rank owns everything): B goes up
    whole, A and C move in row chunks that overlap the multiplication.  Chunked and unchunked sizes, transposes,
    beta != 0 (C goes up first) and a padded C."""
    import ctypes

    def pinned(arr):
        ptr = ctx.host_alloc(arr.nbytes)
        view = np.frombuffer((ctypes.c_float * arr.size).from_address(ptr), dtype=np.float32)
        view[:] = arr.reshape(-1)
        return ptr, view

    for (m, n, k, ta, tb, alpha, beta, padc) in [(4608, 640, 520, 0, 0, 1.0, 0.0, 0), (4100, 384, 300, 1, 1, 1.5, 0.5, 0),
                                                 (700, 200, 96, 0, 1, 1.0, 1.0, 3), (2304, 512, 256, 1, 0, 2.0, 0.0, 0)]:
        cs = make_case(300 + m % 97, ta, tb, m, n, k, 1, pad=(0, 0, padc))
        pa, ha = pinned(cs["a"]); pb, hb = pinned(cs["b"]); pc, hc = pinned(cs["c"])
        da = torch.empty(cs["a"].size, device="cuda"); db = torch.empty(cs["b"].size, device="cuda")
        dc = torch.full((cs["c"].size,), float("nan"), device="cuda")
        ctx.set_gemm_variant(TC3X if m >= 1024 else AUTO)
        ctx.sgemm_row_sharded_host(ta, tb, m, n, k, alpha, ha, cs["lda"], hb, cs["ldb"], beta, hc, cs["ldc"], da, db, dc)
        ctx.sync()
        ctx.set_gemm_variant(AUTO)
        ref, absab = og.gemm_f64_np(ta, tb, m, n, k, alpha, cs["a"], cs["lda"], 0, cs["b"], cs["ldb"], 0, beta, cs["c"], cs["ldc"], 0, 1)
        got = og._view(hc.copy(), m, n, cs["ldc"], 0, 1)
        cin = og._view(cs["c"], m, n, cs["ldc"], 0, 1)
        r, _ = og.tolerance_ratio(got, ref, absab, k, beta=beta, c_in=cin, budget=BUDGET)
        assert r <= 1.0, (m, n, k, ta, tb, r)
        if padc:                                             # the padding columns of the host C keep their contents
            full = hc.reshape(m, cs["ldc"]); orig = cs["c"].reshape(m, cs["ldc"])
            assert np.array_equal(full[:, n:], orig[:, n:])
        for ptr in (pa, pb, pc):
            ctx.host_free(ptr)


def test_storage_calls_round_trip(ctx):
    nbytes = 1 << 20
    d = ctx.malloc(nbytes)
    h = ctx.host_alloc(nbytes)
    import ctypes
    src = (ctypes.c_uint8 * nbytes).from_address(h)
    pattern = np.arange(nbytes, dtype=np.uint8)
    np.frombuffer(src, dtype=np.uint8)[:] = pattern
    ctx.memcpy_h2d(d, h, nbytes)
    d2 = ctx.malloc(nbytes)
    ctx.memcpy_d2d(d2, d, nbytes)
    ctx.memset(d, 0, nbytes)
    back = np.empty(nbytes, dtype=np.uint8)
    ctx.memcpy_d2h(back, d2, nbytes)
    zero = np.ones(nbytes, dtype=np.uint8)
    ctx.memcpy_d2h(zero, d, nbytes)
    ctx.sync()
    assert np.array_equal(back, pattern) and not zero.any()
    ctx.free(d); ctx.free(d2); ctx.host_free(h)


def test_uploads_ahead_of_and_downloads_behind_queued_work(ctx):
    """upload_ahead / download_behind move data on streams of their own and are ordered against the device's
    stream only where they must be.  Operands uploaded ahead are seen by the GEMM enqueued after them although a
    long GEMM was queued before; a result downloaded behind its marker is complete at sync() although another
    long GEMM was queued after the marker; work enqueued after the download does not overwrite its source under
    it; the bytes are counted like those of the plain copies."""
    import ctypes
    m, n, k, big = 1024, 768, 512, 4096
    cs = make_case(77, 0, 0, m, n, k, 1)

    def pinned(arr):
        ptr = ctx.host_alloc(arr.nbytes)
        view = np.frombuffer((ctypes.c_float * arr.size).from_address(ptr), dtype=np.float32)
        view[:] = arr.reshape(-1)
        return ptr, view

    pa, _ = pinned(cs["a"]); pb, _ = pinned(cs["b"])
    pc, hc = pinned(np.full(m * n, np.nan, dtype=np.float32))
    da = torch.empty(m * k, device="cuda"); db = torch.empty(k * n, device="cuda")
    dc = torch.full((m * n,), float("nan"), device="cuda")
    x = torch.randn(big * big, device="cuda"); z = torch.empty(big * big, device="cuda")
    torch.cuda.synchronize()
    up0, down0 = ctx.copy_bytes()
    ctx.upload_fence()
    ctx.sgemm(0, 0, big, big, big, 1.0, x, big, x, big, 0.0, z, big)       # the uploads run beside this one
    ctx.upload_ahead(da, pa, cs["a"].nbytes)
    ctx.upload_ahead(db, pb, cs["b"].nbytes)
    ctx.sgemm(0, 0, m, n, k, 1.0, da, cs["lda"], db, cs["ldb"], 0.0, dc, n)
    marker = ctx.marker_create()
    ctx.marker_record(marker)
    ctx.sgemm(0, 0, big, big, big, 1.0, x, big, x, big, 0.0, z, big)       # the download does not wait for this one
    ctx.download_behind(pc, dc, m * n * 4, marker)
    ctx.memset(dc, 0, m * n * 4)                                           # enqueued after the download
    ctx.sync()
    up1, down1 = ctx.copy_bytes()
    assert (up1 - up0, down1 - down0) == (cs["a"].nbytes + cs["b"].nbytes, m * n * 4)
    ref, absab = og.gemm_f64_np(0, 0, m, n, k, 1.0, cs["a"], cs["lda"], 0, cs["b"], cs["ldb"], 0, 0.0,
                                np.zeros(m * n, dtype=np.float32), n, 0, 1)
    r, _ = og.tolerance_ratio(og._view(hc.copy(), m, n, n, 0, 1), ref, absab, k, budget=BUDGET)
    assert r <= 1.0, r
    assert not dc.any().item()
    ctx.marker_destroy(marker)
    for ptr in (pa, pb, pc):
        ctx.host_free(ptr)


def test_injected_host_side_failures_are_reported_and_survivable(ctx):
    own = SushiCuda([0])                         # a context of its own: its scratch starts empty
    own.set_stream(torch.cuda.current_stream().cuda_stream)
    try:
        _injected_failures(own)
    finally:
        torch.cuda.synchronize()
        own.close()


def _injected_failures(ctx):
    """Failure paths that cannot be provoked on a healthy machine are reached through the host-side hook
    (nothing on the GPU faults): a device allocation, the library's own scratch allocation inside a GEMM, a
    pinned-host allocation and the communicator initialisation each return their error code once, name the
    injection in the message, and leave the context usable."""
    FAIL_DEVICE_ALLOC, FAIL_COMM_INIT, FAIL_HOST_ALLOC = 1, 2, 3
    copies_before = ctx.copy_bytes()
    ctx.inject_failure(FAIL_DEVICE_ALLOC, 1)
    with pytest.raises(SushiCudaError) as e:
        ctx.malloc(1 << 20)
    assert e.value.code == -4 and "injected" in str(e.value)
    p = ctx.malloc(1 << 20)                      # the next call is served again
    ctx.free(p)
    ctx.inject_failure(FAIL_HOST_ALLOC, 2)       # the second next one
    h = ctx.host_alloc(4096)
    with pytest.raises(SushiCudaError) as e:
        ctx.host_alloc(4096)
    assert e.value.code == -4
    ctx.host_free(h)
    # scratch of the tensor path: an unaligned leading dimension forces the pre-pass, whose planes are larger than
    # anything this context has needed so far
    m, n, k = 1536, 1280, 6148
    cs = make_case(91, 0, 0, m, n, k, 1, pad=(1, 0, 0))
    da, db, dc = dev(cs["a"]), dev(cs["b"]), dev(cs["c"])
    ctx.set_gemm_variant(TC3X)
    ctx.inject_failure(FAIL_DEVICE_ALLOC, 1)
    with pytest.raises(SushiCudaError) as e:
        ctx.sgemm(0, 0, m, n, k, 1.0, da, cs["lda"], db, cs["ldb"], 0.0, dc, cs["ldc"])
    assert e.value.code == -4 and "scratch" in str(e.value)
    ctx.sgemm(0, 0, m, n, k, 1.0, da, cs["lda"], db, cs["ldb"], 0.0, dc, cs["ldc"])
    ctx.sync()
    ctx.set_gemm_variant(AUTO)
    ref, absab = og.gemm_f64_np(0, 0, m, n, k, 1.0, cs["a"], cs["lda"], 0, cs["b"], cs["ldb"], 0, 0.0, cs["c"], cs["ldc"], 0, 1)
    r, _ = og.tolerance_ratio(dc.cpu().numpy().reshape(1, m, n), ref, absab, k, budget=BUDGET)
    assert r <= 1.0
    ctx.inject_failure(FAIL_COMM_INIT, 1)
    with pytest.raises(SushiCudaError) as e:
        ctx.comm_init_rank(bytes(128), 1, 0)
    assert e.value.code == -6 and "injected" in str(e.value)
    ctx.inject_failure(FAIL_COMM_INIT, 0)        # cancelling is allowed
    with pytest.raises(SushiCudaError):
        ctx.inject_failure(7, 1)
    assert ctx.copy_bytes() == copies_before     # none of this moved a byte over PCIe through the library


def test_bounded_wait_expiry_reaches_the_host_and_context_survives(ctx):
    """Failure detection without a fault: a kernel-side wait on a barrier nothing arrives on gives
    up after its limit and records a code; sync reports KERNEL_TIMEOUT once, clears it, and the
    same context keeps computing correctly."""
    import time
    from sushiblas_b200 import SushiCudaError
    ctx.sync()
    t0 = time.perf_counter()
    ctx.selftest_bounded_wait(50)
    with pytest.raises(SushiCudaError) as e:
        ctx.sync()
    dt = time.perf_counter() - t0
    assert e.value.code == -5 and "code 99" in str(e.value)
    assert 0.04 < dt < 1.0, dt                  # waited about the limit, not forever
    ctx.sync()                                   # status was cleared: no error any more
    check(ctx, TC3X, 0, 0, 512, 512, 256, 1.0, 0.0)
    check(ctx, SIMT, 0, 0, 64, 64, 64, 1.0, 0.0)
    with pytest.raises(SushiCudaError):
        ctx.selftest_bounded_wait(100000)        # limit out of range is rejected, nothing is launched


@pytest.mark.parametrize("tb", [0, 1])
def test_tall_and_skinny_products(ctx, tb):
    """n <= 32 with many rows goes to the streaming kernel (A read once, 8-way k split per row):
    every column count class, ragged k chunks, padded leading dimensions, alpha / beta, batches."""
    for (m, n, k) in [(4096, 16, 256), (2048, 1, 32), (5000, 5, 100), (3000, 8, 516), (2500, 17, 260), (2049, 32, 1028)]:
        for (alpha, beta) in [(1.0, 0.0), (1.5, 0.5)]:
            check(ctx, AUTO, 0, tb, m, n, k, alpha, beta, seed=800 + n + k)
    check(ctx, AUTO, 0, tb, 4100, 12, 132, -1.0, 1.0, batch=3, pad=(4, 3, 5), seed=850)
    check(ctx, AUTO, 0, tb, 2048, 16, 64, 1.0, 0.0, seed=851, poison_c=True)     # beta == 0: C is not read
    # unaligned leading dimension of A: the tiled kernel serves it, same answer class
    check(ctx, AUTO, 0, tb, 2100, 16, 64, 1.0, 0.5, pad=(1, 0, 0), seed=852)
    # row counts that fill one round of the 28-warp CTA shape (448 rows per CTA, one CTA per SM) take that shape:
    # every column count class, a ragged last row block, ragged and multi-chunk k, batches
    for (m, n, k, batch) in [(66000, 16, 256, 1), (66001, 5, 100, 1), (66300, 32, 516, 1), (65536, 24, 132, 1),
                             (33000, 17, 260, 2)]:
        check(ctx, AUTO, 0, tb, m, n, k, 1.5, 0.5, batch=batch, seed=860 + n)


@pytest.mark.parametrize("variant,m,n", [(AUTO, 4096, 16), (AUTO, 66000, 16), (TC3X, 768, 512), (TC3X, 4096, 2304)])
def test_non_finite_and_huge_inputs_stay_in_their_rows(ctx, variant, m, n):
    """Infinities, NaNs and values near the top of the range in A, on the 3xTF32 paths: both CTA shapes of the
    streaming kernel (which rounds with integer arithmetic on the bit patterns), the tensor kernel splitting
    inside the kernel (small problem) and behind the pre-pass (large one).  An infinity or a NaN makes its own row
    of C non-finite (3xTF32 multiplies the infinity by both parts of the other factor, so the row holds infinities
    of the right sign and NaNs; never a finite number), 2^120 and 3e38 give finite, accurate results, and every
    other row is untouched.  B is positive."""
    k = 256
    a = og.uniform_pm1(870, m * k).reshape(m, k).copy()
    b = (np.abs(og.uniform_pm1(871, k * n)) * 0.5 + 0.25).astype(np.float32).reshape(k, n)
    nan = np.array([0x7fffffff], dtype=np.uint32).view(np.float32)[0]
    special = {0: np.float32(np.inf), 1: np.float32(-np.inf), 2: nan, 3: np.float32(2.0 ** 120), 4: np.float32(3e38)}
    base = m - 40                                            # for m = 66000: inside the last, ragged row block
    for i, v in special.items():
        a[base + 5 * i, 3 + 17 * i] = v
    c = torch.full((m * n,), float("nan"), device="cuda")
    ctx.set_gemm_variant(variant)
    ctx.sgemm(0, 0, m, n, k, 1.0, dev(a.reshape(-1)), k, dev(b.reshape(-1)), n, 0.0, c, n)
    ctx.sync()
    ctx.set_gemm_variant(AUTO)
    got = c.cpu().numpy().reshape(m, n)
    assert np.all((got[base] == np.inf) | np.isnan(got[base]))
    assert np.all((got[base + 5] == -np.inf) | np.isnan(got[base + 5]))
    assert np.all(np.isnan(got[base + 10]))
    with np.errstate(over="ignore", invalid="ignore"):
        ref = a.astype(np.float64) @ b.astype(np.float64)
        absab = np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64)
    for row in (base + 15, base + 20):                       # huge but finite: as accurate as any other row
        assert np.all(np.isfinite(got[row])), row
        assert np.all(np.abs(got[row] - ref[row]) <= BUDGET * 8 * k * 2.0 ** -24 * absab[row]), row
    plain = np.ones(m, dtype=bool)
    plain[[base + 5 * i for i in special]] = False
    r, _ = og.tolerance_ratio(got[plain][None], ref[plain][None], absab[plain][None], k, budget=BUDGET)
    assert r <= 1.0, r


def test_split_inside_the_kernel_equals_pre_split_planes(ctx):
    """Operands of a problem this small are split into hi / lo inside the GEMM kernel (either storage order); the
    rate probe forces the pre-pass and whole tiles.  Same rounding, same per-tile arithmetic: bit-equal results
    in every transpose, and the one-product probe (hi * hi only) stays within TF32 accuracy of the oracle."""
    m, n, k = 1024, 1536, 232                 # 15 k-blocks: too few for the few-tiles K cut, so both paths deal whole tiles
    a = og.uniform_pm1(700, m * k)
    b = og.uniform_pm1(710, k * n)
    da, db = dev(a), dev(b)
    for ta, tb in [(0, 0), (0, 1), (1, 0), (1, 1)]:
        lda, ldb = (m if ta else k), (k if tb else n)
        c1, c2, c3 = (torch.empty(m * n, device="cuda") for _ in range(3))
        ctx.set_gemm_variant(TC3X)
        before = ctx.launch_count()
        ctx.sgemm(ta, tb, m, n, k, 1.0, da, lda, db, ldb, 0.0, c1, n)
        assert ctx.launch_count() - before == 1, (ta, tb)                 # no pre-pass
        before = ctx.launch_count()
        ctx.sgemm_tf32_probe(ta, tb, m, n, k, da, lda, db, ldb, c2, n, 3)
        assert ctx.launch_count() - before == 3, (ta, tb)                 # two pre-pass launches and the GEMM
        ctx.sgemm_tf32_probe(ta, tb, m, n, k, da, lda, db, ldb, c3, n, 1)
        ctx.sync()
        ctx.set_gemm_variant(AUTO)
        assert torch.equal(c1, c2), (ta, tb)
        av = a.reshape(k, m).T if ta else a.reshape(m, k)
        bv = b.reshape(n, k).T if tb else b.reshape(k, n)
        ref = av.astype(np.float64) @ bv.astype(np.float64)
        absab = np.abs(av).astype(np.float64) @ np.abs(bv).astype(np.float64)
        r, _ = og.tolerance_ratio(c1.cpu().numpy().reshape(1, m, n), ref[None], absab[None], k, budget=BUDGET)
        assert r <= 1.0, (ta, tb, r)
        # hi * hi alone: each factor carries a relative error of at most 2^-11
        err1 = np.abs(c3.cpu().numpy().reshape(m, n).astype(np.float64) - ref)
        assert np.all(err1 <= 2.0 ** -9.9 * absab + 1e-30), (ta, tb, float((err1 / absab).max()))
        assert float((err1 / absab).max()) > 2.0 ** -16, "the one-product probe should not be fp32-accurate"


def test_launch_counter_counts_kernels(ctx):
    before = ctx.launch_count()
    check(ctx, SIMT, 0, 0, 64, 64, 64, 1.0, 0.0)
    mid = ctx.launch_count()
    assert mid - before == 1
    # tensor-core path: one pre-pass launch per operand that is not split inside the GEMM kernel.  Aligned
    # operands of small problems are split in the kernel in either storage order: one launch in every transpose
    for (ta, tb) in [(1, 0), (0, 0), (0, 1), (1, 1)]:
        start = ctx.launch_count()
        check(ctx, TC3X, ta, tb, 256, 256, 64, 1.0, 0.0)
        assert ctx.launch_count() - start == 1, (ta, tb)
    # an operand whose leading dimension is not a multiple of 4 floats goes through the pre-pass: A here
    start = ctx.launch_count()
    check(ctx, TC3X, 1, 0, 256, 256, 64, 1.0, 0.0, pad=(1, 0, 0))
    assert ctx.launch_count() - start == 2
