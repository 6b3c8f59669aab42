"""CPU tests of the oracle: the reference's known answers, the integer golden vectors,
the front-end restatement and a cross-check against MKL sgemm (the library family the
reference forwards to).  No GPU."""
import os

import numpy as np
import pytest

from oracle import ref_gemm as og

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "gemm_integer_kat.npz")


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


def test_reference_kat_simple_3x3(golden):
    # tests/blas/level3/test_gemm.cpp:39-63 -- row-major engine, defaults NN, alpha=1, beta=0
    out, _ = og.engine_gemm(golden["ref_simple3x3.a"], (3, 3), golden["ref_simple3x3.b"], (3, 3),
                            golden["ref_simple3x3.c_in"], (3, 3))
    np.testing.assert_allclose(out, golden["ref_simple3x3.c_out"], atol=1e-4, rtol=0)
    assert np.array_equal(out.astype(np.float32), golden["ref_simple3x3.c_out"])


def test_reference_kat_column_major(golden):
    # tests/blas/level3/test_gemm.cpp:65-88 -- column-major engine, 2x2x2, memory {19,43,22,50}
    out, _ = og.engine_gemm(golden["ref_colmajor2x2.a"], (2, 2), golden["ref_colmajor2x2.b"], (2, 2),
                            np.zeros(4, np.float32), (2, 2), layout=og.COLUMN_MAJOR)
    assert np.array_equal(out.astype(np.float32), golden["ref_colmajor2x2.c_out"])


def test_reference_kat_syrk(golden):
    # tests/blas/level3/test_syrk.cpp:39-63 -- row-major, lower, no transpose, alpha=1, beta=0
    out, _ = og.syrk_f64_c(False, False, 3, 2, 1.0, golden["ref_syrk_lower3.a"], 2, 0, 0.0, np.zeros(9, np.float32), 3, 0, 1)
    assert np.array_equal(out.astype(np.float32), golden["ref_syrk_lower3.c_out"])
    # tests/blas/level3/test_syrk.cpp:65-88 -- column-major engine, A created as {K, N} = {3, 2}, transA = true
    # (column-major: lda = A.shape[rank-2] = 3, syrk.cpp:110)
    out, _ = og.syrk_f64_c(False, True, 2, 3, 1.0, golden["ref_syrk_colmajor_trans.a"], 3, 0, 0.0, np.zeros(4, np.float32),
                           2, 0, 1, layout=og.COLUMN_MAJOR)
    assert np.array_equal(out.astype(np.float32), golden["ref_syrk_colmajor_trans.c_out"])
    # column-major (uplo, trans) is row-major (other uplo, other trans) on the same memory
    rng = np.random.default_rng(4)
    n, k = 5, 7
    for upper in (0, 1):
        for trans in (0, 1):
            a = rng.standard_normal(n * k).astype(np.float32)
            c = rng.standard_normal(n * n).astype(np.float32)
            lda_col = k if trans else n
            col, _ = og.syrk_f64_c(upper, trans, n, k, 1.5, a, lda_col, 0, 0.5, c, n, 0, 1, layout=og.COLUMN_MAJOR)
            row, _ = og.syrk_f64_c(not upper, not trans, n, k, 1.5, a, lda_col, 0, 0.5, c, n, 0, 1, layout=og.ROW_MAJOR)
            np.testing.assert_array_equal(col, row)
    # numpy twin agrees with the C restatement
    a = rng.uniform(-1, 1, (2, 9, 6)).astype(np.float32); c = rng.uniform(-1, 1, (2, 9, 9)).astype(np.float32)
    r1, ab1 = og.syrk_f64_c(True, False, 9, 6, 2.0, a, 6, 54, -1.0, c, 9, 81, 2)
    r2, ab2, _ = og.syrk_f64_np(True, False, 9, 6, 2.0, a, 6, 54, -1.0, c, 9, 81, 2)
    np.testing.assert_allclose(r1.reshape(2, 9, 9), r2, rtol=1e-13, atol=1e-13)
    np.testing.assert_allclose(ab1.reshape(2, 9, 9), ab2, rtol=1e-13, atol=1e-13)


def test_column_major_equals_swapped_row_major():
    # the identity the C++ front-end uses to serve gemm.cpp:66-78 with a row-major kernel
    rng = np.random.default_rng(3)
    m, n, k = 5, 4, 6
    for ta in (0, 1):
        for tb in (0, 1):
            a = rng.standard_normal((m * k)).astype(np.float32)
            b = rng.standard_normal((k * n)).astype(np.float32)
            lda = k if ta else m          # column-major: leading dim = rows of the stored matrix
            ldb = n if tb else k
            col, _ = og.gemm_f64_c(ta, tb, m, n, k, 1.5, a, lda, 0, b, ldb, 0, 0.0, None, m, 0, 1,
                                   layout=og.COLUMN_MAJOR)
            row, _ = og.gemm_f64_c(tb, ta, n, m, k, 1.5, b, ldb, 0, a, lda, 0, 0.0, None, m, 0, 1,
                                   layout=og.ROW_MAJOR)
            np.testing.assert_array_equal(col, row)


def _golden_case(g, name):
    ta, tb, m, n, k, alpha, beta, batch, lda, ldb, ldc, sa, sb, sc = [int(v) for v in g[f"{name}.meta"]]
    return dict(ta=ta, tb=tb, m=m, n=n, k=k, alpha=float(alpha), beta=float(beta), batch=batch, lda=lda,
                ldb=ldb, ldc=ldc, sa=sa, sb=sb, sc=sc, a=g[f"{name}.a"], b=g[f"{name}.b"],
                c_in=g[f"{name}.c_in"], c_out=g[f"{name}.c_out"])


def test_integer_golden_vectors(golden):
    for name in golden["names"]:
        c = _golden_case(golden, str(name))
        out, absab = og.gemm_f64_c(c["ta"], c["tb"], c["m"], c["n"], c["k"], c["alpha"], c["a"], c["lda"], c["sa"],
                                   c["b"], c["ldb"], c["sb"], c["beta"], c["c_in"], c["ldc"], c["sc"], c["batch"])
        exp = c["c_out"].astype(np.float64)
        view = lambda x: og._view(x, c["m"], c["n"], c["ldc"], c["sc"], c["batch"])
        assert np.array_equal(view(out), view(exp)), name
        # the fp32 scalar port must agree exactly too (all partial sums are small integers)
        out32 = og.gemm_f32_c(c["ta"], c["tb"], c["m"], c["n"], c["k"], c["alpha"], c["a"], c["lda"], c["sa"],
                              c["b"], c["ldb"], c["sb"], c["beta"], c["c_in"], c["ldc"], c["sc"], c["batch"])
        assert np.array_equal(view(out32), view(c["c_out"])), name
        # and the padding between rows of C is never written
        assert np.array_equal(out32, c["c_out"]), name


def test_c_and_numpy_twins_agree():
    rng = np.random.default_rng(11)
    for (ta, tb, m, n, k, batch, alpha, beta) in [(0, 0, 33, 17, 29, 1, 1.0, 0.0), (1, 0, 20, 31, 45, 2, 1.5, 0.5),
                                                   (0, 1, 64, 64, 64, 3, -2.0, 1.0), (1, 1, 7, 9, 130, 1, 0.25, -0.75)]:
        ar, ac = (k, m) if ta else (m, k)
        br, bc = (n, k) if tb else (k, n)
        a = rng.uniform(-1, 1, (batch, ar, ac)).astype(np.float32)
        b = rng.uniform(-1, 1, (batch, br, bc)).astype(np.float32)
        c = rng.uniform(-1, 1, (batch, m, n)).astype(np.float32)
        r1, ab1 = og.gemm_f64_c(ta, tb, m, n, k, alpha, a, ac, ar * ac, b, bc, br * bc, beta, c, n, m * n, batch)
        r2, ab2 = og.gemm_f64_np(ta, tb, m, n, k, alpha, a, ac, ar * ac, b, bc, br * bc, beta, c, n, m * n, batch)
        np.testing.assert_allclose(r1.reshape(batch, m, n), r2, rtol=1e-13, atol=1e-13)
        np.testing.assert_allclose(ab1.reshape(batch, m, n), ab2, rtol=1e-13, atol=1e-13)


def test_beta_zero_does_not_read_c():
    a = np.ones(4, np.float32); b = np.ones(4, np.float32)
    c = np.full(4, np.nan, np.float32)
    out, _ = og.gemm_f64_c(0, 0, 2, 2, 2, 1.0, a, 2, 0, b, 2, 0, 0.0, c, 2, 0, 1)
    assert np.array_equal(out, np.full(4, 2.0))


def test_tensor_strides_and_params():
    # tensor.hpp:99-116
    assert og.tensor_strides((4, 5, 6), og.ROW_MAJOR) == (30, 6, 1)
    assert og.tensor_strides((4, 5, 6), og.COLUMN_MAJOR) == (1, 4, 20)
    # gemm.cpp:91-105 on the batched benchmark shape {256,512,512}
    s = og.tensor_strides((256, 512, 512))
    p = og.derive_gemm_params((256, 512, 512), s, (256, 512, 512), s, (256, 512, 512), s, False, False)
    assert p == dict(m=512, n=512, k=512, batch=256, lda=512, ldb=512, ldc=512,
                     stride_a=262144, stride_b=262144, stride_c=262144)
    # k comes from A's second-to-last dim when transA (gemm.cpp:93)
    p = og.derive_gemm_params((7, 3), (3, 1), (7, 5), (5, 1), (3, 5), (5, 1), True, False)
    assert (p["m"], p["n"], p["k"], p["lda"], p["batch"], p["stride_a"]) == (3, 5, 7, 3, 1, 0)
    with pytest.raises(RuntimeError, match="at least 2D"):
        og.derive_gemm_params((3,), (1,), (3, 3), (3, 1), (3, 3), (3, 1), False, False)


def test_tolerance_ratio_semantics():
    ref = np.array([[1.0, 2.0]]); absab = np.array([[1.0, 2.0]])
    k = 4
    tol0 = 8 * k * 2.0 ** -24 * 1.0
    r, q = og.tolerance_ratio(ref + np.array([[tol0, 0.0]]), ref, absab, k)
    assert abs(r - 1.0) < 1e-9 and abs(q - 8 * k) < 1e-6
    r, _ = og.tolerance_ratio(ref + np.array([[tol0, 0.0]]), ref, absab, k, budget=0.5)
    assert abs(r - 2.0) < 1e-9
    # the beta term is not scaled by the budget
    cin = np.array([[4.0, 0.0]])
    r, _ = og.tolerance_ratio(ref + np.array([[2.0 ** -24 * 2.0, 0.0]]), ref, np.zeros((1, 2)), k, beta=0.5,
                              c_in=cin, budget=0.5)
    assert abs(r - 1.0) < 1e-9
    r, _ = og.tolerance_ratio(np.array([[np.nan, 2.0]]), ref, absab, k)
    assert r == float("inf")


def test_mkl_sgemm_is_within_tolerance_of_oracle():
    """MKL sgemm (the reference's arithmetic family) lies within the stated bound of the
    fp64 oracle -- i.e. checking a kernel against the oracle at half budget covers any
    conforming reference result by the triangle inequality."""
    torch = pytest.importorskip("torch")
    m = n = k = 256
    a = og.uniform_pm1(1, m * k).reshape(m, k)
    b = og.uniform_pm1(2, k * n).reshape(k, n)
    c0 = og.uniform_pm1(3, m * n).reshape(m, n)
    for ta, tb in [(0, 0), (0, 1), (1, 0), (1, 1)]:
        ref, absab = og.gemm_f64_np(ta, tb, m, n, k, 1.5, a, k, 0, b, n, 0, 0.5, c0, n, 0, 1)
        c = torch.from_numpy(c0.copy())
        og.mkl_proxy_gemm(ta, tb, 1.5, torch.from_numpy(a), torch.from_numpy(b), 0.5, c)
        r, q = og.tolerance_ratio(c.numpy()[None], ref, absab, k, beta=0.5, c_in=c0[None], budget=0.5)
        assert r < 1.0, (ta, tb, r, q)


def test_generator_is_counter_based_and_in_range():
    x = og.uniform_pm1(42, 1000)
    y = og.uniform_pm1(42, 100, start=500)
    assert np.array_equal(x[500:600], y)
    assert x.dtype == np.float32 and x.min() >= -1.0 and x.max() < 1.0
    assert abs(float(x.mean())) < 0.1
    assert not np.array_equal(x, og.uniform_pm1(43, 1000))
    z = og.normal(7, 20000, std=0.02)
    assert abs(float(z.std()) - 0.02) < 0.002 and abs(float(z.mean())) < 0.001


# ------------------------------------------------------------------ TRSM restatement
def test_trsm_oracle_reproduces_the_reference_known_answers():
    # tests/blas/level3/test_trsm.cpp:39-77: row-major, lower, left side
    x = og.trsm_f64_c(1, 0, 0, 0, 2, 2, 1.0, [2, 0, 1, 2], 2, 0, [4, 6, 4, 7], 2, 0, 1)
    assert np.array_equal(x, [2, 3, 1, 2])
    # tests/blas/level3/test_trsm.cpp:79-: column-major engine, upper, left side
    x = og.trsm_f64_c(1, 1, 0, 0, 2, 2, 1.0, [2, 0, 1, 2], 2, 0, [4, 4, 6, 7], 2, 0, 1, layout=og.COLUMN_MAJOR)
    assert np.array_equal(x, [1.0, 2.0, 1.25, 3.5])


def test_trsm_c_restatement_matches_lapack_in_every_mode():
    rng = np.random.default_rng(5)
    for left in (0, 1):
        for upper in (0, 1):
            for trans in (0, 1):
                for unit in (0, 1):
                    m, n, batch = 9, 6, 2
                    dim = m if left else n
                    lda, ldb = dim + 2, n + 1
                    a = (rng.standard_normal((batch, dim, lda)) * 0.2).astype(np.float32)
                    a[:, np.arange(dim), np.arange(dim)] += 3.0
                    b = rng.standard_normal((batch, m, ldb)).astype(np.float32)
                    xc = og.trsm_f64_c(left, upper, trans, unit, m, n, 0.5, a, lda, dim * lda, b, ldb, m * ldb, batch)
                    xn, t = og.trsm_f64_np(left, upper, trans, unit, m, n, 0.5, a, lda, dim * lda, b, ldb, m * ldb, batch)
                    got = og._view(xc, m, n, ldb, m * ldb, batch)
                    assert np.allclose(got, xn, rtol=1e-12, atol=1e-12), (left, upper, trans, unit)
                    bv = og._view(b.ravel(), m, n, ldb, m * ldb, batch)
                    for i in range(batch):
                        assert og.trsm_residual_ratio(left, t[i], got[i], 0.5, bv[i], dim) < 1e-6
                    # a column-major solve is the row-major solve of the transposed equation
                    xcm = og.trsm_f64_c(not left, not upper, trans, unit, n, m, 0.5, a, lda, dim * lda, b, ldb, m * ldb,
                                        batch, layout=og.COLUMN_MAJOR)
                    assert np.allclose(xcm, xc, rtol=1e-12, atol=1e-12), (left, upper, trans, unit)


# ------------------------------------------------------------------ FLOAT64 GEMM restatement
def test_dgemm_oracle_known_answers_and_numpy_agreement():
    # the reference's fp32 GEMM known answers are exactly representable: evaluated in double they pin the fp64 oracle
    a = np.arange(1, 10, dtype=np.float64)
    out, _ = og.dgemm_f80_c(0, 0, 3, 3, 3, 1.0, a, 3, 0, np.eye(3).ravel(), 3, 0, 0.0, np.zeros(9), 3, 0, 1)
    assert out.dtype == np.longdouble and np.array_equal(out.astype(np.float64), a)
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "gemm_integer_kat.npz"))
    for name in g["names"]:
        ta, tb, m, n, k, alpha, beta, batch, lda, ldb, ldc, sa, sb, sc = [int(v) for v in g[f"{name}.meta"]]
        out, _ = og.dgemm_f80_c(ta, tb, m, n, k, float(alpha), g[f"{name}.a"], lda, sa, g[f"{name}.b"], ldb, sb, float(beta),
                                g[f"{name}.c_in"], ldc, sc, batch)
        idx = (np.arange(batch)[:, None, None] * sc + np.arange(m)[None, :, None] * ldc + np.arange(n)[None, None, :]).ravel()
        assert np.array_equal(out[idx].astype(np.float64), g[f"{name}.c_out"][idx].astype(np.float64)), name
    # a conforming dgemm (numpy -> BLAS) sits well inside the bound; column-major equals the swapped row-major call
    rng = np.random.default_rng(11)
    m, n, k = 33, 21, 57
    A, B, C = rng.standard_normal((m, k)), rng.standard_normal((k, n)), rng.standard_normal((m, n))
    for ta, tb in [(0, 0), (0, 1), (1, 0), (1, 1)]:
        a_st = np.ascontiguousarray(A.T) if ta else A
        b_st = np.ascontiguousarray(B.T) if tb else B
        ref, absab = og.dgemm_f80_c(ta, tb, m, n, k, 1.5, a_st, a_st.shape[1], 0, b_st, b_st.shape[1], 0, 0.5, C, n, 0, 1)
        assert og.tolerance_ratio_f64((1.5 * A @ B + 0.5 * C).ravel(), ref, absab, k, 0.5, C.ravel(), budget=0.5) < 1.0
    ref_cm, _ = og.dgemm_f80_c(0, 0, m, n, k, 1.0, np.asfortranarray(A).ravel(order="K"), m, 0,
                               np.asfortranarray(B).ravel(order="K"), k, 0, 0.0, np.zeros(m * n), m, 0, 1,
                               layout=og.COLUMN_MAJOR)
    ref_rm, _ = og.dgemm_f80_c(0, 0, m, n, k, 1.0, A, k, 0, B, n, 0, 0.0, np.zeros(m * n), n, 0, 1)
    assert np.array_equal(ref_cm.reshape(n, m).T, ref_rm.reshape(m, n))
    assert og.tolerance_ratio_f64(np.array([np.nan]), np.array([0.0], np.longdouble), np.array([1.0]), 1) == float("inf")


# ------------------------------------------------------------------ activation restatements
def test_activation_oracle_reproduces_the_reference_known_answers():
    from oracle import ref_activations as oa
    for kind, a, x, want in oa.REFERENCE_FORWARD:
        assert np.allclose(oa.forward(kind, x, a), want, rtol=0, atol=1e-4), oa.NAMES[kind]   # tests/test_common.hpp:48
    for kind, a, dy, s, want in oa.REFERENCE_BACKWARD:
        assert np.allclose(oa.backward(kind, dy, s, a), want, rtol=0, atol=1e-4), oa.NAMES[kind]
    # the backward forms are the derivatives of the forward forms (central differences)
    x = np.linspace(-3.0, 3.0, 25) + 0.013
    for kind, a in [(oa.LEAKY_RELU, 0.1), (oa.ELU, 0.7), (oa.SILU, 0.0), (oa.GELU, 0.0), (oa.SOFTPLUS, 0.0)]:
        num = (oa.forward(kind, x + 1e-6, a) - oa.forward(kind, x - 1e-6, a)) / 2e-6
        assert np.allclose(oa.backward(kind, np.ones_like(x), x, a), num, rtol=1e-6, atol=1e-7), oa.NAMES[kind]
    for kind in (oa.SIGMOID, oa.TANH):
        y = oa.forward(kind, x)
        num = (oa.forward(kind, x + 1e-6) - oa.forward(kind, x - 1e-6)) / 2e-6
        assert np.allclose(oa.backward(kind, np.ones_like(x), y), num, rtol=1e-6, atol=1e-7), oa.NAMES[kind]


def test_mkl_trsm_and_syrk_lie_within_the_bounds_of_the_oracle():
    """The reference forwards TRSM / SYRK to oneMKL; MKL's own fp32 routines (through torch CPU) must sit inside
    the tolerances the GPU tests use against the fp64 restatements -- so those tolerances admit the reference."""
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(21)
    m, n = 96, 40
    for left in (1, 0):
        for upper in (0, 1):
            for trans in (0, 1):
                dim = m if left else n
                a = (rng.uniform(-1, 1, (dim, dim)) * (2.0 / dim)).astype(np.float32)
                a[np.arange(dim), np.arange(dim)] = rng.uniform(3, 5, dim).astype(np.float32)
                b = rng.uniform(-1, 1, (m, n)).astype(np.float32)
                tri = np.triu(a) if upper else np.tril(a)
                op = tri.T if trans else tri
                x = torch.linalg.solve_triangular(torch.from_numpy(np.ascontiguousarray(op)), torch.from_numpy(0.5 * b),
                                                  upper=bool(upper) != bool(trans), left=bool(left)).numpy()
                xref, t = og.trsm_f64_np(left, upper, trans, 0, m, n, 0.5, a, dim, 0, b, n, 0, 1)
                assert og.trsm_residual_ratio(left, t[0], x, 0.5, b, dim) <= 1.0, (left, upper, trans)
                assert np.max(np.abs(x - xref[0])) <= 32.0 * dim * 2.0 ** -24 * np.max(np.abs(xref[0]))
    nn, k = 64, 150
    a = rng.uniform(-1, 1, (nn, k)).astype(np.float32)
    c0 = rng.uniform(-1, 1, (nn, nn)).astype(np.float32)
    got = (1.5 * torch.from_numpy(a) @ torch.from_numpy(a).T + 0.5 * torch.from_numpy(c0)).numpy()
    ref, absaa, mask = og.syrk_f64_np(0, 0, nn, k, 1.5, a, k, 0, 0.5, c0, nn, 0, 1)
    r, _ = og.tolerance_ratio(np.where(mask, got, 0.0)[None], np.where(mask[None], ref, 0.0), absaa, k, beta=0.5,
                              c_in=np.where(mask, c0, 0.0)[None], budget=0.5)
    assert r <= 1.0
