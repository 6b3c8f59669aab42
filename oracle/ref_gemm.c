/*
 * ref_gemm.c -- CPU oracle for the fp32 GEMM path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is a checker: only the test-suite, the smoke check and the CPU-baseline
 * leg of the benchmark may build or call it.  Nothing the library ships routes
 * through it.
 *
 * What it restates
 * ----------------
 * The reference front-end (src/ops/blas/level3/gemm.cpp:82-198) derives BLAS
 * parameters from Tensor metadata and forwards to an external, closed BLAS
 * (oneapi::mkl::blas::row_major::gemm / gemm_batch, call sites gemm.cpp:58,63;
 * the column-major twins at gemm.cpp:71,76).  Intel oneMKL is not vendored in the
 * reference tree and no version is pinned there, so the arithmetic below follows
 * the published BLAS definition that the reference documents in
 * include/SushiBLAS/ops/blas/level3.hpp:57-70:
 *
 *      C <- alpha * op(A) * op(B) + beta * C ,   op(X) = X or X^T
 *
 * with the strided-batch rule of gemm_batch (batch i uses a + i*stride_a, ...)
 * and the BLAS convention that C is not read when beta == 0 (callers in
 * tests/runtime/test_framework_sim.cpp:39-40,51 rely on that).
 *
 * Accumulation is done in double so the result is an (almost) exact reference;
 * (|A||B|)_ij is accumulated alongside for the error bound
 *      |dC_ij| <= 8*K*2^-24*(|A||B|)_ij + 2^-24*|beta*C_ij| .
 *
 * Pinning: the two value-pinning tests the reference holds for this path
 * (tests/blas/level3/test_gemm.cpp:39-63 and 65-88) are reproduced by
 * tests/test_oracle.py.  Transposes, alpha/beta and batching are not covered by any
 * reference test: for those the oracle is pinned only by integer-valued
 * known-answer cases whose result is exact under every summation order.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>

/* Element (r, c) of op(X) where X is stored with leading dimension ld.
 * layout_row != 0: row-major storage, else column-major storage.            */
static inline int64_t op_index(int layout_row, int trans, int64_t r, int64_t c, int64_t ld)
{
    /* stored matrix element (i, j): row-major i*ld + j, column-major j*ld + i */
    int64_t i = trans ? c : r;
    int64_t j = trans ? r : c;
    return layout_row ? i * ld + j : j * ld + i;
}

/*
 * oracle_gemm_f64acc: strided-batched GEMM, fp32 operands, fp64 accumulation.
 *
 *  layout_row : 1 = row-major (gemm.cpp:52-65), 0 = column-major (gemm.cpp:66-78)
 *  c_in       : C before the call (read only when beta != 0); may alias nothing
 *  c_out64    : result in double, same indexing as C (ldc / stride_c), must not be NULL
 *  abs_ab     : optional, same indexing: sum_k |op(A)_ik| * |op(B)_kj|
 * Returns 0, or -1 on invalid arguments.
 */
int oracle_gemm_f64acc(int layout_row, int trans_a, int trans_b,
                       int64_t m, int64_t n, int64_t k,
                       float alpha,
                       const float* a, int64_t lda, int64_t stride_a,
                       const float* b, int64_t ldb, int64_t stride_b,
                       float beta,
                       const float* c_in, int64_t ldc, int64_t stride_c,
                       int64_t batch,
                       double* c_out64, double* abs_ab)
{
    if (m < 0 || n < 0 || k < 0 || batch < 0 || !c_out64) return -1;
    if (m == 0 || n == 0 || batch == 0) return 0;
    if (beta != 0.0f && !c_in) return -1;

    /* Pack op(B) as a dense k x n double panel per batch so the inner loop is
     * unit stride; rows of op(A) are gathered one at a time.                  */
    for (int64_t bi = 0; bi < batch; ++bi)
    {
        const float* ab = a + bi * stride_a;
        const float* bb = b + bi * stride_b;
        double* pb = (double*)malloc(sizeof(double) * (size_t)(k > 0 ? k : 1) * (size_t)n);
        if (!pb) return -1;
        for (int64_t kk = 0; kk < k; ++kk)
            for (int64_t j = 0; j < n; ++j)
                pb[kk * n + j] = (double)bb[op_index(layout_row, trans_b, kk, j, ldb)];

        {
            double* acc = (double*)malloc(sizeof(double) * (size_t)n * 2);
            double* accabs = acc + n;
            for (int64_t i = 0; i < m; ++i)
            {
                for (int64_t j = 0; j < n; ++j) { acc[j] = 0.0; accabs[j] = 0.0; }
                for (int64_t kk = 0; kk < k; ++kk)
                {
                    double av = (double)ab[op_index(layout_row, trans_a, i, kk, lda)];
                    double aabs = fabs(av);
                    const double* brow = pb + kk * n;
                    for (int64_t j = 0; j < n; ++j)
                    {
                        acc[j] += av * brow[j];
                        accabs[j] += aabs * fabs(brow[j]);
                    }
                }
                for (int64_t j = 0; j < n; ++j)
                {
                    int64_t ci = bi * stride_c + (layout_row ? i * ldc + j : j * ldc + i);
                    double v = (double)alpha * acc[j];
                    if (beta != 0.0f) v += (double)beta * (double)c_in[ci];
                    c_out64[ci] = v;
                    if (abs_ab) abs_ab[ci] = accabs[j];
                }
            }
            free(acc);
        }
        free(pb);
    }
    return 0;
}

/*
 * oracle_gemm_f32: same definition with plain fp32 accumulation in k order, as a
 * model of what a conforming single-precision BLAS returns.  Used only as the
 * scalar "port" leg when a CPU timing of the restatement itself is wanted.
 */
int oracle_gemm_f32(int layout_row, int trans_a, int trans_b,
                    int64_t m, int64_t n, int64_t k,
                    float alpha,
                    const float* a, int64_t lda, int64_t stride_a,
                    const float* b, int64_t ldb, int64_t stride_b,
                    float beta,
                    float* c, int64_t ldc, int64_t stride_c,
                    int64_t batch)
{
    if (m < 0 || n < 0 || k < 0 || batch < 0 || !c) return -1;
    for (int64_t bi = 0; bi < batch; ++bi)
    {
        const float* ab = a + bi * stride_a;
        const float* bb = b + bi * stride_b;
        float* cb = c + bi * stride_c;
        for (int64_t i = 0; i < m; ++i)
        {
            for (int64_t j = 0; j < n; ++j)
            {
                float s = 0.0f;
                for (int64_t kk = 0; kk < k; ++kk)
                    s += ab[op_index(layout_row, trans_a, i, kk, lda)] *
                         bb[op_index(layout_row, trans_b, kk, j, ldb)];
                int64_t ci = layout_row ? i * ldc + j : j * ldc + i;
                cb[ci] = (beta == 0.0f) ? alpha * s : alpha * s + beta * cb[ci];
            }
        }
    }
    return 0;
}

/*
 * oracle_check_tolerance: max over the m x n x batch result of
 *      |c_test - c_ref| / (budget * 8*K*2^-24*absab + 2^-24*|beta*c_in|)
 * A value <= 1 means every element is inside the stated bound with its K term scaled by
 * `budget` (the beta term is one fp32 rounding of the output and is not scaled).
 * Elements whose bound is zero must match exactly (ratio reported as +inf if not).
 * Also returns (through *max_ulps_noK) max |dC| / (2^-24 * absab), the error in
 * units that do not grow with K.  Row-major indexing only (ldc, stride_c).
 */
double oracle_check_tolerance(int64_t m, int64_t n, int64_t k, int64_t batch,
                              float beta, double budget,
                              const float* c_test, const double* c_ref,
                              const double* abs_ab, const float* c_in,
                              int64_t ldc, int64_t stride_c,
                              double* max_ulps_noK)
{
    const double u = ldexp(1.0, -24);
    double worst = 0.0, worst_nok = 0.0;
    for (int64_t bi = 0; bi < batch; ++bi)
        for (int64_t i = 0; i < m; ++i)
            for (int64_t j = 0; j < n; ++j)
            {
                int64_t ci = bi * stride_c + i * ldc + j;
                double err = fabs((double)c_test[ci] - c_ref[ci]);
                if (isnan(err)) return INFINITY;
                double bound = budget * 8.0 * (double)k * u * abs_ab[ci];
                if (beta != 0.0f && c_in) bound += u * fabs((double)beta * (double)c_in[ci]);
                double r = (bound > 0.0) ? err / bound : (err == 0.0 ? 0.0 : INFINITY);
                if (r > worst) worst = r;
                if (abs_ab[ci] > 0.0)
                {
                    double q = err / (u * abs_ab[ci]);
                    if (q > worst_nok) worst_nok = q;
                }
            }
    if (max_ulps_noK) *max_ulps_noK = worst_nok;
    return worst;
}

/*
 * oracle_syrk_f64acc: symmetric rank-k update, fp32 operands, fp64 accumulation.
 *
 *      C <- alpha * op(A) * op(A)^T + beta * C   on one triangle of the n x n matrix C
 *
 * Restates what the reference forwards to oneapi::mkl::blas::{row,column}_major::syrk[_batch]
 * (call sites src/ops/blas/level3/syrk.cpp:60-78) after deriving n, k, lda, ldc and the batch
 * strides from the tensors (syrk.cpp:84-116): n from C, k from A (A is n x k, or k x n when
 * trans), only the `upper` or lower triangle is referenced and updated, the other one is left
 * as it is.  c_out64 must arrive holding C's current values (as double) everywhere; elements of
 * the updated triangle are overwritten.  abs_aa (optional) receives sum_k |a_ik||a_jk| there.
 * Pinned by the reference's own known answers tests/blas/level3/test_syrk.cpp:39-103.
 */
int oracle_syrk_f64acc(int layout_row, int upper, int trans, int64_t n, int64_t k, float alpha,
                       const float* a, int64_t lda, int64_t stride_a, float beta,
                       const float* c_in, int64_t ldc, int64_t stride_c, int64_t batch,
                       double* c_out64, double* abs_aa)
{
    if (n < 0 || k < 0 || batch < 0 || !c_out64) return -1;
    for (int64_t bi = 0; bi < batch; ++bi)
    {
        const float* ab = a + bi * stride_a;
        for (int64_t i = 0; i < n; ++i)
            for (int64_t j = 0; j < n; ++j)
            {
                if (upper ? (j < i) : (j > i)) continue;
                double s = 0.0, sabs = 0.0;
                for (int64_t kk = 0; kk < k; ++kk)
                {
                    /* op(A)(i, kk): A stored n x k (trans == 0) or k x n (trans != 0) */
                    double x = (double)ab[op_index(layout_row, trans, i, kk, lda)];
                    double y = (double)ab[op_index(layout_row, trans, j, kk, lda)];
                    s += x * y;
                    sabs += fabs(x) * fabs(y);
                }
                int64_t ci = bi * stride_c + (layout_row ? i * ldc + j : j * ldc + i);
                double v = (double)alpha * s;
                if (beta != 0.0f) v += (double)beta * (double)c_in[ci];
                c_out64[ci] = v;
                if (abs_aa) abs_aa[ci] = sabs;
            }
    }
    return 0;
}

/*
 * oracle_trsm_f64: triangular solve with multiple right-hand sides, fp32 inputs, fp64 substitution.
 *
 *      left != 0:  op(A) * X = alpha * B  (A is m x m)       left == 0:  X * op(A) = alpha * B  (A is n x n)
 *
 * Restates what the reference forwards to oneapi::mkl::blas::{row,column}_major::trsm[_batch]
 * (call sites src/ops/blas/level3/trsm.cpp:61-79) after deriving m, n from B, lda / ldb from the
 * shapes and the batch strides from the tensors (trsm.cpp:85-135).  Only the `upper` or lower
 * triangle of A is read; with unit_diag its diagonal is taken as 1.  x_out64 is indexed like B.
 * Pinned by the reference's own known answers tests/blas/level3/test_trsm.cpp (row-major lower
 * left-side case and column-major upper left-side case).
 */
int oracle_trsm_f64(int layout_row, int left, int upper, int trans, int unit_diag, int64_t m, int64_t n,
                    float alpha, const float* a, int64_t lda, int64_t stride_a,
                    const float* b, int64_t ldb, int64_t stride_b, int64_t batch, double* x_out64)
{
    if (m < 0 || n < 0 || batch < 0 || !x_out64) return -1;
    const int64_t dim = left ? m : n;           /* order of A */
    const int64_t nrhs = left ? n : m;          /* independent systems */
    /* op(A) is lower triangular when exactly one of (upper, trans) is clear and the other ... */
    const int eff_lower = ((upper != 0) == (trans != 0));
    double* t = (double*)malloc(sizeof(double) * (size_t)(dim > 0 ? dim : 1) * (size_t)(dim > 0 ? dim : 1));
    double* x = (double*)malloc(sizeof(double) * (size_t)(dim > 0 ? dim : 1));
    if (!t || !x) { free(t); free(x); return -2; }
    for (int64_t bi = 0; bi < batch; ++bi)
    {
        const float* ab = a + bi * stride_a;
        /* dense T = op(A) restricted to the referenced triangle */
        for (int64_t r = 0; r < dim; ++r)
            for (int64_t c = 0; c < dim; ++c)
            {
                int in_tri = eff_lower ? (c <= r) : (c >= r);
                double v = 0.0;
                if (r == c && unit_diag) v = 1.0;
                else if (in_tri) v = (double)ab[op_index(layout_row, trans, r, c, lda)];
                t[r * dim + c] = v;
            }
        for (int64_t s = 0; s < nrhs; ++s)
        {
            /* left:  T x = alpha b_col(s);   right:  x^T T = alpha b_row(s)  <=>  T^T x = alpha b_row(s)^T */
            #define B_IDX(p) (bi * stride_b + (left ? (layout_row ? (p) * ldb + s : s * ldb + (p)) \
                                                    : (layout_row ? s * ldb + (p) : (p) * ldb + s)))
            #define T_AT(r, c) (left ? t[(r) * dim + (c)] : t[(c) * dim + (r)])
            const int lower_system = left ? eff_lower : !eff_lower;
            if (lower_system)
                for (int64_t i = 0; i < dim; ++i)
                {
                    double acc = (double)alpha * (double)b[B_IDX(i)];
                    for (int64_t k = 0; k < i; ++k) acc -= T_AT(i, k) * x[k];
                    x[i] = acc / T_AT(i, i);
                }
            else
                for (int64_t i = dim - 1; i >= 0; --i)
                {
                    double acc = (double)alpha * (double)b[B_IDX(i)];
                    for (int64_t k = i + 1; k < dim; ++k) acc -= T_AT(i, k) * x[k];
                    x[i] = acc / T_AT(i, i);
                }
            for (int64_t i = 0; i < dim; ++i) x_out64[B_IDX(i)] = x[i];
            #undef B_IDX
            #undef T_AT
        }
    }
    free(t); free(x);
    return 0;
}

/*
 * oracle_dgemm_f80acc: the FLOAT64 branch of the GEMM front-end (src/ops/blas/level3/gemm.cpp:158-169:
 * the same derivation as fp32, alpha / beta widened to double, forwarding to oneMKL gemm[_batch]<double>),
 * fp64 operands accumulated in x87 extended precision (64-bit significand), so that the result can
 * judge an fp64 kernel.  Argument meaning as oracle_gemm_f64acc; c_out80 receives the result as
 * long double, abs_ab (optional) sum_k |a||b|.  The reference holds no fp64 GEMM test; this function
 * is pinned by the reference's fp32 known answers (exactly representable) evaluated in double.
 */
int oracle_dgemm_f80acc(int layout_row, int trans_a, int trans_b, int64_t m, int64_t n, int64_t k, double alpha,
                        const double* a, int64_t lda, int64_t stride_a, const double* b, int64_t ldb, int64_t stride_b,
                        double beta, const double* c_in, int64_t ldc, int64_t stride_c, int64_t batch,
                        long double* c_out80, double* abs_ab)
{
    if (m < 0 || n < 0 || k < 0 || batch < 0 || !c_out80) return -1;
    long double* acc = (long double*)malloc(sizeof(long double) * (size_t)(n > 0 ? n : 1) * 2);
    if (!acc) return -2;
    long double* accabs = acc + (n > 0 ? n : 1);
    for (int64_t bi = 0; bi < batch; ++bi)
    {
        const double* ab = a + bi * stride_a;
        const double* bb = b + bi * stride_b;
        for (int64_t i = 0; i < m; ++i)
        {
            for (int64_t j = 0; j < n; ++j) { acc[j] = 0.0L; accabs[j] = 0.0L; }
            for (int64_t kk = 0; kk < k; ++kk)
            {
                long double av = (long double)ab[op_index(layout_row, trans_a, i, kk, lda)];
                long double aabs = fabsl(av);
                for (int64_t j = 0; j < n; ++j)
                {
                    long double bv = (long double)bb[op_index(layout_row, trans_b, kk, j, ldb)];
                    acc[j] += av * bv;
                    accabs[j] += aabs * fabsl(bv);
                }
            }
            for (int64_t j = 0; j < n; ++j)
            {
                int64_t ci = bi * stride_c + (layout_row ? i * ldc + j : j * ldc + i);
                long double v = (long double)alpha * acc[j];
                if (beta != 0.0) v += (long double)beta * (long double)c_in[ci];
                c_out80[ci] = v;
                if (abs_ab) abs_ab[ci] = (double)accabs[j];
            }
        }
    }
    free(acc);
    return 0;
}
