"""Generates tests/golden/gemm_integer_kat.npz: integer-valued GEMM known answers.

Inputs are small integers, so every product and partial sum is an integer below 2^24 and
the fp32 result is exact under ANY summation order and under the 3xTF32 split (|x| < 2^11
fits the TF32 mantissa).  The expected values are computed here with int64 arithmetic --
independently of the oracle -- and any conforming GEMM, the reference's included
(oneMKL sgemm behind src/ops/blas/level3/gemm.cpp:58,63), must reproduce them bit for bit.
The first two cases are the reference's own value-pinning tests
(tests/blas/level3/test_gemm.cpp:39-63 and 65-88).

Run:  python tests/golden/make_golden.py
"""
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def case(rng, name, ta, tb, m, n, k, alpha, beta, batch=1, pad=(0, 0, 0), lo=-8, hi=9):
    a_rows, a_cols = (k, m) if ta else (m, k)
    b_rows, b_cols = (n, k) if tb else (k, n)
    lda, ldb, ldc = a_cols + pad[0], b_cols + pad[1], n + pad[2]
    sa, sb, sc = a_rows * lda, b_rows * ldb, m * ldc
    a = rng.integers(lo, hi, size=(batch, a_rows, lda)).astype(np.int64)
    b = rng.integers(lo, hi, size=(batch, b_rows, ldb)).astype(np.int64)
    c = rng.integers(lo, hi, size=(batch, m, ldc)).astype(np.int64)
    opa = a[:, :, :a_cols].transpose(0, 2, 1) if ta else a[:, :, :a_cols]
    opb = b[:, :, :b_cols].transpose(0, 2, 1) if tb else b[:, :, :b_cols]
    out = c.copy()
    prod = alpha * np.matmul(opa, opb)
    out[:, :, :n] = prod + (beta * c[:, :, :n] if beta != 0 else 0)
    assert np.abs(np.matmul(np.abs(opa), np.abs(opb))).max() * abs(alpha) < 2 ** 23
    return {
        f"{name}.meta": np.array([ta, tb, m, n, k, alpha, beta, batch, lda, ldb, ldc, sa, sb, sc], dtype=np.int64),
        f"{name}.a": a.astype(np.float32).ravel(),
        f"{name}.b": b.astype(np.float32).ravel(),
        f"{name}.c_in": c.astype(np.float32).ravel(),
        f"{name}.c_out": out.astype(np.float32).ravel(),
    }


def main():
    rng = np.random.default_rng(20240601)
    d = {}
    # reference KAT 1: row-major 3x3, A = 1..9, B = 2*I, C = 0, NN, alpha=1, beta=0 -> 2*A
    a = np.arange(1, 10, dtype=np.float32)
    b = (2 * np.eye(3, dtype=np.float32)).ravel()
    d["ref_simple3x3.meta"] = np.array([0, 0, 3, 3, 3, 1, 0, 1, 3, 3, 3, 9, 9, 9], dtype=np.int64)
    d["ref_simple3x3.a"], d["ref_simple3x3.b"] = a, b
    d["ref_simple3x3.c_in"] = np.zeros(9, dtype=np.float32)
    d["ref_simple3x3.c_out"] = np.array([2, 4, 6, 8, 10, 12, 14, 16, 18], dtype=np.float32)
    # reference KAT 2: column-major 2x2x2; memory images as in the reference test
    d["ref_colmajor2x2.a"] = np.array([1, 3, 2, 4], dtype=np.float32)
    d["ref_colmajor2x2.b"] = np.array([5, 7, 6, 8], dtype=np.float32)
    d["ref_colmajor2x2.c_out"] = np.array([19, 43, 22, 50], dtype=np.float32)

    # reference SYRK KATs (tests/blas/level3/test_syrk.cpp:39-103): row-major lower 3x3 (A 3x2 = 1..6)
    # and column-major lower with transA (A stored K x N = 3 x 2, memory 1..6) -> {14, 32, 0, 77}
    d["ref_syrk_lower3.a"] = np.arange(1, 7, dtype=np.float32)
    d["ref_syrk_lower3.c_out"] = np.array([5, 0, 0, 11, 25, 0, 17, 39, 61], dtype=np.float32)
    d["ref_syrk_colmajor_trans.a"] = np.arange(1, 7, dtype=np.float32)
    d["ref_syrk_colmajor_trans.c_out"] = np.array([14, 32, 0, 77], dtype=np.float32)

    names = []
    specs = [
        ("nn_small", 0, 0, 5, 7, 3, 1, 0, 1, (0, 0, 0)),
        ("nt_small", 0, 1, 6, 4, 9, 2, 1, 1, (0, 0, 0)),
        ("tn_small", 1, 0, 4, 6, 5, -1, 2, 1, (1, 2, 3)),
        ("tt_small", 1, 1, 7, 5, 8, 3, -1, 1, (2, 0, 1)),
        ("nn_batched", 0, 0, 9, 8, 7, 1, 0, 3, (0, 0, 0)),
        ("tn_batched_beta", 1, 0, 8, 9, 6, 2, 1, 2, (0, 0, 0)),
        ("nn_tile", 0, 0, 256, 256, 64, 1, 0, 1, (0, 0, 0)),
        ("nt_tile", 0, 1, 256, 512, 48, 1, 1, 1, (0, 0, 0)),
        ("tn_ragged", 1, 0, 300, 260, 100, 2, -1, 1, (4, 0, 4)),
        ("tt_ragged_batched", 1, 1, 130, 270, 77, 1, 2, 2, (0, 4, 0)),
        ("nn_odd_ld", 0, 0, 129, 131, 65, 1, 1, 1, (1, 3, 5)),
    ]
    for name, ta, tb, m, n, k, alpha, beta, batch, pad in specs:
        big = m * n * k > 100000
        d.update(case(rng, name, ta, tb, m, n, k, alpha, beta, batch, pad, lo=-4 if big else -8, hi=5 if big else 9))
        names.append(name)
    d["names"] = np.array(names)
    np.savez_compressed(os.path.join(HERE, "gemm_integer_kat.npz"), **d)
    print("wrote", len(names) + 4, "cases")


if __name__ == "__main__":
    main()
