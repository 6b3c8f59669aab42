"""The result check bench.py runs after its timed region, exercised on the CPU: the host twin of the
library's counter-based generator, and the sampled float64 comparison with its tolerance."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import bench
from oracle import ref_gemm as og


def test_host_generator_matches_the_oracle_generator():
    idx = np.arange(1000, 5000, dtype=np.uint64)
    assert np.array_equal(bench.uniform_at(7, idx).astype(np.float32), og.uniform_pm1(7, 4000, start=1000))
    g = bench.GenMatrix(7, ld=50, first_index=100)
    full = og.uniform_pm1(7, 100 + 50 * 40).astype(np.float64)
    assert np.array_equal(g.block([3, 9], [0, 49, 7]), np.array([[full[100 + r * 50 + c] for c in (0, 49, 7)] for r in (3, 9)]))


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_check_accepts_an_fp32_product_and_rejects_a_wrong_one(ta, tb):
    torch = pytest.importorskip("torch")
    m, n, k, alpha, beta = 96, 80, 64, 1.5, 0.5
    a_mat = bench.GenMatrix(1, m if ta else k)
    b_mat = bench.GenMatrix(2, k if tb else n)
    c_mat = bench.GenMatrix(3, n)
    a = a_mat.block(np.arange(k if ta else m), np.arange(m if ta else k)).astype(np.float32)
    b = b_mat.block(np.arange(n if tb else k), np.arange(k if tb else n)).astype(np.float32)
    c_in = c_mat.block(np.arange(m), np.arange(n)).astype(np.float32)
    c = (np.float32(alpha) * ((a.T if ta else a) @ (b.T if tb else b)) + np.float32(beta) * c_in).astype(np.float32)
    read = lambda rows: c[np.asarray(rows)].astype(np.float64)
    for mats in ((a_mat, b_mat), (bench.TensorMatrix(torch.from_numpy(a)), bench.TensorMatrix(torch.from_numpy(b)))):
        r, s = bench.check_gemm(ta, tb, m, n, k, alpha, beta, mats[0], mats[1], c_mat, read, np.random.default_rng(0), k_chunk=24)
        assert r <= 1.0 and s == 64 + 4 * n
    bad = c.copy()
    bad[:, 5] += 1e-3
    r, _ = bench.check_gemm(ta, tb, m, n, k, alpha, beta, a_mat, b_mat, c_mat, lambda rows: bad[np.asarray(rows)].astype(np.float64),
                            np.random.default_rng(0))
    assert r > 1.0


def test_both_arms_print_the_same_config_object():
    for name, w in bench.GEMM_WORKLOADS.items():
        cfg = bench.config_of(name, w)
        assert set(cfg) == {"workload", "m", "n", "k", "batch", "alpha", "beta", "transposes"}
