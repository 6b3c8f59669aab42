"""CPU oracle for the fp32 GEMM path -- TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the CPU-baseline / reference legs of the
benchmark may import this module.  The shipped library never does.

It restates, for checking purposes:

* the Tensor stride rule of the reference (include/SushiBLAS/tensor.hpp:99-116),
* the BLAS-parameter derivation of ``Level3::gemm``
  (src/ops/blas/level3/gemm.cpp:87-105),
* the arithmetic the reference delegates to Intel oneMKL
  (``oneapi::mkl::blas::{row,column}_major::gemm[_batch]``, gemm.cpp:58,63,71,76;
  oneMKL is neither vendored nor version-pinned in the reference tree), following
  the BLAS definition quoted in include/SushiBLAS/ops/blas/level3.hpp:57-70, with
  fp64 accumulation.

Pinning status: the oracle reproduces the two value-pinning tests the reference has
for this path (tests/blas/level3/test_gemm.cpp:39-63, 65-88).  For transposes,
alpha/beta and batching the reference holds no test, so parity there is pinned only
by exact integer-valued known answers (tests/golden/).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Sequence, Tuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

U24 = 2.0 ** -24


# --------------------------------------------------------------------------- C side
def build(force: bool = False) -> str:
    """Compile ref_gemm.c into liboracle_gemm.so (next to this file)."""
    so = os.path.join(_HERE, "liboracle_gemm.so")
    src = os.path.join(_HERE, "ref_gemm.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return so


def _lib():
    global _LIB
    if _LIB is None:
        lib = ctypes.CDLL(build())
        i64, f32, dbl = ctypes.c_int64, ctypes.c_float, ctypes.c_double
        p = ctypes.c_void_p
        lib.oracle_gemm_f64acc.restype = ctypes.c_int
        lib.oracle_gemm_f64acc.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                           i64, i64, i64, f32, p, i64, i64, p, i64, i64,
                                           f32, p, i64, i64, i64, p, p]
        lib.oracle_gemm_f32.restype = ctypes.c_int
        lib.oracle_gemm_f32.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                        i64, i64, i64, f32, p, i64, i64, p, i64, i64,
                                        f32, p, i64, i64, i64]
        lib.oracle_syrk_f64acc.restype = ctypes.c_int
        lib.oracle_syrk_f64acc.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, i64, i64, f32, p, i64, i64, f32,
                                           p, i64, i64, i64, p, p]
        lib.oracle_trsm_f64.restype = ctypes.c_int
        lib.oracle_trsm_f64.argtypes = [ctypes.c_int] * 5 + [i64, i64, f32, p, i64, i64, p, i64, i64, i64, p]
        lib.oracle_dgemm_f80acc.restype = ctypes.c_int
        lib.oracle_dgemm_f80acc.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, i64, i64, i64, dbl, p, i64, i64,
                                            p, i64, i64, dbl, p, i64, i64, i64, p, p]
        lib.oracle_check_tolerance.restype = dbl
        lib.oracle_check_tolerance.argtypes = [i64, i64, i64, i64, f32, dbl, p, p, p, p,
                                               i64, i64, ctypes.POINTER(dbl)]
        _LIB = lib
    return _LIB


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


# ------------------------------------------------------------ front-end restatement
ROW_MAJOR, COLUMN_MAJOR = 0, 1


def tensor_strides(dims: Sequence[int], layout: int = ROW_MAJOR) -> Tuple[int, ...]:
    """Contiguous strides as the reference Tensor constructor computes them
    (tensor.hpp:99-107 row-major: last dim fastest; 108-116 column-major: first dim
    fastest)."""
    strides = [0] * len(dims)
    e = 1
    order = range(len(dims) - 1, -1, -1) if layout == ROW_MAJOR else range(len(dims))
    for i in order:
        strides[i] = e
        e *= dims[i]
    return tuple(strides)


def derive_gemm_params(shape_a, strides_a, shape_b, strides_b, shape_c, strides_c,
                       trans_a: bool, trans_b: bool, layout: int = ROW_MAJOR) -> dict:
    """m, n, k, batch, lda/ldb/ldc and batch strides exactly as gemm.cpp:87-105.

    * rank >= 2 is required (gemm.cpp:87);
    * m, n come from C, k from A (gemm.cpp:91-93);
    * batch is the product of C's leading dims (gemm.cpp:96-97);
    * ld* come from *shape* (last dim for row-major, second-to-last for column-major),
      not from strides (gemm.cpp:99-101);
    * batch strides are strides[rank-3] when batch > 1, else 0 (gemm.cpp:103-105).
    """
    ra, rb, rc = len(shape_a), len(shape_b), len(shape_c)
    if ra < 2 or rb < 2 or rc < 2:
        raise RuntimeError("GEMM requires at least 2D tensors.")
    m, n = shape_c[rc - 2], shape_c[rc - 1]
    k = shape_a[ra - 2] if trans_a else shape_a[ra - 1]
    batch = 1
    for d in shape_c[: rc - 2]:
        batch *= d
    row = layout == ROW_MAJOR
    lda = shape_a[ra - 1] if row else shape_a[ra - 2]
    ldb = shape_b[rb - 1] if row else shape_b[rb - 2]
    ldc = shape_c[rc - 1] if row else shape_c[rc - 2]
    if batch > 1 and (ra < 3 or rb < 3):
        # the reference would read strides[-1] here (undefined behaviour)
        raise RuntimeError("batched GEMM needs rank >= 3 operands")
    sa = strides_a[ra - 3] if batch > 1 else 0
    sb = strides_b[rb - 3] if batch > 1 else 0
    sc = strides_c[rc - 3] if batch > 1 else 0
    return dict(m=m, n=n, k=k, batch=batch, lda=lda, ldb=ldb, ldc=ldc,
                stride_a=sa, stride_b=sb, stride_c=sc)


# ------------------------------------------------------------------- arithmetic
def gemm_f64_c(trans_a, trans_b, m, n, k, alpha, a, lda, stride_a, b, ldb, stride_b,
               beta, c_in, ldc, stride_c, batch, layout=ROW_MAJOR, want_abs=True):
    """fp64-accumulated GEMM through the C restatement.  a, b, c_in are flat float32
    buffers.  Returns (c_ref float64 flat, abs_ab float64 flat or None) indexed like C."""
    a = np.ascontiguousarray(a, dtype=np.float32).ravel()
    b = np.ascontiguousarray(b, dtype=np.float32).ravel()
    c_in32 = None if c_in is None else np.ascontiguousarray(c_in, dtype=np.float32).ravel()
    size_c = _extent(m, n, ldc, stride_c, batch, layout)
    out = np.zeros(size_c, dtype=np.float64)
    absab = np.zeros(size_c, dtype=np.float64) if want_abs else None
    rc = _lib().oracle_gemm_f64acc(1 if layout == ROW_MAJOR else 0, int(trans_a), int(trans_b),
                                   m, n, k, alpha, _ptr(a), lda, stride_a, _ptr(b), ldb, stride_b,
                                   beta, _ptr(c_in32), ldc, stride_c, batch, _ptr(out), _ptr(absab))
    if rc != 0:
        raise ValueError("oracle_gemm_f64acc rejected its arguments")
    return out, absab


def syrk_f64_c(upper, trans, n, k, alpha, a, lda, stride_a, beta, c_in, ldc, stride_c, batch, layout=ROW_MAJOR):
    """fp64-accumulated SYRK through the C restatement (syrk.cpp:84-116 semantics).  Returns
    (c float64 flat indexed like C, with the untouched triangle equal to c_in; abs_aa)."""
    a = np.ascontiguousarray(a, dtype=np.float32).ravel()
    c32 = np.ascontiguousarray(c_in, dtype=np.float32).ravel()
    out = c32.astype(np.float64)
    absaa = np.zeros(out.shape, dtype=np.float64)
    rc = _lib().oracle_syrk_f64acc(1 if layout == ROW_MAJOR else 0, int(upper), int(trans), n, k, alpha, _ptr(a), lda,
                                   stride_a, beta, _ptr(c32), ldc, stride_c, batch, _ptr(out), _ptr(absaa))
    if rc != 0:
        raise ValueError("oracle_syrk_f64acc rejected its arguments")
    return out, absaa


def syrk_f64_np(upper, trans, n, k, alpha, a, lda, stride_a, beta, c_in, ldc, stride_c, batch):
    """numpy twin for row-major storage and larger sizes: the GEMM oracle with B = A, masked to
    the triangle.  Returns dense (batch, n, n): result (other triangle = c_in), abs_aa, mask."""
    full, absab = gemm_f64_np(trans, not trans, n, n, k, alpha, a, lda, stride_a, a, lda, stride_a, beta, c_in, ldc,
                              stride_c, batch)
    c32 = np.asarray(c_in, dtype=np.float32).ravel()
    cin = _view(c32, n, n, ldc, stride_c, batch).astype(np.float64)
    i, j = np.indices((n, n))
    mask = (j >= i) if upper else (j <= i)
    return np.where(mask[None], full, cin), np.where(mask[None], absab, 0.0), mask


def dgemm_f80_c(trans_a, trans_b, m, n, k, alpha, a, lda, stride_a, b, ldb, stride_b, beta, c_in, ldc, stride_c, batch,
                layout=ROW_MAJOR):
    """FLOAT64 GEMM (gemm.cpp:158-169) accumulated in x87 extended precision through the C
    restatement.  Returns (c: np.longdouble flat array indexed like C, abs_ab: float64)."""
    assert np.finfo(np.longdouble).nmant >= 63, "this oracle needs an extended-precision long double"
    a = np.ascontiguousarray(a, dtype=np.float64).ravel()
    b = np.ascontiguousarray(b, dtype=np.float64).ravel()
    c64 = np.ascontiguousarray(c_in, dtype=np.float64).ravel()
    out = c64.astype(np.longdouble)
    absab = np.zeros(out.shape, dtype=np.float64)
    rc = _lib().oracle_dgemm_f80acc(1 if layout == ROW_MAJOR else 0, int(trans_a), int(trans_b), m, n, k, alpha,
                                    _ptr(a), lda, stride_a, _ptr(b), ldb, stride_b, beta, _ptr(c64), ldc, stride_c, batch,
                                    _ptr(out), _ptr(absab))
    if rc != 0:
        raise ValueError("oracle_dgemm_f80acc rejected its arguments")
    return out, absab


def tolerance_ratio_f64(got, ref, abs_ab, k, beta=0.0, c_in=None, budget=1.0):
    """fp64 form of the GEMM bound: max over elements of |got - ref| divided by
    budget * 8*K*2^-53 * (|A||B|) + 2^-53 * |beta * C_in|; <= 1 passes.  `ref` is extended precision."""
    got = np.asarray(got, dtype=np.float64)
    if not np.isfinite(got).all():
        return float("inf")
    err = np.abs(got.astype(np.longdouble) - np.asarray(ref, dtype=np.longdouble))
    u = np.longdouble(2.0) ** -53
    bound = budget * 8.0 * max(int(k), 1) * u * np.asarray(abs_ab, dtype=np.longdouble)
    if beta != 0.0 and c_in is not None:
        bound = bound + u * np.abs(np.longdouble(beta) * np.asarray(c_in, dtype=np.longdouble))
    bound = bound + np.longdouble(1e-300)
    return float(np.max(err / bound)) if err.size else 0.0


def trsm_f64_c(left, upper, trans, unit_diag, m, n, alpha, a, lda, stride_a, b, ldb, stride_b, batch, layout=ROW_MAJOR):
    """fp64 substitution through the C restatement (trsm.cpp:85-135 semantics).  Returns X as a
    float64 array indexed like B."""
    a = np.ascontiguousarray(a, dtype=np.float32).ravel()
    b32 = np.ascontiguousarray(b, dtype=np.float32).ravel()
    out = b32.astype(np.float64)
    rc = _lib().oracle_trsm_f64(1 if layout == ROW_MAJOR else 0, int(left), int(upper), int(trans), int(unit_diag), m, n,
                                alpha, _ptr(a), lda, stride_a, _ptr(b32), ldb, stride_b, batch, _ptr(out))
    if rc != 0:
        raise ValueError("oracle_trsm_f64 rejected its arguments")
    return out


def trsm_f64_np(left, upper, trans, unit_diag, m, n, alpha, a, lda, stride_a, b, ldb, stride_b, batch):
    """numpy / LAPACK twin for row-major storage and larger sizes: float64 solve_triangular on the
    referenced triangle.  Returns dense (batch, m, n) float64 X and the dense op(A) used."""
    from scipy.linalg import solve_triangular
    dim = m if left else n
    a32 = np.asarray(a, dtype=np.float32).ravel()
    b32 = np.asarray(b, dtype=np.float32).ravel()
    av = _view(a32, dim, dim, lda, stride_a, batch).astype(np.float64)
    bv = _view(b32, m, n, ldb, stride_b, batch).astype(np.float64)
    xs, ts = [], []
    for i in range(batch):
        tri = np.triu(av[i]) if upper else np.tril(av[i])
        if unit_diag:
            np.fill_diagonal(tri, 1.0)
        t = tri.T if trans else tri
        lower = (bool(upper) == bool(trans))
        if left:
            x = solve_triangular(t, alpha * bv[i], lower=lower)
        else:
            x = solve_triangular(t.T, alpha * bv[i].T, lower=not lower).T
        xs.append(x)
        ts.append(t)
    return np.stack(xs), np.stack(ts)


def trsm_residual_ratio(left, t, x, alpha, b, dim):
    """Componentwise backward-error ratio of a computed solve against the budget
    8 * dim * 2^-24 * (|op(A)| |X| + |alpha B|): <= 1 passes."""
    x = np.asarray(x, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    if left:
        r = t @ x - alpha * b
        scale = np.abs(t) @ np.abs(x) + np.abs(alpha * b)
    else:
        r = x @ t - alpha * b
        scale = np.abs(x) @ np.abs(t) + np.abs(alpha * b)
    bound = 8.0 * max(dim, 1) * 2.0 ** -24 * scale + 1e-37
    return float(np.max(np.abs(r) / bound)) if r.size else 0.0


def gemm_f32_c(trans_a, trans_b, m, n, k, alpha, a, lda, stride_a, b, ldb, stride_b,
               beta, c, ldc, stride_c, batch, layout=ROW_MAJOR):
    """Scalar fp32 triple loop (in place on a copy of c); the slow 'port' timing leg."""
    a = np.ascontiguousarray(a, dtype=np.float32).ravel()
    b = np.ascontiguousarray(b, dtype=np.float32).ravel()
    c = np.array(c, dtype=np.float32).ravel()
    rc = _lib().oracle_gemm_f32(1 if layout == ROW_MAJOR else 0, int(trans_a), int(trans_b),
                                m, n, k, alpha, _ptr(a), lda, stride_a, _ptr(b), ldb, stride_b,
                                beta, _ptr(c), ldc, stride_c, batch)
    if rc != 0:
        raise ValueError("oracle_gemm_f32 rejected its arguments")
    return c


def _extent(m, n, ld, stride, batch, layout=ROW_MAJOR):
    rows, cols = (m, n) if layout == ROW_MAJOR else (n, m)
    if rows == 0 or cols == 0 or batch == 0:
        return max(1, (batch - 1) * stride + 1) if batch else 1
    return (batch - 1) * stride + (rows - 1) * ld + cols


def _view(buf, rows, cols, ld, stride, batch):
    """(batch, rows, cols) strided view over a flat buffer (row-major, leading dim ld)."""
    it = buf.itemsize
    return np.lib.stride_tricks.as_strided(buf, shape=(batch, rows, cols),
                                           strides=(stride * it, ld * it, it), writeable=False)


def gemm_f64_np(trans_a, trans_b, m, n, k, alpha, a, lda, stride_a, b, ldb, stride_b,
                beta, c_in, ldc, stride_c, batch, want_abs=True):
    """numpy twin of gemm_f64_c for row-major storage (float64 matmul); used for the
    sizes the scalar C loop is too slow for.  Returns dense (batch, m, n) arrays."""
    a = np.asarray(a, dtype=np.float32).ravel()
    b = np.asarray(b, dtype=np.float32).ravel()
    av = _view(a, k if trans_a else m, m if trans_a else k, lda, stride_a, batch)
    bv = _view(b, n if trans_b else k, k if trans_b else n, ldb, stride_b, batch)
    a64 = av.astype(np.float64)
    b64 = bv.astype(np.float64)
    if trans_a:
        a64 = a64.transpose(0, 2, 1)
    if trans_b:
        b64 = b64.transpose(0, 2, 1)
    ref = np.float64(np.float32(alpha)) * np.matmul(a64, b64)
    if beta != 0.0:
        c32 = np.asarray(c_in, dtype=np.float32).ravel()
        ref = ref + np.float64(np.float32(beta)) * _view(c32, m, n, ldc, stride_c, batch).astype(np.float64)
    absab = np.matmul(np.abs(a64), np.abs(b64)) if want_abs else None
    return ref, absab


def tolerance_ratio(c_test, c_ref, abs_ab, k, beta=0.0, c_in=None, budget=1.0):
    """max |c_test - c_ref| / (budget*8*K*2^-24*(|A||B|) + 2^-24*|beta*C_in|) over dense
    arrays of equal shape; <= 1 passes.  `budget` scales the K term only: the beta term is
    one fp32 rounding of the output, which no fp32 result can halve.  Second value: max
    error in units of 2^-24*((|A||B|) + |beta*C_in|) (no K factor)."""
    c_test = np.asarray(c_test, dtype=np.float64)
    err = np.abs(c_test - c_ref)
    if not np.all(np.isfinite(c_test)):
        return float("inf"), float("inf")
    bound = budget * 8.0 * k * U24 * abs_ab
    scale = abs_ab
    if beta != 0.0 and c_in is not None:
        bc = np.abs(np.float64(np.float32(beta)) * np.asarray(c_in, dtype=np.float64))
        bound = bound + U24 * bc
        scale = abs_ab + bc
    with np.errstate(divide="ignore", invalid="ignore"):
        r = np.where(bound > 0, err / bound, np.where(err == 0, 0.0, np.inf))
        q = np.where(scale > 0, err / (U24 * scale), 0.0)
    return float(r.max(initial=0.0)), float(q.max(initial=0.0))


def engine_gemm(a_buf, shape_a, b_buf, shape_b, c_buf, shape_c, trans_a=False, trans_b=False,
                alpha=1.0, beta=0.0, layout=ROW_MAJOR):
    """What ``engine.blas().gemm(A, B, C, tA, tB, alpha, beta)`` computes on contiguous
    tensors created by ``Engine::create_tensor`` with the given layout: parameters from
    derive_gemm_params, arithmetic from the C restatement.  Buffers are the tensors'
    storage in memory order.  Returns (C result float64 in memory order, abs_ab)."""
    p = derive_gemm_params(shape_a, tensor_strides(shape_a, layout), shape_b, tensor_strides(shape_b, layout),
                           shape_c, tensor_strides(shape_c, layout), trans_a, trans_b, layout)
    return gemm_f64_c(trans_a, trans_b, p["m"], p["n"], p["k"], alpha, a_buf, p["lda"], p["stride_a"],
                      b_buf, p["ldb"], p["stride_b"], beta, c_buf, p["ldc"], p["stride_c"], p["batch"],
                      layout=layout)


# ------------------------------------------------------------ seeded input generator
_GOLDEN = np.uint64(0x9E3779B97F4A7C15)


def _splitmix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = x + _GOLDEN
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def hash_u32(seed: int, start: int, count: int) -> np.ndarray:
    """Counter-based 32-bit stream: element i is a pure function of (seed, i)."""
    idx = np.arange(start, start + count, dtype=np.uint64)
    with np.errstate(over="ignore"):
        key = _splitmix64(np.full(1, seed, dtype=np.uint64))[0]
        return (_splitmix64(idx ^ key) >> np.uint64(32)).astype(np.uint32)


def uniform_pm1(seed: int, count: int, start: int = 0) -> np.ndarray:
    """i.i.d. uniform [-1, 1) float32: (u32 >> 8) * 2^-23 - 1 (exact in fp32, so the
    device generator in the library produces bit-identical values)."""
    u = hash_u32(seed, start, count) >> np.uint32(8)
    return (u.astype(np.float32) * np.float32(2.0 ** -23) - np.float32(1.0)).astype(np.float32)


def normal(seed: int, count: int, std: float = 1.0, start: int = 0) -> np.ndarray:
    """i.i.d. normal(0, std) float32 by Box-Muller on two counter-based uniforms
    (host only; evaluated in float64 and rounded once)."""
    u1 = (hash_u32(seed, start, count) >> np.uint32(8)).astype(np.float64) * 2.0 ** -24
    u2 = (hash_u32(seed ^ 0x5DEECE66D, start, count) >> np.uint32(8)).astype(np.float64) * 2.0 ** -24
    r = np.sqrt(-2.0 * np.log(1.0 - u1))
    return (std * r * np.cos(2.0 * np.pi * u2)).astype(np.float32)


# ------------------------------------------------ MKL proxy for the reference CPU path
def mkl_proxy_gemm(trans_a, trans_b, alpha, a, b, beta, c, threads=None):
    """The closest runnable stand-in for the reference's CPU arithmetic: Intel MKL sgemm
    as linked into PyTorch's CPU build (the reference calls oneMKL's DPC++ BLAS,
    gemm.cpp:58,63, which on a CPU device dispatches to the same sgemm family).
    a, b, c are torch CPU float32 tensors (2-D or 3-D batched); c is updated in place
    and returned.  This is a timing baseline, not the correctness oracle."""
    import torch

    if threads:
        torch.set_num_threads(int(threads))
    opa = a.transpose(-1, -2) if trans_a else a
    opb = b.transpose(-1, -2) if trans_b else b
    with torch.backends.mkldnn.flags(enabled=False):
        if a.dim() == 2:
            if beta == 0.0:
                torch.mm(opa, opb, out=c)
                if alpha != 1.0:
                    c.mul_(alpha)
            else:
                torch.addmm(c, opa, opb, beta=beta, alpha=alpha, out=c)
        else:
            if beta == 0.0:
                torch.bmm(opa, opb, out=c)
                if alpha != 1.0:
                    c.mul_(alpha)
            else:
                torch.baddbmm(c, opa, opb, beta=beta, alpha=alpha, out=c)
    return c
