"""ctypes binding of the C ABI in include/sushiblas_cuda.h.

Thin by design: every method forwards to exactly one exported function and raises
``SushiCudaError`` on a non-zero status.  There is no fallback: if the shared library is
missing it is an error, and every compute call needs a CUDA device.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Sequence

from ._build import LIB_PATH

_i64 = ctypes.c_int64
_f32 = ctypes.c_float
_f64 = ctypes.c_double
_int = ctypes.c_int
_vp = ctypes.c_void_p
_sz = ctypes.c_size_t

GEMM_AUTO, GEMM_SIMT, GEMM_TC3X = 0, 1, 2

class GemmDesc(ctypes.Structure):
    """sushi_cuda_gemm_desc"""
    _fields_ = [("trans_a", ctypes.c_int32), ("trans_b", ctypes.c_int32),
                ("m", _i64), ("n", _i64), ("k", _i64), ("alpha", _f32),
                ("a", _vp), ("lda", _i64), ("stride_a", _i64),
                ("b", _vp), ("ldb", _i64), ("stride_b", _i64),
                ("beta", _f32), ("c", _vp), ("ldc", _i64), ("stride_c", _i64),
                ("batch", _i64), ("epilogue", ctypes.c_int32), ("act_param", _f32)]


# name -> (restype, argtypes); mirrors include/sushiblas_cuda.h one to one
SIGNATURES = {
    "sushi_cuda_device_count": (_int, [ctypes.POINTER(_int)]),
    "sushi_cuda_init": (_int, [ctypes.POINTER(_int), _int, ctypes.POINTER(_vp)]),
    "sushi_cuda_destroy": (_int, [_vp]),
    "sushi_cuda_last_error": (ctypes.c_char_p, [_vp]),
    "sushi_cuda_sync": (_int, [_vp, _int]),
    "sushi_cuda_set_stream": (_int, [_vp, _int, _vp]),
    "sushi_cuda_get_stream": (_int, [_vp, _int, ctypes.POINTER(_vp)]),
    "sushi_cuda_selftest_bounded_wait": (_int, [_vp, _int, _int]),
    "sushi_cuda_set_gemm_variant": (_int, [_vp, _int]),
    "sushi_cuda_launch_count": (_int, [_vp, ctypes.POINTER(_i64)]),
    "sushi_cuda_inject_failure": (_int, [_vp, _int, _int]),
    "sushi_cuda_copy_bytes": (_int, [_vp, ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_uint64)]),
    "sushi_cuda_kernel_timing_enable": (_int, [_vp, _int]),
    "sushi_cuda_kernel_timing_read": (_int, [_vp, _int, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(_i64),
                                             ctypes.POINTER(ctypes.c_double), ctypes.POINTER(_i64)]),
    "sushi_cuda_malloc": (_int, [_vp, _int, _sz, ctypes.POINTER(_vp)]),
    "sushi_cuda_free": (_int, [_vp, _int, _vp]),
    "sushi_cuda_host_alloc": (_int, [_vp, _sz, ctypes.POINTER(_vp)]),
    "sushi_cuda_host_free": (_int, [_vp, _vp]),
    "sushi_cuda_memcpy_h2d": (_int, [_vp, _int, _vp, _vp, _sz]),
    "sushi_cuda_memcpy_d2h": (_int, [_vp, _int, _vp, _vp, _sz]),
    "sushi_cuda_memcpy_d2d": (_int, [_vp, _int, _vp, _vp, _sz]),
    "sushi_cuda_memset": (_int, [_vp, _int, _vp, _int, _sz]),
    "sushi_cuda_upload_fence": (_int, [_vp, _int]),
    "sushi_cuda_upload_ahead": (_int, [_vp, _int, _vp, _vp, _sz]),
    "sushi_cuda_marker_create": (_int, [_vp, _int, ctypes.POINTER(_vp)]),
    "sushi_cuda_marker_record": (_int, [_vp, _int, _vp]),
    "sushi_cuda_marker_destroy": (_int, [_vp, _vp]),
    "sushi_cuda_download_behind": (_int, [_vp, _int, _vp, _vp, _sz, _vp]),
    "sushi_cuda_sgemm": (_int, [_vp, _int, _int, _int, _i64, _i64, _i64, _f32, _vp, _i64, _vp, _i64,
                                _f32, _vp, _i64]),
    "sushi_cuda_sgemm_strided_batched": (_int, [_vp, _int, _int, _int, _i64, _i64, _i64, _f32,
                                                _vp, _i64, _i64, _vp, _i64, _i64, _f32, _vp, _i64, _i64, _i64]),
    "sushi_cuda_sgemm_strided_batched_ex": (_int, [_vp, _int, _int, _int, _i64, _i64, _i64, _f32,
                                                   _vp, _i64, _i64, _vp, _i64, _i64, _f32, _vp, _i64, _i64, _i64, _int]),
    "sushi_cuda_relu": (_int, [_vp, _int, _vp, _i64]),
    "sushi_cuda_activation": (_int, [_vp, _int, _int, _f32, _vp, _i64]),
    "sushi_cuda_activation_backward": (_int, [_vp, _int, _int, _f32, _vp, _vp, _vp, _i64]),
    "sushi_cuda_sgemm_strided_batched_act": (_int, [_vp, _int, _int, _int, _i64, _i64, _i64, _f32, _vp, _i64, _i64,
                                                    _vp, _i64, _i64, _f32, _vp, _i64, _i64, _i64, _int, _f32]),
    "sushi_cuda_ssyrk": (_int, [_vp, _int, _int, _int, _i64, _i64, _f32, _vp, _i64, _f32, _vp, _i64]),
    "sushi_cuda_ssyrk_strided_batched": (_int, [_vp, _int, _int, _int, _i64, _i64, _f32, _vp, _i64, _i64, _f32,
                                                _vp, _i64, _i64, _i64]),
    "sushi_cuda_dgemm": (_int, [_vp, _int, _int, _int, _i64, _i64, _i64, _f64, _vp, _i64, _vp, _i64, _f64, _vp, _i64]),
    "sushi_cuda_dgemm_strided_batched": (_int, [_vp, _int, _int, _int, _i64, _i64, _i64, _f64, _vp, _i64, _i64,
                                                _vp, _i64, _i64, _f64, _vp, _i64, _i64, _i64]),
    "sushi_cuda_strsm": (_int, [_vp, _int, _int, _int, _int, _int, _i64, _i64, _f32, _vp, _i64, _vp, _i64]),
    "sushi_cuda_strsm_strided_batched": (_int, [_vp, _int, _int, _int, _int, _int, _i64, _i64, _f32, _vp, _i64, _i64,
                                                _vp, _i64, _i64, _i64]),
    "sushi_cuda_sgemm_grouped": (_int, [_vp, _int, ctypes.POINTER(GemmDesc), _i64]),
    "sushi_cuda_sgemm_strided_batched_host": (_int, [_vp, _int, _int, _int, _i64, _i64, _i64, _f32,
                                                     _vp, _i64, _i64, _vp, _i64, _i64, _f32, _vp, _i64, _i64, _i64]),
    "sushi_cuda_gemm_workspace_bytes": (_int, [_i64, _i64, _i64, _i64, ctypes.POINTER(_sz)]),
    "sushi_cuda_reserve_workspace": (_int, [_vp, _int, _sz]),
    "sushi_cuda_partition": (_int, [_i64, _int, _int, ctypes.POINTER(_i64), ctypes.POINTER(_i64)]),
    "sushi_cuda_comm_unique_id": (_int, [_vp]),
    "sushi_cuda_comm_init_rank": (_int, [_vp, _int, _vp, _int, _int]),
    "sushi_cuda_comm_destroy": (_int, [_vp]),
    "sushi_cuda_ipc_export": (_int, [_vp, _int, _vp, _vp]),
    "sushi_cuda_ipc_open": (_int, [_vp, _int, _vp, ctypes.POINTER(_vp)]),
    "sushi_cuda_ipc_close": (_int, [_vp, _int, _vp]),
    "sushi_cuda_comm_set_peer_buffers": (_int, [_vp, _int, ctypes.POINTER(_vp), _int, _sz]),
    "sushi_cuda_row_sharded_exchange": (_int, [_i64, _i64, _i64, _int, _int, _int, _int, ctypes.POINTER(_int)]),
    "sushi_cuda_batch_sharded_exchange": (_int, [_i64, _i64, _i64, _i64, _int, _int, _int, _int, ctypes.POINTER(_int)]),
    "sushi_cuda_sgemm_row_sharded": (_int, [_vp, _int, _int, _int, _i64, _i64, _i64, _f32, _vp, _i64, _vp, _i64,
                                            _f32, _vp, _i64, _int]),
    "sushi_cuda_sgemm_row_sharded_host": (_int, [_vp, _int, _int, _int, _i64, _i64, _i64, _f32, _vp, _i64, _vp, _i64,
                                                 _f32, _vp, _i64, _vp, _vp, _vp]),
    "sushi_cuda_sgemm_batch_sharded": (_int, [_vp, _int, _int, _int, _i64, _i64, _i64, _f32,
                                              _vp, _i64, _i64, _vp, _i64, _i64, _f32, _vp, _i64, _i64, _i64, _int]),
    "sushi_cuda_sgemm_static_scratch": (_int, [_vp, _int, _int, _i64, _i64, _i64, _f32, _vp, _i64, _vp, _i64,
                                               _f32, _vp, _i64, _vp]),
    "sushi_cuda_fill_uniform": (_int, [_vp, _int, _vp, _i64, ctypes.c_uint64, _i64]),
    "sushi_cuda_sgemm_tf32_probe": (_int, [_vp, _int, _int, _int, _i64, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _int]),
}

_LIB = None


class SushiCudaError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"sushi_cuda error {code}: {message}")
        self.code = code


def load_library(path: Optional[str] = None):
    """dlopen libsushiblas_cuda.so and attach the prototypes.  Never builds, never falls back."""
    global _LIB
    if _LIB is not None and path is None:
        return _LIB
    path = path or os.environ.get("SUSHIBLAS_CUDA_LIB", LIB_PATH)
    if not os.path.exists(path):
        raise FileNotFoundError(
            f"{path} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
            "(the library has no CPU fallback)")
    lib = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError if the .so does not export it
        fn.restype = res
        fn.argtypes = args
    _LIB = lib
    return lib


def partition(total: int, nranks: int, rank: int):
    """Contiguous block of `total` owned by `rank` (pure host arithmetic; no GPU needed)."""
    lib = load_library()
    first, count = _i64(), _i64()
    rc = lib.sushi_cuda_partition(total, nranks, rank, ctypes.byref(first), ctypes.byref(count))
    if rc != 0:
        raise SushiCudaError(rc, lib.sushi_cuda_last_error(None).decode())
    return first.value, count.value


def batch_sharded_exchange(m: int, n: int, k: int, batch: int, nranks: int, variant: int = GEMM_AUTO, sm_count: int = 148,
                           gather: int = 2) -> int:
    """0 none, 1 NCCL all-gather, 2 fused peer stores (pure host arithmetic over rank-independent quantities)."""
    lib = load_library()
    out = _int()
    rc = lib.sushi_cuda_batch_sharded_exchange(m, n, k, batch, nranks, variant, sm_count, gather, ctypes.byref(out))
    if rc != 0:
        raise SushiCudaError(rc, lib.sushi_cuda_last_error(None).decode())
    return out.value


def row_sharded_exchange(m: int, n: int, k: int, nranks: int, variant: int = GEMM_AUTO, sm_count: int = 148,
                         gather: int = 2) -> int:
    """0 none, 1 NCCL slabs, 2 fused peer stores (pure host arithmetic over rank-independent quantities)."""
    lib = load_library()
    out = _int()
    rc = lib.sushi_cuda_row_sharded_exchange(m, n, k, nranks, variant, sm_count, gather, ctypes.byref(out))
    if rc != 0:
        raise SushiCudaError(rc, lib.sushi_cuda_last_error(None).decode())
    return out.value


def workspace_bytes(m: int, n: int, k: int, batch: int = 1) -> int:
    lib = load_library()
    out = _sz()
    rc = lib.sushi_cuda_gemm_workspace_bytes(m, n, k, batch, ctypes.byref(out))
    if rc != 0:
        raise SushiCudaError(rc, lib.sushi_cuda_last_error(None).decode())
    return out.value


STATIC_SCRATCH_BYTES = 32 << 20


def sgemm_static_scratch(stream_ptr, trans_a, trans_b, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc, status_dev=None):
    """Allocation-free GEMM on the current device (no context): operand planes live in the
    library's fixed scratch array.  See include/sushiblas_cuda.h for the limits."""
    lib = load_library()
    rc = lib.sushi_cuda_sgemm_static_scratch(stream_ptr, int(trans_a), int(trans_b), m, n, k, alpha, _addr(a), lda,
                                             _addr(b), ldb, beta, _addr(c), ldc, _addr(status_dev))
    if rc != 0:
        raise SushiCudaError(rc, lib.sushi_cuda_last_error(None).decode())


def _addr(x) -> Optional[int]:
    """Device/host address from an int, a torch tensor or a numpy array."""
    if x is None:
        return None
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        return x.data_ptr()
    if hasattr(x, "ctypes"):
        return x.ctypes.data
    raise TypeError(f"cannot take the address of {type(x)!r}")


class SushiCuda:
    """One context (``sushi_cuda_ctx``).  ``dev`` arguments index the device list given here."""

    def __init__(self, devices: Optional[Sequence[int]] = None):
        self.lib = load_library()
        self._ctx = _vp()
        if devices:
            arr = (_int * len(devices))(*devices)
            rc = self.lib.sushi_cuda_init(arr, len(devices), ctypes.byref(self._ctx))
        else:
            rc = self.lib.sushi_cuda_init(None, 0, ctypes.byref(self._ctx))
        if rc != 0:
            raise SushiCudaError(rc, self.lib.sushi_cuda_last_error(None).decode())

    # -- plumbing
    def _check(self, rc: int):
        if rc != 0:
            raise SushiCudaError(rc, self.lib.sushi_cuda_last_error(self._ctx).decode())

    def close(self):
        if self._ctx:
            self.lib.sushi_cuda_destroy(self._ctx)
            self._ctx = _vp()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def sync(self, dev: int = 0):
        self._check(self.lib.sushi_cuda_sync(self._ctx, dev))

    def set_stream(self, stream_ptr: Optional[int], dev: int = 0):
        self._check(self.lib.sushi_cuda_set_stream(self._ctx, dev, stream_ptr))

    def get_stream(self, dev: int = 0) -> int:
        out = _vp()
        self._check(self.lib.sushi_cuda_get_stream(self._ctx, dev, ctypes.byref(out)))
        return out.value or 0

    def selftest_bounded_wait(self, limit_ms: int, dev: int = 0):
        self._check(self.lib.sushi_cuda_selftest_bounded_wait(self._ctx, dev, limit_ms))

    def set_gemm_variant(self, variant: int):
        self._check(self.lib.sushi_cuda_set_gemm_variant(self._ctx, variant))

    def inject_failure(self, site: int, nth: int = 1):
        """Host-side fault injection: the nth next call reaching `site` (FAIL_* below) fails without touching the GPU."""
        self._check(self.lib.sushi_cuda_inject_failure(self._ctx, int(site), int(nth)))

    def copy_bytes(self):
        """(host->device, device->host) bytes moved through memcpy_h2d / memcpy_d2h so far."""
        up, down = ctypes.c_uint64(0), ctypes.c_uint64(0)
        self._check(self.lib.sushi_cuda_copy_bytes(self._ctx, ctypes.byref(up), ctypes.byref(down)))
        return int(up.value), int(down.value)

    def launch_count(self) -> int:
        out = _i64()
        self._check(self.lib.sushi_cuda_launch_count(self._ctx, ctypes.byref(out)))
        return out.value

    def kernel_timing_enable(self, enable: bool):
        self._check(self.lib.sushi_cuda_kernel_timing_enable(self._ctx, int(enable)))

    def kernel_timing_read(self, dev: int = 0):
        """(gemm_ms, gemm_launches, prepass_ms, prepass_launches) since the last read."""
        g, p = ctypes.c_double(), ctypes.c_double()
        gl, pl = _i64(), _i64()
        self._check(self.lib.sushi_cuda_kernel_timing_read(self._ctx, dev, ctypes.byref(g), ctypes.byref(gl),
                                                           ctypes.byref(p), ctypes.byref(pl)))
        return g.value, gl.value, p.value, pl.value

    # -- storage
    def malloc(self, nbytes: int, dev: int = 0) -> int:
        out = _vp()
        self._check(self.lib.sushi_cuda_malloc(self._ctx, dev, nbytes, ctypes.byref(out)))
        return out.value

    def free(self, ptr: int, dev: int = 0):
        self._check(self.lib.sushi_cuda_free(self._ctx, dev, ptr))

    def host_alloc(self, nbytes: int) -> int:
        out = _vp()
        self._check(self.lib.sushi_cuda_host_alloc(self._ctx, nbytes, ctypes.byref(out)))
        return out.value

    def host_free(self, ptr: int):
        self._check(self.lib.sushi_cuda_host_free(self._ctx, ptr))

    def memcpy_h2d(self, dst, src, nbytes: int, dev: int = 0):
        self._check(self.lib.sushi_cuda_memcpy_h2d(self._ctx, dev, _addr(dst), _addr(src), nbytes))

    def memcpy_d2h(self, dst, src, nbytes: int, dev: int = 0):
        self._check(self.lib.sushi_cuda_memcpy_d2h(self._ctx, dev, _addr(dst), _addr(src), nbytes))

    def memcpy_d2d(self, dst, src, nbytes: int, dev: int = 0):
        self._check(self.lib.sushi_cuda_memcpy_d2d(self._ctx, dev, _addr(dst), _addr(src), nbytes))

    def upload_fence(self, dev: int = 0):
        """Uploads issued with upload_ahead() from now on start after everything enqueued so far."""
        self._check(self.lib.sushi_cuda_upload_fence(self._ctx, dev))

    def upload_ahead(self, dst, src, nbytes: int, dev: int = 0):
        """Host-to-device copy on the upload stream; work enqueued afterwards waits for it, earlier work does not."""
        self._check(self.lib.sushi_cuda_upload_ahead(self._ctx, dev, _addr(dst), _addr(src), nbytes))

    def marker_create(self, dev: int = 0) -> int:
        m = _vp(None)
        self._check(self.lib.sushi_cuda_marker_create(self._ctx, dev, ctypes.byref(m)))
        return m.value

    def marker_record(self, marker: int, dev: int = 0):
        """The marker names the work enqueued on the device's stream so far."""
        self._check(self.lib.sushi_cuda_marker_record(self._ctx, dev, marker))

    def marker_destroy(self, marker: int):
        self._check(self.lib.sushi_cuda_marker_destroy(self._ctx, marker))

    def download_behind(self, dst, src, nbytes: int, marker: int, dev: int = 0):
        """Device-to-host copy that starts once the work before `marker` is done; sync() covers it."""
        self._check(self.lib.sushi_cuda_download_behind(self._ctx, dev, _addr(dst), _addr(src), nbytes, marker))

    def memset(self, dst, byte: int, nbytes: int, dev: int = 0):
        self._check(self.lib.sushi_cuda_memset(self._ctx, dev, _addr(dst), byte, nbytes))

    def reserve_workspace(self, nbytes: int, dev: int = 0):
        self._check(self.lib.sushi_cuda_reserve_workspace(self._ctx, dev, nbytes))

    # -- GEMM (device pointers)
    def sgemm(self, trans_a, trans_b, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc, dev: int = 0):
        self._check(self.lib.sushi_cuda_sgemm(self._ctx, dev, int(trans_a), int(trans_b), m, n, k, alpha,
                                              _addr(a), lda, _addr(b), ldb, beta, _addr(c), ldc))

    def sgemm_strided_batched(self, trans_a, trans_b, m, n, k, alpha, a, lda, stride_a, b, ldb, stride_b,
                              beta, c, ldc, stride_c, batch, dev: int = 0):
        self._check(self.lib.sushi_cuda_sgemm_strided_batched(
            self._ctx, dev, int(trans_a), int(trans_b), m, n, k, alpha, _addr(a), lda, stride_a,
            _addr(b), ldb, stride_b, beta, _addr(c), ldc, stride_c, batch))

    def sgemm_strided_batched_ex(self, trans_a, trans_b, m, n, k, alpha, a, lda, stride_a, b, ldb, stride_b,
                                 beta, c, ldc, stride_c, batch, epilogue: int, dev: int = 0):
        self._check(self.lib.sushi_cuda_sgemm_strided_batched_ex(
            self._ctx, dev, int(trans_a), int(trans_b), m, n, k, alpha, _addr(a), lda, stride_a,
            _addr(b), ldb, stride_b, beta, _addr(c), ldc, stride_c, batch, epilogue))

    def ssyrk(self, upper, trans, n, k, alpha, a, lda, beta, c, ldc, stride_a=0, stride_c=0, batch=1, dev: int = 0):
        self._check(self.lib.sushi_cuda_ssyrk_strided_batched(self._ctx, dev, int(upper), int(trans), n, k, alpha,
                                                              _addr(a), lda, stride_a, beta, _addr(c), ldc, stride_c, batch))

    def dgemm(self, trans_a, trans_b, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc, stride_a=0, stride_b=0, stride_c=0,
              batch=1, dev: int = 0):
        self._check(self.lib.sushi_cuda_dgemm_strided_batched(self._ctx, dev, int(trans_a), int(trans_b), m, n, k, alpha,
                                                              _addr(a), lda, stride_a, _addr(b), ldb, stride_b, beta,
                                                              _addr(c), ldc, stride_c, batch))

    def strsm(self, left, upper, trans, unit_diag, m, n, alpha, a, lda, b, ldb, stride_a=0, stride_b=0, batch=1,
              dev: int = 0):
        self._check(self.lib.sushi_cuda_strsm_strided_batched(self._ctx, dev, int(left), int(upper), int(trans),
                                                              int(unit_diag), m, n, alpha, _addr(a), lda, stride_a,
                                                              _addr(b), ldb, stride_b, batch))

    def sgemm_grouped(self, problems, dev: int = 0):
        """problems: iterable of dicts with the fields of sushi_cuda_gemm_desc (pointers may be tensors)."""
        problems = list(problems)
        arr = (GemmDesc * len(problems))()
        for d, q in zip(arr, problems):
            d.trans_a, d.trans_b = int(q.get("trans_a", 0)), int(q.get("trans_b", 0))
            d.m, d.n, d.k = q["m"], q["n"], q["k"]
            d.alpha, d.beta = q.get("alpha", 1.0), q.get("beta", 0.0)
            d.a, d.lda, d.stride_a = _addr(q["a"]), q["lda"], q.get("stride_a", 0)
            d.b, d.ldb, d.stride_b = _addr(q["b"]), q["ldb"], q.get("stride_b", 0)
            d.c, d.ldc, d.stride_c = _addr(q["c"]), q["ldc"], q.get("stride_c", 0)
            d.batch, d.epilogue, d.act_param = q.get("batch", 1), q.get("epilogue", 0), q.get("act_param", 0.0)
        self._check(self.lib.sushi_cuda_sgemm_grouped(self._ctx, dev, arr, len(problems)))

    def relu(self, x, count: int, dev: int = 0):
        self._check(self.lib.sushi_cuda_relu(self._ctx, dev, _addr(x), count))

    def activation(self, kind: int, x, count: int, param: float = 0.0, dev: int = 0):
        self._check(self.lib.sushi_cuda_activation(self._ctx, dev, int(kind), param, _addr(x), count))

    def activation_backward(self, kind: int, dy, saved, dx, count: int, param: float = 0.0, dev: int = 0):
        self._check(self.lib.sushi_cuda_activation_backward(self._ctx, dev, int(kind), param, _addr(dy), _addr(saved),
                                                            _addr(dx), count))

    def sgemm_strided_batched_act(self, trans_a, trans_b, m, n, k, alpha, a, lda, stride_a, b, ldb, stride_b,
                                  beta, c, ldc, stride_c, batch, activation: int, act_param: float = 0.0, dev: int = 0):
        self._check(self.lib.sushi_cuda_sgemm_strided_batched_act(
            self._ctx, dev, int(trans_a), int(trans_b), m, n, k, alpha, _addr(a), lda, stride_a,
            _addr(b), ldb, stride_b, beta, _addr(c), ldc, stride_c, batch, int(activation), act_param))

    # -- GEMM (host pointers, staged)
    def sgemm_strided_batched_host(self, trans_a, trans_b, m, n, k, alpha, a, lda, stride_a, b, ldb, stride_b,
                                   beta, c, ldc, stride_c, batch, dev: int = 0):
        self._check(self.lib.sushi_cuda_sgemm_strided_batched_host(
            self._ctx, dev, int(trans_a), int(trans_b), m, n, k, alpha, _addr(a), lda, stride_a,
            _addr(b), ldb, stride_b, beta, _addr(c), ldc, stride_c, batch))

    # -- multi-GPU
    def comm_unique_id(self) -> bytes:
        buf = ctypes.create_string_buffer(128)
        self._check(self.lib.sushi_cuda_comm_unique_id(buf))
        return buf.raw

    def comm_init_rank(self, unique_id: bytes, nranks: int, rank: int, dev: int = 0):
        buf = ctypes.create_string_buffer(unique_id, 128)
        self._check(self.lib.sushi_cuda_comm_init_rank(self._ctx, dev, buf, nranks, rank))

    def comm_destroy(self):
        self._check(self.lib.sushi_cuda_comm_destroy(self._ctx))

    def ipc_export(self, base_ptr, dev: int = 0) -> bytes:
        buf = ctypes.create_string_buffer(64)
        self._check(self.lib.sushi_cuda_ipc_export(self._ctx, dev, _addr(base_ptr), buf))
        return buf.raw

    def ipc_open(self, handle: bytes, dev: int = 0) -> int:
        out = _vp()
        self._check(self.lib.sushi_cuda_ipc_open(self._ctx, dev, ctypes.create_string_buffer(handle, 64), ctypes.byref(out)))
        return out.value

    def ipc_close(self, peer_ptr: int, dev: int = 0):
        self._check(self.lib.sushi_cuda_ipc_close(self._ctx, dev, peer_ptr))

    def comm_set_peer_buffers(self, buffers: Sequence[int], bytes_each: int, dev: int = 0):
        arr = (_vp * len(buffers))(*buffers)
        self._check(self.lib.sushi_cuda_comm_set_peer_buffers(self._ctx, dev, arr, len(buffers), bytes_each))

    def sgemm_row_sharded(self, trans_a, trans_b, m, n, k, alpha, a_local, lda, b, ldb, beta, c_full, ldc,
                          gather=True, dev: int = 0):
        self._check(self.lib.sushi_cuda_sgemm_row_sharded(
            self._ctx, dev, int(trans_a), int(trans_b), m, n, k, alpha, _addr(a_local), lda, _addr(b), ldb,
            beta, _addr(c_full), ldc, int(gather)))

    def sgemm_row_sharded_host(self, trans_a, trans_b, m, n, k, alpha, a_local_host, lda, b_host, ldb, beta, c_block_host, ldc,
                               a_local_dev, b_dev, c_block_dev, dev: int = 0):
        """Host buffers in and out (pinned for overlap); the three device buffers are caller-owned scratch."""
        self._check(self.lib.sushi_cuda_sgemm_row_sharded_host(
            self._ctx, dev, int(trans_a), int(trans_b), m, n, k, alpha, _addr(a_local_host), lda, _addr(b_host), ldb,
            beta, _addr(c_block_host), ldc, _addr(a_local_dev), _addr(b_dev), _addr(c_block_dev)))

    def sgemm_batch_sharded(self, trans_a, trans_b, m, n, k, alpha, a_local, lda, stride_a, b_local, ldb, stride_b,
                            beta, c_full, ldc, stride_c, batch, gather: bool = True, dev: int = 0):
        self._check(self.lib.sushi_cuda_sgemm_batch_sharded(
            self._ctx, dev, int(trans_a), int(trans_b), m, n, k, alpha, _addr(a_local), lda, stride_a,
            _addr(b_local), ldb, stride_b, beta, _addr(c_full), ldc, stride_c, batch, int(gather)))

    # -- harness helpers
    def sgemm_tf32_probe(self, trans_a, trans_b, m, n, k, a, lda, b, ldb, c, ldc, products: int, dev: int = 0):
        self._check(self.lib.sushi_cuda_sgemm_tf32_probe(self._ctx, dev, int(trans_a), int(trans_b), m, n, k, _addr(a), lda,
                                                         _addr(b), ldb, _addr(c), ldc, int(products)))

    def fill_uniform(self, dst, count: int, seed: int, first_index: int = 0, dev: int = 0):
        self._check(self.lib.sushi_cuda_fill_uniform(self._ctx, dev, _addr(dst), count, seed, first_index))
