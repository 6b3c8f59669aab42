"""sushiblas_b200 -- B200 (sm_100a) backend for the SushiBLAS fp32 GEMM path.

The product is the C-ABI shared library ``libsushiblas_cuda.so`` (declared in
``include/sushiblas_cuda.h``) and the C++ Engine/Tensor headers above it.  This package
only builds that library in-tree and binds it with ctypes for the tests and the benchmark.
"""
from ._build import build_library, build_cpp_tests, LIB_PATH  # noqa: F401
from .capi import SushiCuda, SushiCudaError, load_library  # noqa: F401
