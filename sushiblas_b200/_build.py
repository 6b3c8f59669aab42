"""In-tree build of the sm_100a backend (libsushiblas_cuda.so) with nvcc.

The shared object is written next to this file so that it ships with a source snapshot;
nothing is installed into site-packages and no JIT cache is used.
"""
from __future__ import annotations

import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB_PATH = os.path.join(HERE, "libsushiblas_cuda.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def _sources():
    out = []
    for base, _, files in os.walk(CSRC):
        for f in files:
            if f.endswith((".cu", ".cuh", ".cpp", ".hpp", ".h")):
                out.append(os.path.join(base, f))
    out.append(os.path.join(ROOT, "include", "sushiblas_cuda.h"))
    return out


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(s) > t for s in _sources())


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile csrc/sushi_cuda.cu for sm_100a.  Needs nvcc only (no GPU)."""
    if not force and not is_stale():
        return LIB_PATH
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: cannot build libsushiblas_cuda.so")
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + [
        "-o", LIB_PATH, os.path.join(CSRC, "sushi_cuda.cu"), "-ldl"]
    subprocess.check_call(cmd, cwd=ROOT)
    return LIB_PATH


CPP_TESTS = ("test_host_logic", "test_engine_gemm", "test_engine_sharded", "test_io_npy")
CPP_BIN_DIR = os.path.join(ROOT, "tests", "cpp", "bin")


def build_cpp_tests(force: bool = False) -> dict:
    """Compile the C++ API tests (g++ -std=c++20) against the in-tree headers and library."""
    build_library()
    os.makedirs(CPP_BIN_DIR, exist_ok=True)
    gxx = shutil.which("g++") or "g++"
    out = {}
    headers = []
    for base, _, files in os.walk(os.path.join(ROOT, "include")):
        headers += [os.path.join(base, f) for f in files]
    for name in CPP_TESTS:
        src = os.path.join(ROOT, "tests", "cpp", name + ".cpp")
        exe = os.path.join(CPP_BIN_DIR, name)
        deps = [src, os.path.join(ROOT, "tests", "cpp", "check.hpp"), LIB_PATH] + headers
        if force or not os.path.exists(exe) or any(os.path.getmtime(d) > os.path.getmtime(exe) for d in deps):
            subprocess.check_call([gxx, "-std=c++20", "-O2", "-Wall", "-Wextra", "-I", os.path.join(ROOT, "include"),
                                   src, "-L", HERE, "-lsushiblas_cuda", "-Wl,-rpath,$ORIGIN/../../../sushiblas_b200",
                                   "-o", exe], cwd=ROOT)
        out[name] = exe
    return out
