"""The C++ Engine/Tensor/Storage API (include/SushiBLAS, include/SushiRuntime) above the C ABI:
compiled with g++ and run as separate programs.  Host logic runs anywhere; the Engine tests --
the reference's own GEMM tests and caller shapes -- need the GPU."""
import subprocess

import pytest


@pytest.fixture(scope="module")
def binaries(lib_path):
    from sushiblas_b200 import build_cpp_tests
    return build_cpp_tests()


def _run(exe):
    p = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stdout + p.stderr
    assert " 0 failed" in p.stdout
    return p.stdout


def test_cpp_host_logic(binaries):
    out = _run(binaries["test_host_logic"])
    assert "gemm_parameter_derivation" in out


@pytest.mark.gpu
def test_cpp_engine_gemm(binaries):
    out = _run(binaries["test_engine_gemm"])
    for name in ("SimpleGEMM3x3", "SimpleGEMMColumnMajor", "DeviceStorageWithExplicitStaging"):
        assert f"[ OK ] {name}" in out
    print(out)
