"""The C++ Engine/Tensor/Storage API (include/SushiBLAS, include/SushiRuntime) above the C ABI:
compiled with g++ and run as separate programs.  Host logic runs anywhere; the Engine tests --
the reference's own GEMM tests and caller shapes -- need the GPU."""
import os
import subprocess

import numpy as np
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


def test_cpp_host_logic(binaries, tmp_path):
    env = dict(os.environ, SUSHI_TEST_TMPDIR=str(tmp_path))
    p = subprocess.run([binaries["test_host_logic"]], capture_output=True, text=True, timeout=600, env=env)
    assert p.returncode == 0 and " 0 failed" in p.stdout, p.stdout + p.stderr
    assert "gemm_parameter_derivation" in p.stdout
    # the .npy files the C++ side wrote from host-resident tensors open in numpy with the right order and values
    a = np.load(tmp_path / "host_logic_rowmajor.npy")
    assert a.dtype == np.float32 and a.shape == (3, 5) and not np.isfortran(a)
    assert np.array_equal(a.ravel(), 0.25 * np.arange(15, dtype=np.float32) - 1.0)
    f = np.load(tmp_path / "host_logic_fortran.npy")
    assert np.isfortran(f) and np.array_equal(f.ravel(order="F"), np.arange(15, dtype=np.float32))


@pytest.mark.gpu
def test_cpp_engine_gemm(binaries):
    out = _run(binaries["test_engine_gemm"])
    for name in ("SimpleGEMM3x3", "SimpleGEMMColumnMajor", "DeviceStorageWithExplicitStaging"):
        assert f"[ OK ] {name}" in out
    print(out)


@pytest.mark.gpu
def test_cpp_io_npy_round_trips_with_numpy(binaries, tmp_path):
    """Files numpy writes load into DEVICE / SHARED tensors, the files written back are byte for
    byte numpy's, and a GEMM result saved from a DEVICE tensor reads back in numpy."""
    d = str(tmp_path)
    x = np.arange(60, dtype=np.float32).reshape(6, 10)
    np.save(os.path.join(d, "in_rowmajor.npy"), x)
    np.save(os.path.join(d, "in_fortran.npy"), np.asfortranarray(x))
    p = subprocess.run([binaries["test_io_npy"], d], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0 and " 0 failed" in p.stdout, p.stdout + p.stderr
    assert "skipped" not in p.stdout
    for name in ("rowmajor", "fortran"):
        with open(os.path.join(d, f"in_{name}.npy"), "rb") as f, open(os.path.join(d, f"echo_{name}.npy"), "rb") as g:
            assert f.read() == g.read(), name
    assert np.isfortran(np.load(os.path.join(d, "echo_fortran.npy")))
    a, b, c = (np.load(os.path.join(d, f"gemm_{n}.npy")) for n in "abc")
    assert a.shape == (5, 7) and b.shape == (7, 3) and c.dtype == np.float32
    assert np.array_equal(c, (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32))   # small integers: exact
    assert np.array_equal(np.load(os.path.join(d, "vec.npy")), np.arange(4, dtype=np.float32) * 0.5)
    assert np.array_equal(np.fromfile(os.path.join(d, "gemm_c.bin"), dtype=np.float32).reshape(5, 3), c)
