"""Sharded entry points on real GPUs (needs at least 2; skipped otherwise): one process per
GPU, NCCL and fused peer-store exchange; every rank must hold identical bits, equal to the
single-GPU result up to fp32 summation order."""
import os
import subprocess
import sys

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_gemm_matches_single_gpu(world, lib_path):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    worker = os.path.join(os.path.dirname(__file__), "multi_gpu_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    p = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                        "--master-addr", "127.0.0.1", "--master-port", str(29500 + world), worker],
                       capture_output=True, text=True, timeout=600, env=env)
    assert p.returncode == 0, p.stdout[-4000:] + p.stderr[-4000:]
    assert "total failures=0" in p.stdout


def test_cpp_engine_row_sharded_two_processes(tmp_path, lib_path):
    """The C++ API's distributed RuntimeContext + gemm_row_sharded, two processes on two GPUs;
    the NCCL id travels through a file."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from sushiblas_b200 import build_cpp_tests
    exe = build_cpp_tests()["test_engine_sharded"]
    id_file = str(tmp_path / "nccl_id.bin")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([exe, str(r), "2", id_file], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
             for r in range(2)]
    outs = [p.communicate(timeout=300)[0] for p in procs]
    for p, out in zip(procs, outs):
        assert p.returncode == 0, out
        assert " 0 failed" in out
