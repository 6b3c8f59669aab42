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
