import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


@pytest.fixture(scope="session")
def lib_path():
    """Path of the in-tree C-ABI library; built on demand (nvcc only, no GPU needed)."""
    from sushiblas_b200 import build_library
    return build_library()


@pytest.fixture(scope="session")
def ctx(lib_path):
    """A library context on cuda:0 running on torch's current stream."""
    import torch
    from sushiblas_b200 import SushiCuda
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.set_device(0)
    c = SushiCuda([0])
    # torch work and library kernels share one explicit stream (handle 0 of torch's default
    # stream would select the context's own stream instead)
    s = torch.cuda.Stream()
    torch.cuda.set_stream(s)
    c.set_stream(s.cuda_stream)
    yield c
    torch.cuda.synchronize()
    c.close()
