"""The C-ABI library loads and exports every symbol include/sushiblas_cuda.h declares;
host-only entry points behave; compute entry points fail loudly without a device.  No GPU."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "sushiblas_cuda.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return re.findall(r"SUSHI_CUDA_API\s+[\w\s\*]+?\b(sushi_cuda_\w+)\s*\(", text)


def test_header_symbols_are_all_exported(lib_path):
    names = declared_symbols()
    assert len(names) >= 25
    lib = ctypes.CDLL(lib_path)
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_binding_covers_the_header(lib_path):
    from sushiblas_b200 import capi
    assert sorted(capi.SIGNATURES) == sorted(declared_symbols())
    capi.load_library()


def test_partition_rule(lib_path):
    from sushiblas_b200.capi import partition, SushiCudaError
    assert partition(32768, 8, 3) == (12288, 4096)
    assert partition(256, 8, 7) == (224, 32)
    # uneven: block = ceil(10/4) = 3 -> 3,3,3,1
    assert [partition(10, 4, r) for r in range(4)] == [(0, 3), (3, 3), (6, 3), (9, 1)]
    # more ranks than units: trailing ranks own nothing
    assert [partition(2, 4, r)[1] for r in range(4)] == [1, 1, 0, 0]
    for total in (0, 1, 7, 100, 65536):
        for nr in (1, 2, 3, 8):
            blocks = [partition(total, nr, r) for r in range(nr)]
            assert sum(c for _, c in blocks) == total
            pos = 0
            for first, count in blocks:
                assert first == pos or count == 0
                pos += count
    with pytest.raises(SushiCudaError):
        partition(10, 0, 0)
    with pytest.raises(SushiCudaError):
        partition(10, 2, 2)


def test_workspace_bytes(lib_path):
    from sushiblas_b200.capi import workspace_bytes
    # planes: 2 (hi/lo) * ceil(k/16) * rows_pad(256) * 16 * 4 bytes per operand
    assert workspace_bytes(4096, 4096, 4096) == 2 * (2 * 256 * 4096 * 16 * 4)
    assert workspace_bytes(1, 1, 1) == 2 * (2 * 1 * 256 * 16 * 4)
    assert workspace_bytes(512, 512, 512, 256) == 256 * 2 * (2 * 32 * 512 * 16 * 4)


def test_no_device_fails_loudly(lib_path):
    """Without a CUDA device there is no fallback: context creation reports an error."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    from sushiblas_b200 import SushiCuda, SushiCudaError
    with pytest.raises(SushiCudaError) as e:
        SushiCuda([0])
    assert e.value.code in (-2, -3)


def test_missing_library_is_an_error_not_a_fallback(tmp_path):
    from sushiblas_b200 import capi
    with pytest.raises(FileNotFoundError, match="no CPU fallback"):
        capi.load_library(str(tmp_path / "libsushiblas_cuda.so"))
    # the product package never imports the oracle
    import subprocess, sys
    code = ("import sys; import sushiblas_b200, sushiblas_b200.capi; "
            "bad = [m for m in sys.modules if m == 'oracle' or m.startswith('oracle.')]; sys.exit(1 if bad else 0)")
    assert subprocess.run([sys.executable, "-c", code], cwd=ROOT).returncode == 0


def test_header_is_plain_c(tmp_path):
    """The drop-in boundary must be consumable from C (cgo / JNI / ctypes generators read it as C):
    the header compiles as C99 on its own and its structs have the layout the Python binding assumes."""
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    src = tmp_path / "abi_check.c"
    src.write_text(
        '#include <stddef.h>\n#include <stdio.h>\n#include "sushiblas_cuda.h"\n'
        "int main(void) {\n"
        '  printf("%zu %zu %zu %zu\\n", sizeof(sushi_cuda_gemm_desc), offsetof(sushi_cuda_gemm_desc, alpha),\n'
        "         offsetof(sushi_cuda_gemm_desc, epilogue), offsetof(sushi_cuda_gemm_desc, act_param));\n"
        "  return (SUSHI_ACT_SOFTPLUS == 8 && (int)SUSHI_EPILOGUE_RELU == (int)SUSHI_ACT_RELU) ? 0 : 1;\n}\n")
    exe = tmp_path / "abi_check"
    subprocess.check_call([gcc, "-std=c99", "-Wall", "-Werror", "-pedantic", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)])
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0
    import ctypes
    from sushiblas_b200.capi import GemmDesc
    size, off_alpha, off_epi, off_param = (int(v) for v in out.stdout.split())
    assert size == ctypes.sizeof(GemmDesc)
    assert off_alpha == GemmDesc.alpha.offset and off_epi == GemmDesc.epilogue.offset and off_param == GemmDesc.act_param.offset


def test_row_sharded_exchange_is_decided_without_the_rank(lib_path):
    """The exchange a sharded GEMM runs (and so the collectives each rank issues) is a function of the
    shared problem only: uneven partitions -- a short last block, empty trailing ranks -- cannot send
    ranks down different paths."""
    from sushiblas_b200.capi import row_sharded_exchange, partition, GEMM_AUTO, GEMM_SIMT, GEMM_TC3X
    # headline shape: fused at every rank count
    for g in (2, 4, 8):
        assert row_sharded_exchange(32768, 32768, 32768, g) == 2
    assert row_sharded_exchange(32768, 32768, 32768, 1) == 0
    assert row_sharded_exchange(32768, 32768, 32768, 8, gather=0) == 0
    assert row_sharded_exchange(32768, 32768, 32768, 8, gather=1) == 1
    # AUTO, m = 1017 on 8 ranks: blocks of 128 and a last block of 121 rows, too small for the tensor
    # path -- every rank (also those with 128 rows) must take the NCCL exchange
    assert [partition(1017, 8, r)[1] for r in range(8)] == [128] * 7 + [121]
    assert row_sharded_exchange(1017, 512, 512, 8, GEMM_AUTO) == 1
    # forced tensor path, fewer rows than ranks: trailing ranks are empty, the others fused
    assert [partition(5, 8, r)[1] for r in range(8)] == [1, 1, 1, 1, 1, 0, 0, 0]
    assert row_sharded_exchange(5, 512, 512, 8, GEMM_TC3X) == 2
    assert row_sharded_exchange(5, 512, 512, 8, GEMM_SIMT) == 1
    # K below 4 never runs on the tensor path; n must allow 128-bit peer stores
    assert row_sharded_exchange(4096, 512, 3, 2, GEMM_TC3X) == 1
    assert row_sharded_exchange(4096, 510, 512, 2, GEMM_TC3X) == 1
    assert row_sharded_exchange(0, 512, 512, 2, GEMM_TC3X) == 1


def test_batch_sharded_exchange_is_decided_without_the_rank(lib_path):
    """Same rule for the batch-sharded form: the fused exchange is chosen from the largest and the last batch
    block, so ranks with fewer (or no) entries issue the same collectives as the others."""
    from sushiblas_b200.capi import batch_sharded_exchange, partition, GEMM_AUTO, GEMM_SIMT, GEMM_TC3X
    for g in (2, 4, 8):
        assert batch_sharded_exchange(512, 512, 512, 256, g) == 2           # the batched configuration
    assert batch_sharded_exchange(512, 512, 512, 256, 1) == 0
    assert batch_sharded_exchange(512, 512, 512, 256, 8, gather=0) == 0
    assert batch_sharded_exchange(512, 512, 512, 256, 8, gather=1) == 1
    # fewer entries than ranks under the forced tensor path: trailing ranks own nothing, everybody fused
    assert [partition(3, 4, r)[1] for r in range(4)] == [1, 1, 1, 0]
    assert batch_sharded_exchange(512, 256, 128, 3, 4, GEMM_TC3X) == 2
    assert batch_sharded_exchange(512, 256, 128, 3, 4, GEMM_SIMT) == 1
    # tiny entries under AUTO go to the FFMA kernel on every rank: no peer stores anywhere
    assert batch_sharded_exchange(32, 32, 32, 5, 2, GEMM_AUTO) == 1
    assert batch_sharded_exchange(512, 510, 512, 8, 2, GEMM_TC3X) == 1      # n must allow 128-bit peer stores
    assert batch_sharded_exchange(512, 512, 3, 8, 2, GEMM_TC3X) == 1        # K < 4 never runs on the tensor path
