"""GPU parity tests of the activation family (C ABI sushi_cuda_activation*, and as a GEMM epilogue)
against the float64 oracle.

Tolerance (floating point): |got - ref| <= 4 * 2^-24 * max(|ref|, |x|) + 1e-7 for the stand-alone
kernels (single-precision exp / tanh / log evaluated on values of that size); the reference's own
known answers are checked to 1e-4, the tolerance of the reference's tests.  A fused GEMM epilogue
must equal the GEMM followed by the stand-alone kernel bit for bit.
"""
import numpy as np
import pytest

from oracle import ref_activations as oa
from oracle import ref_gemm as og

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

KINDS = [(oa.RELU, 0.0), (oa.LEAKY_RELU, 0.01), (oa.LEAKY_RELU, 0.3), (oa.SIGMOID, 0.0), (oa.TANH, 0.0), (oa.ELU, 1.0),
         (oa.ELU, 0.5), (oa.SILU, 0.0), (oa.GELU, 0.0), (oa.SOFTPLUS, 0.0)]


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(np.asarray(x, dtype=np.float32))).cuda()


def within(got, ref, scale):
    bound = 4.0 * 2.0 ** -24 * np.maximum(np.abs(ref), np.abs(scale)) + 1e-7
    return float(np.max(np.abs(got.astype(np.float64) - ref) / bound))


def test_reference_known_answers(ctx):
    for kind, a, x, want in oa.REFERENCE_FORWARD:
        t = dev(x)
        ctx.activation(kind, t, t.numel(), a)
        ctx.sync()
        assert np.allclose(t.cpu().numpy(), want, rtol=0, atol=1e-4), oa.NAMES[kind]
    for kind, a, dy, s, want in oa.REFERENCE_BACKWARD:
        dx = torch.zeros(len(dy), device="cuda")
        ctx.activation_backward(kind, dev(dy), dev(s), dx, len(dy), a)
        ctx.sync()
        assert np.allclose(dx.cpu().numpy(), want, rtol=0, atol=1e-4), oa.NAMES[kind]


@pytest.mark.parametrize("kind,a", KINDS)
def test_forward_and_backward_match_the_oracle(ctx, kind, a):
    for count, offset in [(1, 0), (5, 0), (1023, 1), (1 << 20, 0), ((1 << 20) + 3, 2)]:      # unaligned starts and tails
        x = og.normal(900 + kind, count + offset, 2.0)[offset:]
        buf = dev(np.concatenate([np.zeros(offset, np.float32), x]))
        t = buf[offset:]
        ctx.activation(kind, t, count, a)
        ctx.sync()
        ref = oa.forward(kind, x.astype(np.float64), a)
        assert within(t.cpu().numpy(), ref, x) <= 1.0, (oa.NAMES[kind], count, offset)
        dy = og.uniform_pm1(950 + kind, count)
        saved = ref.astype(np.float32) if kind in (oa.SIGMOID, oa.TANH) else x
        dx = torch.empty(count, device="cuda")
        ctx.activation_backward(kind, dev(dy), dev(saved), dx, count, a)
        ctx.sync()
        refb = oa.backward(kind, dy.astype(np.float64), saved.astype(np.float64), a)
        assert within(dx.cpu().numpy(), refb, np.maximum(np.abs(dy), np.abs(saved))) <= 1.0, (oa.NAMES[kind], count, offset)
    # NaN handling of relu: x > 0 ? x : 0
    t = torch.tensor([float("nan"), -1.0, 2.0], device="cuda")
    ctx.activation(oa.RELU, t, 3)
    ctx.sync()
    assert t.cpu().tolist() == [0.0, 0.0, 2.0]


@pytest.mark.parametrize("kind,a", [(oa.LEAKY_RELU, 0.2), (oa.SIGMOID, 0.0), (oa.GELU, 0.0), (oa.ELU, 1.0), (oa.TANH, 0.0)])
def test_fused_gemm_epilogue_equals_gemm_then_activation(ctx, kind, a):
    """Every kernel family: FFMA tiles, skinny MMA kernel, tensor path interior / ragged tiles, cooperative
    split-K, many tiles; with beta and padded C."""
    for (m, n, k, ldc_pad, beta) in [(70, 50, 33, 3, 0.5), (4096, 16, 64, 0, 0.0), (512, 512, 2048, 0, 1.0), (300, 520, 300, 4, 0.5),
                                      (2304, 2304, 256, 0, 0.0)]:
        aa = og.uniform_pm1(40 + m, m * k) * 0.5
        bb = og.uniform_pm1(41 + n, k * n) * 0.5
        ldc = n + ldc_pad
        c0 = og.uniform_pm1(42, m * ldc)
        da, db = dev(aa), dev(bb)
        c1, c2 = dev(c0), dev(c0)
        ctx.sgemm_strided_batched_act(0, 0, m, n, k, 1.0, da, k, 0, db, n, 0, beta, c1, ldc, 0, 1, kind, a)
        ctx.sgemm(0, 0, m, n, k, 1.0, da, k, db, n, beta, c2, ldc)
        ctx.sync()
        plain = c2.cpu().numpy().reshape(m, ldc)
        view = c2.view(m, ldc)[:, :n].contiguous()
        ctx.activation(kind, view, m * n, a)
        ctx.sync()
        got = c1.cpu().numpy().reshape(m, ldc)
        assert np.array_equal(got[:, :n], view.cpu().numpy()), (oa.NAMES[kind], m, n, k)
        assert np.array_equal(got[:, n:], plain[:, n:]), "C padding was overwritten"


def test_invalid_arguments_are_rejected(ctx):
    from sushiblas_b200 import SushiCudaError
    x = torch.zeros(16, device="cuda")
    with pytest.raises(SushiCudaError):
        ctx.activation(9, x, 16)
    with pytest.raises(SushiCudaError):
        ctx.activation_backward(0, x, x, x, 16)
    with pytest.raises(SushiCudaError):
        ctx.activation(oa.RELU, None, 16)
    with pytest.raises(SushiCudaError):
        ctx.sgemm_strided_batched_act(0, 0, 4, 4, 4, 1.0, x, 4, 0, x, 4, 0, 0.0, x, 4, 0, 1, 12)
    ctx.activation(oa.RELU, x, 0)             # empty: nothing to do
