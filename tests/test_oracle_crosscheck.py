"""The CPU oracle against an independent float64 implementation (tests/f64_forward.py) on the
shapes the reference's own known-answer vectors do not pin: depthwise with stride 2 and SAME
padding, 3x3 SAME convolution over many input channels, matMul with K beyond one 48-wide block
(backend_cpu.ts:83), and the whole MobileNetV1 forward.  The oracle follows the reference's loop
nests with float32 stores; the float64 code uses shifted-slice sums and BLAS.  They may differ by
float32 rounding of the accumulation (about K * 2^-24 of the tensor's scale), never by more: an
indexing, padding or ordering slip in either moves the result by whole terms of the sum.
"""
import numpy as np
import pytest

import f64_forward as f64
import oracle
from oracle import mobilenet as oracle_net


def _rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def _err(got, want):
    return float(np.abs(np.asarray(got, np.float64) - want).max() / np.abs(want).max())


@pytest.mark.parametrize("shape,stride", [((2, 112, 112, 32), 2), ((2, 14, 14, 64), 1), ((1, 15, 17, 8), 2),
                                          ((1, 7, 7, 16), 2), ((1, 28, 28, 256), 2)])
def test_depthwise_same_padding(shape, stride):
    rng = _rng(11)
    x = rng.uniform(0, 1, shape).astype(np.float32)
    w = rng.normal(0, 0.5, (3, 3, shape[3], 1)).astype(np.float32)
    ci = oracle.compute_conv2d_info(shape, w.shape, stride, 1, "same", None, True)
    got = oracle.depthwise_conv2d(x, w, ci)
    want = f64.depthwise_same(x, w, stride)
    assert got.shape == want.shape
    assert _err(got, want) <= 1e-6


@pytest.mark.parametrize("shape,cout,stride,dilation", [((2, 56, 56, 64), 64, 1, 1), ((1, 224, 224, 3), 32, 2, 1),
                                                        ((1, 19, 23, 12), 8, 2, 1), ((1, 20, 20, 16), 8, 1, 2)])
def test_conv3x3_same_padding(shape, cout, stride, dilation):
    rng = _rng(12)
    x = rng.uniform(0, 1, shape).astype(np.float32)
    w = rng.normal(0, np.sqrt(2.0 / (9 * shape[3])), (3, 3, shape[3], cout)).astype(np.float32)
    ci = oracle.compute_conv2d_info(shape, w.shape, stride, dilation, "same")
    got = oracle.conv2d(x, w, ci)
    want = f64.conv2d_same(x, w, stride, dilation)
    assert got.shape == want.shape
    # one float32 rounding per multiply-add over K = 9 * Cin terms
    assert _err(got, want) <= 1e-5


@pytest.mark.parametrize("m,k,n", [(65, 67, 66), (256, 1024, 1024), (50, 49, 7), (3, 200, 96)])
def test_matmul_beyond_one_block(m, k, n):
    rng = _rng(13)
    a = rng.uniform(-1, 1, (1, m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (1, k, n)).astype(np.float32)
    got = oracle.batch_matmul(a, b)[0]
    want = f64.matmul(a[0], b[0])
    assert _err(got, want) <= 2e-6


@pytest.mark.parametrize("quantized", [False, True])
def test_mobilenet_forward(quantized):
    """Whole network, two images: float weights (gain 1.5) and the same weights stored uint8."""
    from tfjs_core_b200 import mobilenet
    params = mobilenet.make_weights(3, gain=1.5)
    if quantized:
        params = f64.quantize_params(params)
    x = mobilenet.make_input(3, 2)
    got, got_p = oracle_net.forward(x, params)
    want, want_p = f64.forward(x, params)
    assert _err(got, want) <= 1e-5
    assert (got.argmax(1) == want.argmax(1)).all()
    assert np.abs(got_p - want_p).max() <= 1e-6


def test_dequantisation_matches_the_loader_formula():
    rng = _rng(14)
    q = rng.integers(0, 256, 4096, dtype=np.uint8)
    for scale, mn in ((0.1, -1.0), (0.0123456789, -1.5802469), (1e-3, -0.128)):
        want = (q.astype(np.float64) * scale + mn).astype(np.float32)
        assert np.array_equal(oracle.dequant_u8(q, scale, mn), want)
