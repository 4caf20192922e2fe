"""Gradient kernels (conv2dDerInput / DerFilter, depthwiseConv2DDerInput / DerFilter, max / avg
pool backprop, step, transpose).

CPU part: the oracle's restatement against gradient cases of the reference's own spec files,
transcribed as data with their line numbers.  GPU part: the CUDA kernels against the oracle,
bit for bit (they walk the same loop nests with float64 accumulators).
"""
import numpy as np
import pytest

import oracle
from gpu_util import tf  # noqa: F401


def _rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


# ---- the oracle against the reference's spec values ---------------------------------------------
def test_oracle_conv2d_gradients():
    # ops/conv2d_test.ts:398-423: x [3,3,1] = 1..9, filter ones [2,2,1,1], dy [3,1,2,0]
    x = np.arange(1, 10, dtype=np.float32).reshape(1, 3, 3, 1)
    w = np.ones((2, 2, 1, 1), np.float32)
    dy = np.array([3, 1, 2, 0], np.float32).reshape(1, 2, 2, 1)
    ci = oracle.compute_conv2d_info(x.shape, w.shape, 1, 1, "valid")
    assert oracle.conv2d_der_input(dy, w, ci).ravel().tolist() == [3, 4, 1, 5, 6, 1, 2, 2, 0]
    assert oracle.conv2d_der_filter(x, dy, ci).ravel().tolist() == [13, 19, 31, 37]
    # ops/conv2d_test.ts:425-452: the same image and dy twice in a batch of 2
    x2, dy2 = np.concatenate([x, x]), np.concatenate([dy, dy])
    ci2 = oracle.compute_conv2d_info(x2.shape, w.shape, 1, 1, "valid")
    assert oracle.conv2d_der_input(dy2, w, ci2).ravel().tolist() == [3, 4, 1, 5, 6, 1, 2, 2, 0] * 2
    assert oracle.conv2d_der_filter(x2, dy2, ci2).ravel().tolist() == [26, 38, 62, 74]


def test_oracle_depthwise_gradients():
    # ops/conv2d_depthwise_test.ts:580-650: two 2x2 RGB images, 2x2 filters, chMul 2, same, dy = 1
    images = np.array([[[[2, 3, 1], [3, 0, 2]], [[0, 4, 1], [3, 1, 3]]],
                       [[[2, 1, 0], [0, 3, 3]], [[4, 0, 1], [1, 4, 1]]]], np.float32)
    filt = np.array([[[[1, 1], [1, 1], [0, 0]], [[0, 1], [1, 1], [1, 1]]],
                     [[[1, 0], [1, 1], [0, 0]], [[0, 1], [1, 0], [0, 0]]]], np.float32)
    ci = oracle.compute_conv2d_info(images.shape, filt.shape, 1, 1, "same", None, True)
    dy = np.ones(ci.outShape, np.float32)
    want_dx = np.array([[[[2, 2, 0], [3, 4, 2]], [[3, 4, 0], [5, 7, 2]]]] * 2, np.float32)
    want_dw = np.array([[[[15, 15], [16, 16], [12, 12]], [[7, 7], [8, 8], [9, 9]]],
                        [[[8, 8], [9, 9], [6, 6]], [[4, 4], [5, 5], [4, 4]]]], np.float32)
    assert np.array_equal(oracle.depthwise_der_input(dy, filt, ci), want_dx)
    assert np.array_equal(oracle.depthwise_der_filter(images, dy, ci), want_dw)
    # :612-623 "wrt input, squared output": dy = 2 * y
    y = oracle.depthwise_conv2d(images, filt, ci)
    want = np.array([[[[20, 30, 0], [34, 34, 8]], [[10, 50, 0], [46, 44, 12]]],
                     [[[18, 24, 0], [8, 52, 12]], [[30, 40, 0], [22, 76, 4]]]], np.float32)
    assert np.array_equal(oracle.depthwise_der_input(2 * y, filt, ci), want)


@pytest.mark.parametrize("x,dy,f,s,dil,kind,want", [
    # ops/pool_test.ts:141-150
    (np.arange(1, 10), [1, 2, 3, 4], 2, 1, 1, "max", [0, 0, 0, 0, 1, 2, 0, 3, 4]),
    # :188-197 duplicate max value
    ([0, 0, 0, 0, 5, 0, 0, 0, 0], [1, 2, 3, 4], 2, 1, 1, "max", [0, 0, 0, 0, 10, 0, 0, 0, 0]),
    # :249-266, x [5,5,1] f 3 s 2
    (np.arange(25), [1, 2, 3, 4], 3, 2, 1, "max",
     [0] * 12 + [1, 0, 2] + [0] * 7 + [3, 0, 4]),
    # :268-286 duplicate max value
    ([0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 24, 13, 14, 15, 16, 17, 18, 19, 20, 21, 22, 23, 12],
     [1, 2, 3, 4], 3, 2, 1, "max", [0] * 12 + [10] + [0] * 12),
    # :468-482 avg
    ([1, 2, 3, 4, 5, 6, 7, 9, 8], [1, 2, 3, 4], 2, 1, 1, "avg",
     [0.25, 0.75, 0.5, 1, 2.5, 1.5, 0.75, 1.75, 1]),
    # :792-816 max with dilation 2, duplicate max values
    ([0, 0, 0, 0, 0, 0, 1, 1, 0, 0, 0, 1, 1] + [0] * 12, np.arange(1, 10), 2, 1, 2, "max",
     [0, 0, 0, 0, 0, 0, 5, 10, 0, 0, 0, 10, 20] + [0] * 12),
])
def test_oracle_pool_gradients(x, dy, f, s, dil, kind, want):
    x = np.asarray(x, np.float32)
    side = int(round(np.sqrt(x.size)))
    x = x.reshape(1, side, side, 1)
    ci = oracle.compute_pool2d_info(x.shape, [f, f], s, dil, "valid")
    dy = np.asarray(dy, np.float32).reshape(ci.outShape)
    np.testing.assert_allclose(oracle.pool_backprop(dy, x, ci, kind).ravel(), want, atol=1e-6)


def test_oracle_step():
    # backend_cpu.ts:1520-1534: NaN stays NaN, x > 0 -> 1, else alpha
    x = np.array([-2, 0, 3, np.nan, 1e-30], np.float32)
    out = oracle.step(x, 0.25)
    assert out[:3].tolist() == [0.25, 0.25, 1.0] and np.isnan(out[3]) and out[4] == 1.0


def test_oracle_gradients_match_finite_differences():
    """d/dx and d/dw of sum(dy * conv(x, w)) by central differences in float64."""
    rng = _rng(3)
    x = rng.normal(0, 1, (1, 5, 6, 2)).astype(np.float32)
    w = rng.normal(0, 1, (3, 3, 2, 3)).astype(np.float32)
    ci = oracle.compute_conv2d_info(x.shape, w.shape, 2, 1, "same")
    dy = rng.normal(0, 1, ci.outShape).astype(np.float32)

    def loss(xx, ww):
        return float((oracle.conv2d(xx, ww, ci).astype(np.float64) * dy).sum())
    dx, dw = oracle.conv2d_der_input(dy, w, ci), oracle.conv2d_der_filter(x, dy, ci)
    for idx in [(0, 0, 0, 0), (0, 2, 3, 1), (0, 4, 5, 0)]:
        xp, xm = x.copy(), x.copy()
        xp[idx] += 1e-2
        xm[idx] -= 1e-2
        assert abs((loss(xp, w) - loss(xm, w)) / 2e-2 - dx[idx]) < 2e-3
    for idx in [(0, 0, 0, 0), (1, 2, 1, 2), (2, 0, 0, 1)]:
        wp, wm = w.copy(), w.copy()
        wp[idx] += 1e-2
        wm[idx] -= 1e-2
        assert abs((loss(x, wp) - loss(x, wm)) / 2e-2 - dw[idx]) < 2e-3


# ---- the CUDA kernels against the oracle -----------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("b,h,w,cin,cout,f,s,pad", [
    (2, 9, 10, 3, 8, 3, 2, "same"), (1, 8, 8, 16, 24, 1, 1, "valid"), (3, 7, 5, 4, 6, 3, 1, "same"),
    (2, 12, 11, 5, 130, 2, 2, "valid"), (1, 6, 6, 2, 2, 5, 1, 2),
])
def test_conv2d_gradient_kernels(tf, b, h, w, cin, cout, f, s, pad):
    from tfjs_core_b200 import conv_util
    bk = tf.ENGINE.backend
    rng = _rng(b * 100 + h + cout)
    x = rng.normal(0, 1, (b, h, w, cin)).astype(np.float32)
    wt = rng.normal(0, 1, (f, f, cin, cout)).astype(np.float32)
    oci = oracle.compute_conv2d_info(x.shape, wt.shape, s, 1, pad)
    dci = conv_util.compute_conv2d_info(x.shape, wt.shape, s, 1, pad)
    dy = rng.normal(0, 1, oci.outShape).astype(np.float32)
    dx = bk.conv2dDerInput(tf.ops.tensor(dy), tf.ops.tensor(wt), dci)
    dw = bk.conv2dDerFilter(tf.ops.tensor(x), tf.ops.tensor(dy), dci)
    assert dx.shape == list(x.shape) and dw.shape == list(wt.shape)
    assert np.array_equal(dx.dataSync().reshape(x.shape), oracle.conv2d_der_input(dy, wt, oci))
    assert np.array_equal(dw.dataSync().reshape(wt.shape), oracle.conv2d_der_filter(x, dy, oci))


@pytest.mark.gpu
@pytest.mark.parametrize("b,h,w,c,mul,f,s,pad", [
    (2, 14, 14, 32, 1, 3, 1, "same"), (2, 15, 14, 8, 1, 3, 2, "same"), (1, 6, 7, 3, 2, 2, 1, "same"),
    (3, 9, 9, 160, 1, 3, 2, "valid"),
])
def test_depthwise_gradient_kernels(tf, b, h, w, c, mul, f, s, pad):
    from tfjs_core_b200 import conv_util
    bk = tf.ENGINE.backend
    rng = _rng(b + h * 7 + c)
    x = rng.normal(0, 1, (b, h, w, c)).astype(np.float32)
    wt = rng.normal(0, 1, (f, f, c, mul)).astype(np.float32)
    oci = oracle.compute_conv2d_info(x.shape, wt.shape, s, 1, pad, None, True)
    dci = conv_util.compute_conv2d_info(x.shape, wt.shape, s, 1, pad, None, True)
    dy = rng.normal(0, 1, oci.outShape).astype(np.float32)
    dx = bk.depthwiseConv2DDerInput(tf.ops.tensor(dy), tf.ops.tensor(wt), dci)
    dw = bk.depthwiseConv2DDerFilter(tf.ops.tensor(x), tf.ops.tensor(dy), dci)
    assert np.array_equal(dx.dataSync().reshape(x.shape), oracle.depthwise_der_input(dy, wt, oci))
    assert np.array_equal(dw.dataSync().reshape(wt.shape), oracle.depthwise_der_filter(x, dy, oci))


@pytest.mark.gpu
@pytest.mark.parametrize("shape,f,s,dil,pad", [((2, 7, 7, 1024), 7, 1, 1, "valid"), ((2, 9, 8, 6), (3, 2), 2, 1, "same"),
                                               ((1, 5, 5, 3), 2, 1, 2, "valid"), ((3, 12, 12, 20), 3, 2, 1, "same")])
def test_pool_backprop_kernels(tf, shape, f, s, dil, pad):
    from tfjs_core_b200 import conv_util
    bk = tf.ENGINE.backend
    rng = _rng(sum(shape))
    x = rng.integers(-3, 4, shape).astype(np.float32)   # duplicates: ties go to the first maximum
    fs = [f, f] if isinstance(f, int) else list(f)
    oci = oracle.compute_pool2d_info(shape, fs, s, dil, pad)
    dci = conv_util.compute_pool2d_info(list(shape), fs, s, dil, pad)
    dy = rng.normal(0, 1, oci.outShape).astype(np.float32)
    xt, dyt = tf.ops.tensor(x), tf.ops.tensor(dy)
    y = bk.maxPool(xt, dci)
    got_max = bk.maxPoolBackprop(dyt, xt, y, dci).dataSync().reshape(shape)
    got_avg = bk.avgPoolBackprop(dyt, xt, dci).dataSync().reshape(shape)
    assert np.array_equal(got_max, oracle.pool_backprop(dy, x, oci, "max"))
    assert np.array_equal(got_avg, oracle.pool_backprop(dy, x, oci, "avg"))


@pytest.mark.gpu
def test_step_and_transpose(tf):
    bk = tf.ENGINE.backend
    x = np.array([-2, 0, 3, np.nan, 1e-30, -0.0, 7], np.float32)
    got = bk.step(tf.ops.tensor(x), 0.25).dataSync()
    want = oracle.step(x, 0.25)
    assert np.array_equal(got, want, equal_nan=True)
    a = _rng(1).normal(0, 1, (2, 3, 4, 5)).astype(np.float32)
    for perm in ([3, 0, 1, 2], [0, 2, 1, 3], [1, 0, 3, 2], [0, 1, 2, 3]):
        t = bk.transpose(tf.ops.tensor(a), perm)
        assert t.shape == [a.shape[p] for p in perm]
        assert np.array_equal(t.dataSync().reshape(t.shape), a.transpose(perm))
