"""CUDA kernels against the CPU oracle on seeded inputs (through the op layer and the C ABI).

Bars: memory-bound kernels (depthwise, direct conv, bias/clip/relu, pooling, softmax) follow
the reference's operation order and must agree to <= 2 ulp (double rounding of the oracle's
float64 temporaries is the only source of difference); contractions on tensor cores use a
different summation order, so they are held to the stated tolerances: max relative error
(floored at 1 % of the tensor's largest magnitude) <= 1e-5 for 3xTF32 and <= 1e-3 for TF32.
"""
import numpy as np
import pytest

import oracle
from gpu_util import rel_err, tf, ulp_diff  # noqa: F401

pytestmark = pytest.mark.gpu

TOL = {"3xtf32": 1e-5, "tf32": 1e-3}


def _rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


# ---- BASELINE config 1: fused matMul 256x1024x1024 + bias + relu, seed 0 ----------------------
@pytest.mark.parametrize("mode", ["3xtf32", "tf32"])
def test_config1_fused_matmul(tf, mode):
    rng = _rng(0)
    a = rng.uniform(-1, 1, (256, 1024)).astype(np.float32)
    lim = np.sqrt(6.0 / 2048)
    b = rng.uniform(-lim, lim, (1024, 1024)).astype(np.float32)
    bias = rng.normal(0, 0.01, 1024).astype(np.float32)
    want = oracle.fused_matmul(a[None], b[None], bias=bias, activation="relu")[0]
    bk = tf.ENGINE.backend
    bk.setMathMode(mode)
    try:
        got = tf.ops.fused_matmul(tf.ops.tensor(a), tf.ops.tensor(b), bias=tf.ops.tensor(bias),
                                  activation="relu").dataSync().reshape(want.shape)
    finally:
        bk.setMathMode("3xtf32")
    assert rel_err(got, want) <= TOL[mode]


# ---- BASELINE config 2: fused conv2d 8x56x56x64 * 3x3x64x64, same, bias, relu, seed 1 ---------
@pytest.mark.parametrize("mode", ["3xtf32", "tf32"])
def test_config2_fused_conv2d(tf, mode):
    rng = _rng(1)
    x = rng.uniform(0, 1, (8, 56, 56, 64)).astype(np.float32)
    w = rng.normal(0, np.sqrt(2.0 / (3 * 3 * 64)), (3, 3, 64, 64)).astype(np.float32)
    bias = rng.normal(0, 0.01, 64).astype(np.float32)
    ci = oracle.compute_conv2d_info(x.shape, w.shape, 1, 1, "same")
    want = oracle.fused_conv2d(x, w, ci, bias=bias, activation="relu")
    bk = tf.ENGINE.backend
    bk.setMathMode(mode)
    try:
        got = tf.ops.fused_conv2d(tf.ops.tensor(x), tf.ops.tensor(w), 1, "same", bias=tf.ops.tensor(bias),
                                  activation="relu").dataSync().reshape(want.shape)
    finally:
        bk.setMathMode("3xtf32")
    assert rel_err(got, want) <= TOL[mode]


# ---- BASELINE config 3: depthwise 8x112x112x32 * 3x3x32x1 s2 same, then bias and relu6, seed 2 -
@pytest.mark.parametrize("fused", [False, True])
def test_config3_depthwise_bias_relu6(tf, fused):
    rng = _rng(2)
    x = rng.uniform(0, 1, (8, 112, 112, 32)).astype(np.float32)
    w = rng.normal(0, np.sqrt(2.0 / 9), (3, 3, 32, 1)).astype(np.float32)
    bias = rng.normal(0, 0.01, 32).astype(np.float32)
    ci = oracle.compute_conv2d_info(x.shape, w.shape, 2, 1, "same", None, True)
    want = oracle.unary("clip", oracle.binary("add", oracle.depthwise_conv2d(x, w, ci), bias), 0, 6)
    xt, wt, bt = tf.ops.tensor(x), tf.ops.tensor(w), tf.ops.tensor(bias)
    if fused:
        from tfjs_core_b200 import conv_util
        dci = conv_util.compute_conv2d_info(x.shape, w.shape, 2, 1, "same", None, True)
        got = tf.ENGINE.backend.fusedDepthwiseConv2D(xt, wt, dci, bt, "relu6")
    else:
        got = tf.ops.clip_by_value(tf.ops.add(tf.ops.depthwise_conv2d(xt, wt, 2, "same"), bt), 0, 6)
    got = got.dataSync().reshape(want.shape)
    assert ulp_diff(got, want) <= 2


# ---- contraction shapes: tile edges, tails, transposes -----------------------------------------
@pytest.mark.parametrize("m,k,n", [(130, 68, 72), (1, 32, 8), (127, 4, 1000), (300, 96, 40),
                                   (128, 32, 64), (513, 260, 264), (64, 1024, 1000)])
@pytest.mark.parametrize("mode", ["3xtf32", "tf32"])
def test_matmul_shapes(tf, m, k, n, mode):
    rng = _rng(m * 7 + k * 3 + n)
    a = rng.uniform(-1, 1, (1, m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (1, k, n)).astype(np.float32)
    bias = rng.normal(0, 1, n).astype(np.float32)
    want = oracle.fused_matmul(a, b, bias=bias, activation=None)
    bk = tf.ENGINE.backend
    bk.setMathMode(mode)
    try:
        got = tf.ops.fused_matmul(tf.ops.tensor(a), tf.ops.tensor(b), bias=tf.ops.tensor(bias)).dataSync()
    finally:
        bk.setMathMode("3xtf32")
    assert rel_err(got.reshape(want.shape), want) <= TOL[mode]


@pytest.mark.parametrize("ta,tb", [(False, True), (True, False), (True, True)])
def test_matmul_transposes_tensor_core(tf, ta, tb):
    rng = _rng(11)
    m, k, n, batch = 96, 64, 48, 3
    a = rng.uniform(-1, 1, (batch, k, m) if ta else (batch, m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (batch, n, k) if tb else (batch, k, n)).astype(np.float32)
    want = oracle.batch_matmul(a, b, ta, tb)
    got = tf.ops.matmul(tf.ops.tensor(a), tf.ops.tensor(b), ta, tb).dataSync().reshape(want.shape)
    assert rel_err(got, want) <= 1e-5


def test_matmul_integer_exact(tf):
    """Small integers are exact in tf32, so the tensor-core result must equal the oracle's
    bit for bit whatever the summation order (the idea of tfjs-webgpu/src/matmul_test.ts:58)."""
    rng = _rng(5)
    a = rng.integers(0, 10, (1, 260, 132)).astype(np.float32)
    b = rng.integers(0, 10, (1, 132, 136)).astype(np.float32)
    want = oracle.batch_matmul(a, b)
    for mode in ("3xtf32", "tf32"):
        tf.ENGINE.backend.setMathMode(mode)
        got = tf.ops.matmul(tf.ops.tensor(a), tf.ops.tensor(b)).dataSync().reshape(want.shape)
        tf.ENGINE.backend.setMathMode("3xtf32")
        assert np.array_equal(got, want), mode


def test_matmul_zero_sized(tf):
    # ops/matmul_test.ts:621-642
    a = tf.ops.tensor(np.zeros((0, 3), np.float32), [0, 3])
    b = tf.ops.tensor(np.ones((3, 2), np.float32))
    out = tf.ops.matmul(a, b)
    assert out.shape == [0, 2] and out.dataSync().size == 0


def test_matmul_nan_propagates(tf):
    a = np.ones((1, 128, 32), np.float32)
    a[0, 5, 7] = np.nan
    b = np.ones((1, 32, 16), np.float32)
    got = tf.ops.matmul(tf.ops.tensor(a), tf.ops.tensor(b)).dataSync().reshape(128, 16)
    assert np.isnan(got[5]).all() and not np.isnan(np.delete(got, 5, 0)).any()


# ---- pointwise conv through the GEMM, with every epilogue -----------------------------------
@pytest.mark.parametrize("act", ["linear", "relu", "prelu", "relu6"])
def test_pointwise_conv_epilogues(tf, act):
    rng = _rng(21)
    x = rng.uniform(-1, 1, (2, 14, 14, 64)).astype(np.float32)
    w = rng.uniform(-0.3, 0.3, (1, 1, 64, 128)).astype(np.float32)
    bias = rng.normal(0, 0.5, 128).astype(np.float32)
    alpha = rng.uniform(0, 1, 128).astype(np.float32)
    ci = oracle.compute_conv2d_info(x.shape, w.shape, 1, 1, "same")
    y = oracle.binary("add", oracle.conv2d(x, w, ci), bias)
    if act == "relu":
        want = oracle.unary("relu", y)
    elif act == "prelu":
        want = oracle.binary("prelu", y, alpha)
    elif act == "relu6":
        want = oracle.unary("clip", y, 0, 6)
    else:
        want = y
    from tfjs_core_b200 import conv_util
    dci = conv_util.compute_conv2d_info(x.shape, w.shape, 1, 1, "same")
    got = tf.ENGINE.backend.fusedConv2d(tf.ops.tensor(x), tf.ops.tensor(w), dci, tf.ops.tensor(bias), act,
                                        tf.ops.tensor(alpha) if act == "prelu" else None)
    assert rel_err(got.dataSync().reshape(want.shape), want) <= 1e-5


# ---- memory-bound kernels: exactness --------------------------------------------------------
@pytest.mark.parametrize("shape,fshape,stride,pad,dil", [
    ((2, 9, 11, 8), (3, 3, 8, 1), 1, "same", 1),
    ((2, 10, 10, 12), (3, 3, 12, 1), 2, "same", 1),
    ((1, 7, 7, 1024), (3, 3, 1024, 1), 1, "same", 1),
    ((1, 13, 9, 5), (3, 3, 5, 2), 1, "valid", 1),
    ((1, 12, 12, 4), (2, 3, 4, 1), 1, "same", 2),
    ((3, 15, 15, 16), (3, 3, 16, 1), 2, "valid", 1),
])
def test_depthwise_shapes(tf, shape, fshape, stride, pad, dil):
    rng = _rng(sum(shape))
    x = rng.uniform(-1, 1, shape).astype(np.float32)
    w = rng.uniform(-1, 1, fshape).astype(np.float32)
    ci = oracle.compute_conv2d_info(shape, fshape, stride, dil, pad, None, True)
    want = oracle.depthwise_conv2d(x, w, ci)
    got = tf.ops.depthwise_conv2d(tf.ops.tensor(x), tf.ops.tensor(w), stride, pad, "NHWC", dil)
    assert got.shape == list(want.shape)
    assert ulp_diff(got.dataSync(), want) <= 2


@pytest.mark.parametrize("shape,stride,pad", [
    ((3, 14, 14, 64), 1, "same"),       # MobileNet's 14x14 layers, two channel groups short of a wave
    ((2, 14, 14, 96), 1, "same"),       # 32-channel groups
    ((5, 14, 14, 512), 2, "same"),      # 14 -> 7, pad bottom / right only
    ((2, 7, 7, 1024), 1, "same"),       # the last depthwise layer
    ((1, 16, 16, 32), 1, "valid"),      # no padding: the window starts inside the image
    ((1, 9, 9, 128), 1, "valid"),
    ((170, 7, 7, 128), 1, "same"),      # more items than CTAs: the stage ring wraps
])
@pytest.mark.parametrize("epilogue", [None, "bias_relu6", "bias_relu"])
def test_depthwise_image_window(tf, shape, stride, pad, epilogue):
    """3x3 depthwise on 14x14 / 7x7 outputs goes through the whole-image TMA kernel; results are
    those of MathBackendCPU.depthwiseConv2D bit for bit (up to the double rounding), borders included."""
    from tfjs_core_b200 import conv_util
    rng = _rng(sum(shape) + stride)
    C = shape[3]
    x = rng.uniform(-1, 1, shape).astype(np.float32)
    w = rng.uniform(-1, 1, (3, 3, C, 1)).astype(np.float32)
    bias = rng.normal(0, 0.5, C).astype(np.float32)
    ci = oracle.compute_conv2d_info(shape, w.shape, stride, 1, pad, None, True)
    want = oracle.depthwise_conv2d(x, w, ci)
    bk = tf.ENGINE.backend
    dci = conv_util.compute_conv2d_info(shape, w.shape, stride, 1, pad, None, True)
    xt, wt = tf.ops.tensor(x), tf.ops.tensor(w)
    names = []
    bk.profileBegin(4)
    if epilogue is None:
        got = bk.depthwiseConv2D(xt, wt, dci)
    else:
        want = oracle.binary("add", want, bias)
        want = oracle.unary("clip", want, 0, 6) if epilogue == "bias_relu6" else oracle.unary("relu", want)
        got = bk.fusedDepthwiseConv2D(xt, wt, dci, tf.ops.tensor(bias), epilogue[5:])
    names = [n for n, _ in bk.profileEnd()]
    assert any("image window" in n for n in names), names
    assert got.shape == list(want.shape)
    assert ulp_diff(got.dataSync(), want) <= 2


def test_depthwise_image_window_skips_taps_outside(tf):
    """A non-finite filter tap must not leak into the outputs whose tap lies outside the image:
    the reference skips those taps (backend_cpu.ts:2002-2014), it does not multiply them by zero."""
    rng = _rng(77)
    x = rng.uniform(-1, 1, (2, 14, 14, 32)).astype(np.float32)
    w = rng.uniform(-1, 1, (3, 3, 32, 1)).astype(np.float32)
    w[0, 0, 3, 0] = np.inf      # top-left tap: outside for the first row and the first column
    w[2, 1, 5, 0] = np.nan      # bottom-centre tap: outside for the last row
    ci = oracle.compute_conv2d_info(x.shape, w.shape, 1, 1, "same", None, True)
    want = oracle.depthwise_conv2d(x, w, ci)
    got = tf.ops.depthwise_conv2d(tf.ops.tensor(x), tf.ops.tensor(w), 1, "same").dataSync().reshape(want.shape)
    assert np.isfinite(want[:, 0, :, 3]).all() and np.isfinite(want[:, 13, :, 5]).all()
    np.testing.assert_array_equal(np.isnan(got), np.isnan(want))
    np.testing.assert_array_equal(np.isinf(got), np.isinf(want))
    ok = np.isfinite(want)
    assert ulp_diff(got[ok], want[ok]) <= 2


@pytest.mark.parametrize("shape,fshape,stride,pad,dil", [
    ((2, 16, 16, 3), (3, 3, 3, 32), 2, "same", 1),      # stem geometry
    ((1, 15, 17, 3), (3, 3, 3, 32), 2, "same", 1),      # odd input, conv_util_test.ts:82-99
    ((1, 9, 9, 5), (3, 3, 5, 7), 1, "valid", 1),
    ((2, 8, 8, 4), (1, 1, 4, 6), 2, "same", 1),
    ((1, 10, 10, 2), (2, 2, 2, 3), 1, "same", 2),
    ((1, 6, 6, 8), (3, 3, 8, 16), 1, 1, 1),
])
def test_direct_conv_shapes(tf, shape, fshape, stride, pad, dil):
    """The CUDA-core convolution kernels (tensor cores switched off) follow the reference's tap
    order and agree to the last bits; the same shapes through the default dispatch (implicit
    GEMM on the tensor cores where the shape allows) meet the 3xTF32 tolerance."""
    rng = _rng(sum(shape) + 1)
    x = rng.uniform(-1, 1, shape).astype(np.float32)
    w = rng.uniform(-1, 1, fshape).astype(np.float32)
    ci = oracle.compute_conv2d_info(shape, fshape, stride, dil, pad)
    want = oracle.conv2d(x, w, ci)
    bk = tf.ENGINE.backend
    bk.setOption("use_tensor_cores", 0)
    try:
        got = tf.ops.conv2d(tf.ops.tensor(x), tf.ops.tensor(w), stride, pad, "NHWC", dil)
    finally:
        bk.setOption("use_tensor_cores", 1)
    assert got.shape == list(want.shape)
    assert ulp_diff(got.dataSync(), want) <= 2
    got = tf.ops.conv2d(tf.ops.tensor(x), tf.ops.tensor(w), stride, pad, "NHWC", dil)
    assert rel_err(got.dataSync().reshape(want.shape), want) <= 1e-5


@pytest.mark.parametrize("shape,fshape,stride,pad,dil", [
    ((2, 20, 20, 8), (3, 3, 8, 16), 1, "same", 1),       # K = 72: k-blocks straddle taps
    ((1, 19, 23, 12), (3, 3, 12, 40), 2, "same", 1),     # odd sizes, stride 2, N tail
    ((2, 16, 16, 64), (3, 3, 64, 64), 1, "same", 1),     # config-2 channel counts
    ((1, 14, 14, 32), (5, 5, 32, 24), 1, "valid", 1),
    ((1, 17, 17, 4), (3, 3, 4, 8), 1, "same", 2),        # dilation 2
    ((3, 9, 9, 16), (1, 1, 16, 32), 2, "same", 1),       # strided 1x1 ("im2row" in the reference's specs)
    ((2, 33, 31, 3), (3, 3, 3, 32), 2, "same", 1),       # 3-channel gather, odd width: unaligned rows
    ((1, 32, 32, 3), (3, 3, 3, 16), 1, "same", 1),
    ((1, 12, 12, 3), (2, 3, 3, 8), 1, "valid", 1),
    ((70, 8, 8, 8), (3, 3, 8, 8), 1, "same", 1),         # many tiles, M tail
])
@pytest.mark.parametrize("mode", ["3xtf32", "tf32"])
def test_implicit_gemm_conv(tf, shape, fshape, stride, pad, dil, mode):
    rng = _rng(sum(shape) + sum(fshape))
    x = rng.uniform(-1, 1, shape).astype(np.float32)
    w = rng.uniform(-1, 1, fshape).astype(np.float32)
    bias = rng.normal(0, 1, fshape[3]).astype(np.float32)
    ci = oracle.compute_conv2d_info(shape, fshape, stride, dil, pad)
    want = oracle.fused_conv2d(x, w, ci, bias=bias, activation="relu")
    bk = tf.ENGINE.backend
    bk.setMathMode(mode)
    try:
        before = bk.launchCount()
        got = tf.ops.fused_conv2d(tf.ops.tensor(x), tf.ops.tensor(w), stride, pad, dilations=dil,
                                  bias=tf.ops.tensor(bias), activation="relu")
        t = bk.time(lambda: tf.ops.fused_conv2d(tf.ops.tensor(x), tf.ops.tensor(w), stride, pad, dilations=dil,
                                                bias=tf.ops.tensor(bias), activation="relu"))
    finally:
        bk.setMathMode("3xtf32")
    assert "launches" in t["getExtraProfileInfo"]() and bk.launchCount() > before
    assert got.shape == list(want.shape)
    assert rel_err(got.dataSync().reshape(want.shape), want) <= TOL[mode]


def test_elementwise_and_reductions(tf):
    rng = _rng(31)
    x = rng.normal(0, 3, (4, 7, 7, 36)).astype(np.float32)
    b = rng.normal(0, 1, 36).astype(np.float32)
    col = rng.normal(0, 1, (4, 1, 7, 1)).astype(np.float32)
    o = tf.ops
    xt = o.tensor(x)
    assert np.array_equal(o.add(xt, o.tensor(b)).dataSync().reshape(x.shape), oracle.binary("add", x, b))
    assert np.array_equal(o.add(o.tensor(b), xt).dataSync().reshape(x.shape), oracle.binary("add", b, x))
    for name, fn in (("add", o.add), ("sub", o.sub), ("mul", o.mul), ("div", o.div)):
        assert np.array_equal(fn(xt, o.tensor(col)).dataSync().reshape(x.shape), oracle.binary(name, x, col)), name
    assert np.array_equal(o.relu(xt).dataSync().reshape(x.shape), oracle.unary("relu", x))
    assert np.array_equal(o.clip_by_value(xt, 0, 6).dataSync().reshape(x.shape), oracle.unary("clip", x, 0, 6))
    assert ulp_diff(o.exp(xt).dataSync(), oracle.unary("exp", x)) <= 1
    xp = np.abs(x) + 0.1
    assert ulp_diff(o.log(o.tensor(xp)).dataSync(), oracle.unary("log", xp)) <= 1
    r = x.reshape(-1, 36)
    assert ulp_diff(o.sum(o.tensor(r), -1).dataSync(), oracle.sum_last(r)) <= 1
    assert np.array_equal(o.max(o.tensor(r), -1).dataSync(), oracle.max_last(r))
    assert np.array_equal(o.arg_max(o.tensor(r), -1).dataSync(), oracle.argmax_last(r))


def test_nan_rules(tf):
    o = tf.ops
    x = np.array([[np.nan, 1, 2], [1, np.nan, 3], [-np.inf, -np.inf, -np.inf]], np.float32)
    assert np.array_equal(o.max(o.tensor(x), -1).dataSync(), oracle.max_last(x), equal_nan=True)
    assert np.array_equal(o.arg_max(o.tensor(x), -1).dataSync(), oracle.argmax_last(x))
    v = np.array([np.nan, -1, 0, 7], np.float32)
    assert np.array_equal(o.relu(o.tensor(v)).dataSync(), oracle.unary("relu", v), equal_nan=True)
    assert np.array_equal(o.clip_by_value(o.tensor(v), 0, 6).dataSync(), oracle.unary("clip", v, 0, 6),
                          equal_nan=True)


def test_softmax_matches_chain_and_oracle(tf):
    rng = _rng(41)
    x = rng.normal(0, 4, (64, 1000)).astype(np.float32)
    want = oracle.softmax_last(x)
    chain = tf.ops.softmax(tf.ops.tensor(x)).dataSync().reshape(x.shape)
    fused = tf.ops.fused_softmax(tf.ops.tensor(x)).dataSync().reshape(x.shape)
    assert ulp_diff(fused, want) <= 2 and ulp_diff(chain, want) <= 2
    assert ulp_diff(fused, chain) <= 2


def test_pooling(tf):
    rng = _rng(51)
    x = rng.normal(0, 1, (3, 7, 7, 1024)).astype(np.float32)
    ci = oracle.compute_pool2d_info(x.shape, [7, 7], 1, 1, "valid")
    got = tf.ops.avg_pool(tf.ops.tensor(x), [7, 7], 1, "valid").dataSync().reshape(3, 1, 1, 1024)
    assert np.array_equal(got, oracle.pool(x, ci, "avg"))
    x2 = rng.normal(0, 1, (2, 9, 8, 6)).astype(np.float32)
    for kind, op in (("max", tf.ops.max_pool), ("avg", tf.ops.avg_pool)):
        ci = oracle.compute_pool2d_info(x2.shape, [3, 2], 2, 1, "same")
        got = op(tf.ops.tensor(x2), [3, 2], 2, "same")
        assert np.array_equal(got.dataSync().reshape(ci.outShape), oracle.pool(x2, ci, kind)), kind


@pytest.mark.parametrize("shape,fsize,stride,pad", [
    ((2, 13, 17, 8), [3, 3], 2, "same"),       # overlapping windows, ragged borders
    ((1, 112, 112, 64), [3, 3], 2, "same"),    # MobileNet-sized plane
    ((3, 10, 12, 16), [2, 2], 2, "valid"),     # four taps: the exact-reciprocal branch of the average
    ((2, 9, 9, 4), [3, 3], 1, "same"),         # border windows of 4 and 6 taps, interior of 9
    ((1, 8, 8, 12), [2, 3], 1, 1),             # numeric padding
])
def test_pooling_128_bit_kernel(tf, shape, fsize, stride, pad):
    """Channel counts that are multiples of four take the 128-bit pooling kernel: bit-identical to
    the oracle (float64 sum over the in-bounds taps in row-major order, divided by their count;
    max ignores NaN, avg propagates it, backend_cpu.ts:2299-2339)."""
    bk = tf.ENGINE.backend
    rng = _rng(shape[1] * shape[3])
    x = rng.normal(0, 1, shape).astype(np.float32)
    x[0, 1, 2, 1] = np.nan
    ci = oracle.compute_pool2d_info(x.shape, fsize, stride, 1, pad)
    for kind, op in (("max", tf.ops.max_pool), ("avg", tf.ops.avg_pool)):
        bk.profileBegin()
        got = op(tf.ops.tensor(x), fsize, stride, pad).dataSync().reshape(ci.outShape)
        assert any("128-bit" in n for n, _ in bk.profileEnd())
        want = oracle.pool(x, ci, kind)
        np.testing.assert_array_equal(np.isnan(got), np.isnan(want))
        ok = ~np.isnan(want)
        assert np.array_equal(got[ok], want[ok]), kind


# ---- quantised weights ----------------------------------------------------------------------
def test_quantized_weights_pointwise_and_depthwise(tf):
    rng = _rng(61)
    bk = tf.ENGINE.backend
    x = rng.uniform(-1, 1, (2, 14, 14, 64)).astype(np.float32)
    q = rng.integers(0, 256, (1, 1, 64, 96), dtype=np.uint8)
    scale, mn = 0.0123, -128 * 0.0123
    w = oracle.dequant_u8(q, scale, mn)
    ci = oracle.compute_conv2d_info(x.shape, w.shape, 1, 1, "same")
    want = oracle.conv2d(x, w, ci)
    wq = bk.registerQuantized(list(q.shape), q, scale, mn)
    assert np.array_equal(wq.dataSync().reshape(w.shape), w)
    got = tf.ops.conv2d(tf.ops.tensor(x), wq, 1, "same").dataSync().reshape(want.shape)
    assert rel_err(got, want) <= 1e-5
    qd = rng.integers(0, 256, (3, 3, 64, 1), dtype=np.uint8)
    wd = oracle.dequant_u8(qd, scale, mn)
    cid = oracle.compute_conv2d_info(x.shape, wd.shape, 1, 1, "same", None, True)
    wantd = oracle.depthwise_conv2d(x, wd, cid)
    gotd = tf.ops.depthwise_conv2d(tf.ops.tensor(x), bk.registerQuantized(list(qd.shape), qd, scale, mn), 1, "same")
    assert ulp_diff(gotd.dataSync(), wantd) <= 2


@pytest.mark.parametrize("math", ["3xtf32", "tf32"])
@pytest.mark.parametrize("m,k,n,transpose_b", [(256, 64, 96, False), (300, 100, 72, False),
                                               (1000, 515, 260, True), (129, 7, 8, False),
                                               (4096, 512, 512, False)])
@pytest.mark.parametrize("scale,mn", [(0.0071, -0.9), (0.016726349282588395, -1.4048376681967356)])
def test_quantized_matmul_dequantised_in_the_main_loop(tf, math, m, k, n, transpose_b, scale, mn):
    """uint8 weights stay bytes in device memory and are dequantised tile by tile inside the
    GEMM.  The result must equal, bit for bit, the same GEMM fed the dequantised float weights
    (both round the same float32 values to tf32), and match the oracle within the mode's bound.
    For the first (scale, min) pair a float32 fma reproduces the float64 dequantisation on all
    256 byte values and the kernel dequantises arithmetically; for the second it does not and
    the kernel uses its 256-entry table."""
    rng = _rng(1000 + m + k + n)
    bk = tf.ENGINE.backend
    bk.setMathMode(math)
    bk.setOption("dequant_in_gemm", 1)
    try:
        a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
        q = rng.integers(0, 256, (n, k) if transpose_b else (k, n), dtype=np.uint8)
        w = oracle.dequant_u8(q, scale, mn)
        wq = bk.registerQuantized(list(q.shape), q, scale, mn)
        bias = rng.normal(0, 1, n).astype(np.float32)
        got_q = tf.ops.fused_matmul(tf.ops.tensor(a), wq, False, transpose_b, bias=tf.ops.tensor(bias),
                                    activation="relu").dataSync().reshape(m, n)
        got_f = tf.ops.fused_matmul(tf.ops.tensor(a), tf.ops.tensor(w), False, transpose_b,
                                    bias=tf.ops.tensor(bias), activation="relu").dataSync().reshape(m, n)
        assert np.array_equal(got_q, got_f)
        want = oracle.fused_matmul(a[None], w[None], False, transpose_b, bias=bias, activation="relu")[0]
        assert rel_err(got_q, want) <= (1e-3 if math == "tf32" else 1e-5)
        # the same call with the option off takes the cached float planes: identical bits again
        bk.setOption("dequant_in_gemm", 0)
        got_c = tf.ops.fused_matmul(tf.ops.tensor(a), wq, False, transpose_b, bias=tf.ops.tensor(bias),
                                    activation="relu").dataSync().reshape(m, n)
        assert np.array_equal(got_c, got_q)
    finally:
        bk.setOption("dequant_in_gemm", 0)
        bk.setMathMode("3xtf32")


# ---- whole network ---------------------------------------------------------------------------
def test_mobilenet_end_to_end_float_weights(tf):
    """BASELINE config 4 at a small batch: logits within 1e-4 of the oracle's (relative to the
    largest logit), identical argmax, probabilities within 1e-5, for both forward paths."""
    from oracle import mobilenet as oracle_net
    from tfjs_core_b200 import mobilenet
    params = mobilenet.make_weights(3, gain=1.5)
    x = mobilenet.make_input(3, 2)
    want_logits, want_probs = oracle_net.forward(x, params)
    net = mobilenet.MobileNetV1(params, tf.ENGINE.backend)
    try:
        # the first pass also repacks every weight tensor for the tensor cores (cached afterwards)
        for t in net.forward_fused(tf.ops.tensor(x)):
            t.dispose()
        for fwd in (net.forward_fused, net.forward_reference_api):
            before = tf.ENGINE.backend.launchCount()
            logits, probs = fwd(tf.ops.tensor(x))
            launches = tf.ENGINE.backend.launchCount() - before
            got = logits.dataSync().reshape(want_logits.shape)
            assert rel_err(got, want_logits) <= 1e-4, fwd.__name__
            assert (got.argmax(1) == want_logits.argmax(1)).all()
            assert np.abs(probs.dataSync().reshape(want_probs.shape) - want_probs).max() <= 1e-5
            assert launches == (30 if fwd == net.forward_fused else 77), launches
    finally:
        net.dispose()


@pytest.mark.parametrize("quantized", [False, True, "in-loop"])
def test_mobilenet_every_layer_against_the_oracle(tf, quantized):
    """Each of the 28 weighted layers is run on the device with the ORACLE's activations as
    input and compared with the oracle's output of that layer.  (With the uint8 weights of
    config 5, |w| up to 2.56 and fan-in up to 1024, the random network amplifies a 1e-6
    perturbation by orders of magnitude per layer, so an end-to-end comparison would test the
    network's conditioning, not the kernels.)"""
    from oracle import mobilenet as oracle_net
    from tfjs_core_b200 import conv_util, mobilenet
    bk = tf.ENGINE.backend
    params = mobilenet.make_weights(4 if quantized else 3, quantized=bool(quantized), gain=1.5)
    x = mobilenet.make_input(3, 2)
    _, _, inter = oracle_net.forward(x, params, return_intermediates=True)
    net = mobilenet.MobileNetV1(params, bk)
    # "in-loop": the pointwise layers keep their weights uint8 and dequantise inside the GEMM
    bk.setOption("dequant_in_gemm", 1 if quantized == "in-loop" else 0)
    try:
        prev = x
        for name, kind, shape, stride in mobilenet.layer_specs():
            if name == "fc":
                break
            w, b = net.params[name]
            xin = tf.ops.tensor(prev)
            if kind == "dw":
                ci = conv_util.compute_conv2d_info(prev.shape, shape, stride, 1, "same", None, True)
                out = bk.fusedDepthwiseConv2D(xin, w, ci, b, "relu6")
            else:
                ci = conv_util.compute_conv2d_info(prev.shape, shape, stride, 1, "same")
                out = bk.fusedConv2d(xin, w, ci, b, "relu6")
            want = inter[name]
            got = out.dataSync().reshape(want.shape)
            if kind == "dw":
                assert ulp_diff(got, want) <= 2, name
            else:
                # error relative to the largest pre-activation value: relu6 clips outputs to
                # [0, 6] while the sums behind them reach the hundreds with these weights, and
                # the float32 rounding of those sums is what the two implementations differ by
                wf = oracle_net.float_weights(params)[name][0]
                oci = oracle.compute_conv2d_info(prev.shape, shape, stride, 1, "same")
                scale = np.abs(oracle.conv2d(prev, wf, oci)).max()
                err = np.abs(got.astype(np.float64) - want).max() / scale
                assert err <= 1e-5, (name, err)
            xin.dispose()
            out.dispose()
            prev = want
    finally:
        bk.setOption("dequant_in_gemm", 0)
        net.dispose()


def test_mobilenet_quantized_end_to_end_runs(tf):
    """Config 5's network end to end: finite probabilities that sum to one, and the class the
    oracle picks for each image."""
    from oracle import mobilenet as oracle_net
    from tfjs_core_b200 import mobilenet
    params = mobilenet.make_weights(4, quantized=True)
    x = mobilenet.make_input(4, 2)
    want_logits, _ = oracle_net.forward(x, params)
    net = mobilenet.MobileNetV1(params, tf.ENGINE.backend)
    try:
        logits, probs = net.forward_fused(tf.ops.tensor(x))
        p = probs.dataSync().reshape(2, 1000)
        assert np.isfinite(p).all() and np.allclose(p.sum(1), 1.0, atol=1e-4)
        # this network amplifies rounding differences layer by layer (see the per-layer test), so
        # end to end only a loose agreement is meaningful: logits within 10 % of the largest one,
        # and the device's class among the oracle's three best
        got = logits.dataSync().reshape(2, 1000)
        assert rel_err(got, want_logits) <= 0.1
        top3 = np.argsort(want_logits, axis=1)[:, -3:]
        assert all(got[i].argmax() in top3[i] for i in range(2))
    finally:
        net.dispose()


def test_memory_is_recycled(tf):
    """tf.memory()-style leak check (engine_test.ts:307-368) plus the allocator's promise that a
    steady-state loop does not call cudaMalloc."""
    rng = _rng(71)
    x = tf.ops.tensor(rng.uniform(-1, 1, (4, 28, 28, 32)).astype(np.float32))
    w = tf.ops.tensor(rng.uniform(-1, 1, (1, 1, 32, 64)).astype(np.float32))

    def step():
        return tf.ENGINE.tidy(lambda: tf.ops.clip_by_value(tf.ops.conv2d(x, w, 1, "same"), 0, 6).dataSync())
    step()
    m0 = tf.ENGINE.memory()
    for _ in range(5):
        step()
    m1 = tf.ENGINE.memory()
    assert m1["numTensors"] == m0["numTensors"] and m1["numBytes"] == m0["numBytes"]
    assert m1["numDeviceAllocs"] == m0["numDeviceAllocs"]
    assert m1["numBytesInGPU"] == m0["numBytesInGPU"]


def test_graph_capture_refuses_unprepared_weights(tf):
    """While a graph is captured, kernels are recorded and not run, so a weight layout prepared
    during capture would be cached without ever having been written.  The first use of a weight
    tensor inside a capture is therefore an error that says what to do, the context stays usable,
    and after one eager pass the same capture succeeds and replays to the eager result."""
    bk = tf.ENGINE.backend
    rng = _rng(91)
    x = rng.uniform(-1, 1, (1, 256, 64)).astype(np.float32)
    q = rng.integers(0, 256, (1, 64, 128), dtype=np.uint8)
    xt = tf.ops.tensor(x)
    wq = bk.registerQuantized(list(q.shape), q, 0.01, -1.28)
    bk.graphBegin()
    try:
        with pytest.raises(NotImplementedError, match="eagerly"):
            bk.fusedBatchMatMul(xt, wq)
    finally:
        g = bk.graphEnd()
        bk.graphDestroy(g)
    eager = bk.fusedBatchMatMul(xt, wq)           # prepares the tensor-core layout of wq
    want = eager.dataSync().copy()
    bk.graphBegin()
    out = bk.fusedBatchMatMul(xt, wq)
    g = bk.graphEnd()
    try:
        again = bk.fusedBatchMatMul(xt, wq).dataSync()   # an eager call before the first replay
        assert np.array_equal(again, want)
        bk.graphLaunch(g)
        assert np.array_equal(out.dataSync(), want)
    finally:
        bk.graphDestroy(g)
        for t in (eager, out, xt, wq):
            t.dispose()
