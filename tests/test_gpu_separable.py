"""fusedSeparableConv2d: depthwise 3x3 (+bias, activation) fused into the pointwise GEMM.

The fused kernel performs the arithmetic of the two separate kernels operation for operation,
so in TF32 mode its output must equal theirs bit for bit; against the CPU oracle it is held to
the contraction tolerance.  Shapes cover whole and overhanging 8x16 patches, both strides, the
smallest and largest channel counts the kernel takes, and shapes it does not take (those run
the two kernels inside the same call).
"""
import numpy as np
import pytest

import oracle
from gpu_util import rel_err, tf  # noqa: F401

pytestmark = pytest.mark.gpu


def _rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def _case(tf, b, h, w, c, n, stride, seed, dw_act="relu6", pw_act="relu6", bias=True):
    from tfjs_core_b200 import conv_util
    bk = tf.ENGINE.backend
    rng = _rng(seed)
    x = rng.uniform(-1, 1, (b, h, w, c)).astype(np.float32)
    wd = rng.normal(0, 0.5, (3, 3, c, 1)).astype(np.float32)
    wp = rng.uniform(-1, 1, (1, 1, c, n)).astype(np.float32) / np.float32(np.sqrt(c))
    bd = rng.normal(0, 0.3, c).astype(np.float32) if bias else None
    bp = rng.normal(0, 0.3, n).astype(np.float32) if bias else None
    ci = conv_util.compute_conv2d_info(x.shape, wd.shape, stride, 1, "same", None, True)
    t = lambda a: None if a is None else tf.ops.tensor(a)  # noqa: E731
    xt, wdt, wpt, bdt, bpt = t(x), t(wd), t(wp), t(bd), t(bp)
    fused = bk.fusedSeparableConv2d(xt, wdt, wpt, ci, bdt, dw_act, bpt, pw_act)
    mid = bk.fusedDepthwiseConv2D(xt, wdt, ci, bdt, dw_act)
    ci2 = conv_util.compute_conv2d_info(mid.shape, wp.shape, 1, 1, "valid")
    two = bk.fusedConv2d(mid, wpt, ci2, bpt, pw_act)
    got, ref = fused.dataSync().reshape(two.shape), two.dataSync().reshape(two.shape)
    return x, wd, wp, bd, bp, ci, got, ref


def _oracle(x, wd, wp, bd, bp, stride, dw_act, pw_act):
    def act(y, a):
        if a == "relu6":
            return oracle.unary("clip", y, 0, 6)
        if a == "relu":
            return oracle.unary("relu", y)
        return y
    ci = oracle.compute_conv2d_info(x.shape, wd.shape, stride, 1, "same", None, True)
    mid = oracle.depthwise_conv2d(x, wd, ci)
    if bd is not None:
        mid = oracle.binary("add", mid, bd)
    mid = act(mid, dw_act)
    ci2 = oracle.compute_conv2d_info(mid.shape, wp.shape, 1, 1, "valid")
    y = oracle.conv2d(mid, wp, ci2)
    if bp is not None:
        y = oracle.binary("add", y, bp)
    return act(y, pw_act)


SHAPES = [
    # b, h, w, c, n, stride
    (2, 16, 16, 32, 64, 1),     # whole patches, one k-block
    (2, 20, 23, 64, 96, 1),     # patches overhang right and bottom; N not a multiple of 32
    (1, 14, 14, 128, 128, 2),   # stride 2, odd output size 7x7
    (3, 17, 19, 256, 256, 2),   # stride 2, overhang, largest C and N
    (2, 28, 28, 256, 256, 1),
    (1, 7, 7, 32, 8, 1),        # one partial patch, smallest N
    (5, 9, 40, 96, 200, 1),
]


@pytest.mark.parametrize("b,h,w,c,n,stride", SHAPES)
def test_fused_equals_the_two_kernels_and_matches_the_oracle(tf, b, h, w, c, n, stride):
    bk = tf.ENGINE.backend
    bk.setMathMode("tf32")
    bk.setOption("fuse_separable", 2)  # also the shapes the default leaves to the two kernels
    try:
        before = bk.launchCount()
        x, wd, wp, bd, bp, ci, got, ref = _case(tf, b, h, w, c, n, stride, seed=b * 1000 + c + n)
        assert np.array_equal(got, ref)
        want = _oracle(x, wd, wp, bd, bp, stride, "relu6", "relu6")
        assert rel_err(got, want) <= 1e-3
        # pack weights (first use) + fused + depthwise + pointwise = at most 5 launches: the fused
        # call was a single kernel
        assert bk.launchCount() - before <= 5
    finally:
        bk.setOption("fuse_separable", 1)
        bk.setMathMode("3xtf32")


@pytest.mark.parametrize("b,h,w,c,n,stride", [
    (16, 112, 112, 32, 64, 1),    # 1568 patches of one k-block: about 11 per CTA, every ring wraps
    (24, 56, 56, 128, 128, 1),    # 672 patches of four k-blocks, two depthwise groups
    (24, 56, 56, 128, 256, 2),    # 192 patches of four k-blocks, two half-windows each
    (40, 112, 112, 64, 128, 2),   # 1120 patches, three window stages
    (64, 28, 28, 256, 256, 1),    # 512 patches of eight k-blocks, A tiles built in place over their windows
])
def test_fused_many_patches_per_cta(tf, b, h, w, c, n, stride):
    """Sizes at which every CTA works through several patches, so that the stage rings, the A
    slots and the tensor-memory accumulators are reused many times: the fused kernel must still
    equal the two separate kernels bit for bit (the oracle would take minutes at these sizes; the
    two kernels are checked against it at the small sizes above)."""
    bk = tf.ENGINE.backend
    bk.setMathMode("tf32")
    bk.setOption("fuse_separable", 2)
    try:
        _, _, _, _, _, _, got, ref = _case(tf, b, h, w, c, n, stride, seed=b + c + n)
        assert np.array_equal(got, ref)
    finally:
        bk.setOption("fuse_separable", 1)
        bk.setMathMode("3xtf32")


@pytest.mark.parametrize("dw_act,pw_act,bias", [("linear", "linear", False), ("relu", "linear", True),
                                                 (("clip", -0.5, 0.75), "relu", True)])
def test_fused_epilogue_variants(tf, dw_act, pw_act, bias):
    bk = tf.ENGINE.backend
    bk.setMathMode("tf32")
    try:
        _, _, _, _, _, _, got, ref = _case(tf, 2, 24, 20, 64, 128, 1, seed=77, dw_act=dw_act, pw_act=pw_act,
                                           bias=bias)
        assert np.array_equal(got, ref)
    finally:
        bk.setMathMode("3xtf32")


@pytest.mark.parametrize("c,n,mode", [(512, 512, "tf32"), (64, 512, "tf32"), (40, 64, "tf32"), (64, 64, "3xtf32")])
def test_shapes_outside_the_fused_kernel_run_the_two_kernels(tf, c, n, mode):
    bk = tf.ENGINE.backend
    bk.setMathMode(mode)
    try:
        x, wd, wp, bd, bp, ci, got, ref = _case(tf, 1, 14, 14, c, n, 1, seed=c + n)
        assert np.array_equal(got, ref)
    finally:
        bk.setMathMode("3xtf32")


def test_option_off_forces_two_kernels_with_identical_output(tf):
    bk = tf.ENGINE.backend
    bk.setMathMode("tf32")
    try:
        _, _, _, _, _, _, fused, _ = _case(tf, 2, 16, 16, 32, 64, 1, seed=5)
        bk.setOption("fuse_separable", 0)
        _, _, _, _, _, _, unfused, _ = _case(tf, 2, 16, 16, 32, 64, 1, seed=5)
        assert np.array_equal(fused, unfused)
    finally:
        bk.setOption("fuse_separable", 1)
        bk.setMathMode("3xtf32")


def test_quantised_filters(tf):
    """uint8 depthwise and pointwise filters (config 5) through the fused kernel."""
    from tfjs_core_b200 import conv_util
    bk = tf.ENGINE.backend
    bk.setMathMode("tf32")
    try:
        rng = _rng(9)
        x = rng.uniform(-1, 1, (2, 16, 32, 64)).astype(np.float32)
        qd = rng.integers(0, 256, (3, 3, 64, 1), dtype=np.uint8)
        qp = rng.integers(0, 256, (1, 1, 64, 128), dtype=np.uint8)
        s, m = 0.004, -0.5
        wd, wp = oracle.dequant_u8(qd, s, m), oracle.dequant_u8(qp, s, m)
        ci = conv_util.compute_conv2d_info(x.shape, wd.shape, 1, 1, "same", None, True)
        xt = tf.ops.tensor(x)
        got = bk.fusedSeparableConv2d(xt, bk.registerQuantized(list(qd.shape), qd, s, m),
                                      bk.registerQuantized(list(qp.shape), qp, s, m), ci, None, "relu6", None,
                                      "relu6").dataSync()
        ref = bk.fusedSeparableConv2d(xt, tf.ops.tensor(wd), tf.ops.tensor(wp), ci, None, "relu6", None,
                                      "relu6").dataSync()
        assert np.array_equal(got, ref)
    finally:
        bk.setMathMode("3xtf32")


def test_mobilenet_with_fused_blocks_equals_the_layerwise_forward(tf):
    from tfjs_core_b200 import mobilenet
    bk = tf.ENGINE.backend
    bk.setMathMode("tf32")
    params = mobilenet.make_weights(4, quantized=True)
    net = mobilenet.MobileNetV1(params, bk)
    try:
        x = tf.ops.tensor(mobilenet.make_input(11, 3))
        a = [t.dataSync() for t in net.forward_fused(x)]
        before = bk.launchCount()
        b = [t.dataSync() for t in net.forward_separable(x)]
        launches = bk.launchCount() - before
        assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
        assert launches == 1 + 5 + 2 * 8 + 3, launches  # blocks 1-5 fused by default
    finally:
        net.dispose()
        bk.setMathMode("3xtf32")


# ---- the 3-channel 3x3 stem through the same kernel skeleton (window TMA + on-chip im2col) ----
@pytest.mark.parametrize("b,h,w,n,stride,pad", [
    (2, 224, 224, 32, 2, "same"),   # the network's stem: pad right / bottom only
    (1, 20, 24, 40, 1, "same"),     # pad left 1: the window starts 1 float past a 16-byte boundary
    (3, 17, 16, 8, 2, "valid"),
    (2, 9, 12, 256, 2, "same"),     # odd height: pad top 1, left 0... widest N
    (1, 33, 40, 64, 1, "valid"),
])
def test_rgb_stem_conv(tf, b, h, w, n, stride, pad):
    bk = tf.ENGINE.backend
    bk.setMathMode("tf32")
    try:
        rng = _rng(h * w + n)
        # small integers are exact in tf32: the result must equal the oracle's bit for bit
        x = rng.integers(-4, 5, (b, h, w, 3)).astype(np.float32)
        wt = rng.integers(-3, 4, (3, 3, 3, n)).astype(np.float32)
        bias = rng.integers(-5, 6, n).astype(np.float32)
        ci = oracle.compute_conv2d_info(x.shape, wt.shape, stride, 1, pad)
        want = oracle.fused_conv2d(x, wt, ci, bias=bias, activation="relu")
        before = bk.launchCount()
        got = tf.ops.fused_conv2d(tf.ops.tensor(x), tf.ops.tensor(wt), stride, pad, bias=tf.ops.tensor(bias),
                                  activation="relu")
        assert bk.launchCount() - before == 2  # weight repack + one kernel
        assert np.array_equal(got.dataSync().reshape(want.shape), want)
        # and real-valued data within the TF32 bound
        x = rng.uniform(-1, 1, (b, h, w, 3)).astype(np.float32)
        wt = rng.normal(0, 0.3, (3, 3, 3, n)).astype(np.float32)
        want = oracle.fused_conv2d(x, wt, ci, bias=bias, activation="relu")
        got = tf.ops.fused_conv2d(tf.ops.tensor(x), tf.ops.tensor(wt), stride, pad, bias=tf.ops.tensor(bias),
                                  activation="relu")
        assert rel_err(got.dataSync().reshape(want.shape), want) <= 1e-3
    finally:
        bk.setMathMode("3xtf32")


@pytest.mark.parametrize("b,h,w,n,stride,pad", [
    (2, 224, 224, 32, 2, "same"),   # the network's stem
    (1, 20, 24, 40, 1, "same"),     # pad left 1, N not a multiple of 32
    (3, 17, 16, 8, 2, "valid"),
    (2, 9, 12, 128, 2, "same"),     # widest N the 3xTF32 variant takes
    (2, 9, 12, 256, 2, "same"),     # wider: the gather kernel, same tolerance
])
def test_rgb_stem_conv_3xtf32(tf, b, h, w, n, stride, pad):
    """The stem in 3xTF32: the im2col threads write tf32 hi and lo tiles, the filter arrives as hi and
    lo planes, three tensor-core products per k-step.  Within 1e-5 of the oracle, also on values
    with large dynamic range and with a non-finite pixel (which must poison only the outputs whose
    window holds it)."""
    bk = tf.ENGINE.backend
    bk.setMathMode("3xtf32")
    rng = _rng(h * w + n + 7)
    x = (rng.uniform(-1, 1, (b, h, w, 3)) * 10.0 ** rng.integers(-3, 3, (b, h, w, 3))).astype(np.float32)
    wt = rng.normal(0, 0.3, (3, 3, 3, n)).astype(np.float32)
    bias = rng.normal(0, 0.3, n).astype(np.float32)
    ci = oracle.compute_conv2d_info(x.shape, wt.shape, stride, 1, pad)
    want = oracle.fused_conv2d(x, wt, ci, bias=bias, activation="relu")
    bk.profileBegin(8)
    got = tf.ops.fused_conv2d(tf.ops.tensor(x), tf.ops.tensor(wt), stride, pad, bias=tf.ops.tensor(bias),
                              activation="relu")
    out = got.dataSync().reshape(want.shape)
    names = [name for name, _ in bk.profileEnd()]
    assert any("window TMA, 3xTF32" in name for name in names) == (n <= 128), names
    assert rel_err(out, want) <= 1e-5
    x[0, 3, 4, 1] = np.inf
    want = oracle.fused_conv2d(x, wt, ci, bias=bias, activation="linear")
    out = tf.ops.fused_conv2d(tf.ops.tensor(x), tf.ops.tensor(wt), stride, pad, bias=tf.ops.tensor(bias)
                              ).dataSync().reshape(want.shape)
    assert np.array_equal(np.isfinite(out), np.isfinite(want))
    ok = np.isfinite(want)
    assert rel_err(out[ok], want[ok]) <= 1e-5


# ---- dense convolution fed entirely by TMA: one shifted-patch load per filter tap ----------------
@pytest.mark.parametrize("b,h,w,cin,n,fh,fw,dil,pad", [
    (8, 56, 56, 64, 64, 3, 3, 1, "same"),     # BASELINE config 2's shape
    (2, 20, 23, 32, 40, 3, 3, 1, "same"),     # overhanging patches, N not a multiple of 32
    (1, 9, 9, 64, 8, 5, 5, 2, "same"),        # dilation 2: taps reach 4 pixels out
    (3, 16, 16, 96, 256, 1, 3, 1, "valid"),   # asymmetric filter, widest N
    (2, 7, 30, 32, 32, 2, 2, 1, 1),           # numeric pad
])
def test_conv2d_shifted_patch_tma(tf, b, h, w, cin, n, fh, fw, dil, pad):
    bk = tf.ENGINE.backend
    bk.setMathMode("tf32")
    try:
        rng = _rng(h * 31 + cin + n)
        x = rng.integers(-3, 4, (b, h, w, cin)).astype(np.float32)
        wt = rng.integers(-2, 3, (fh, fw, cin, n)).astype(np.float32)
        bias = rng.integers(-5, 6, n).astype(np.float32)
        ci = oracle.compute_conv2d_info(x.shape, wt.shape, 1, dil, pad)
        want = oracle.fused_conv2d(x, wt, ci, bias=bias, activation="relu")
        bk.profileBegin(8)
        got = tf.ops.fused_conv2d(tf.ops.tensor(x), tf.ops.tensor(wt), 1, pad, dilations=dil,
                                  bias=tf.ops.tensor(bias), activation="relu")
        names = [name for name, _ in bk.profileEnd()]
        assert names[-1] == "conv2d_tcgen05 (shifted-patch TMA, TF32)", names
        # small integers are exact in tf32: bit-identical to the oracle whatever the summation order
        assert np.array_equal(got.dataSync().reshape(want.shape), want)
        x = rng.uniform(-1, 1, x.shape).astype(np.float32)
        wt = rng.normal(0, 0.2, wt.shape).astype(np.float32)
        want = oracle.fused_conv2d(x, wt, ci, bias=bias, activation="relu")
        got = tf.ops.fused_conv2d(tf.ops.tensor(x), tf.ops.tensor(wt), 1, pad, dilations=dil,
                                  bias=tf.ops.tensor(bias), activation="relu")
        assert rel_err(got.dataSync().reshape(want.shape), want) <= 1e-3
    finally:
        bk.setMathMode("3xtf32")


@pytest.mark.parametrize("b,h,w,cin,n,fh,fw,dil,pad", [
    (8, 56, 56, 64, 64, 3, 3, 1, "same"),     # BASELINE config 2's shape
    (2, 20, 23, 32, 40, 3, 3, 1, "same"),     # overhanging patches, N not a multiple of 32
    (1, 9, 9, 64, 8, 5, 5, 2, "same"),        # dilation 2
    (3, 16, 16, 96, 128, 1, 3, 1, "valid"),   # widest N the 3xTF32 variant takes
    (3, 16, 16, 96, 256, 1, 3, 1, "valid"),   # wider: the gather kernel, same tolerance
])
def test_conv2d_shifted_patch_tma_3xtf32(tf, b, h, w, cin, n, fh, fw, dil, pad):
    """The same convolution in 3xTF32: the helper warps split each TMA-loaded A tile into tf32 hi (in
    place) and lo (behind it), the filter arrives as hi and lo planes, three products per k-step.
    Within 1e-5 of the oracle on values spread over several orders of magnitude."""
    bk = tf.ENGINE.backend
    bk.setMathMode("3xtf32")
    rng = _rng(h * 31 + cin + n + 3)
    x = (rng.uniform(-1, 1, (b, h, w, cin)) * 10.0 ** rng.integers(-2, 2, (b, h, w, cin))).astype(np.float32)
    wt = rng.normal(0, 0.2, (fh, fw, cin, n)).astype(np.float32)
    bias = rng.normal(0, 0.3, n).astype(np.float32)
    ci = oracle.compute_conv2d_info(x.shape, wt.shape, 1, dil, pad)
    want = oracle.fused_conv2d(x, wt, ci, bias=bias, activation="relu")
    bk.profileBegin(8)
    got = tf.ops.fused_conv2d(tf.ops.tensor(x), tf.ops.tensor(wt), 1, pad, dilations=dil,
                              bias=tf.ops.tensor(bias), activation="relu")
    out = got.dataSync().reshape(want.shape)
    names = [name for name, _ in bk.profileEnd()]
    assert (names[-1] == "conv2d_tcgen05 (shifted-patch TMA, 3xTF32)") == (n <= 128), names
    assert rel_err(out, want) <= 1e-5


@pytest.mark.parametrize("c,h,stride", [(32, 16, 1), (64, 28, 2), (256, 28, 1)])
def test_non_finite_filter_taps_at_the_border(tf, c, h, stride):
    """The reference skips filter taps that fall outside the image (backend_cpu.ts:2002-2014);
    it does not multiply them by zero, so an inf or NaN tap must not leak into the border
    outputs.  The fused kernel gets its padding from zero-filled loads (0 * inf = NaN), so a
    separable call with such a filter must take the depthwise kernels, which skip those taps
    (strip kernel at 16 and 28 pixels, image kernel at 14 and 7): same NaN / inf pattern as the
    oracle, finite values within the contraction tolerance."""
    from tfjs_core_b200 import conv_util
    bk = tf.ENGINE.backend
    bk.setMathMode("tf32")
    bk.setOption("fuse_separable", 2)
    try:
        rng = _rng(c + h)
        n = 64
        x = rng.uniform(0.1, 1, (2, h, h, c)).astype(np.float32)
        wd = rng.normal(0, 0.5, (3, 3, c, 1)).astype(np.float32)
        # SAME padding at stride 2 on an even image pads the bottom and the right only, so the taps
        # that can fall outside at both strides are those of the last filter row / column
        wd[2, 2, 3, 0] = np.inf      # bottom-right tap: outside for the last row and the last column
        wd[2, 1, 5, 0] = np.nan      # bottom-centre tap: outside for the last row
        wp = np.zeros((1, 1, c, n), np.float32)
        wp[0, 0, np.arange(c), np.arange(c) % n] = 1.0   # output channel j sums channels j, j+64, ...
        ci = conv_util.compute_conv2d_info(x.shape, wd.shape, stride, 1, "same", None, True)
        names_before = bk.launchCount()
        bk.profileBegin()
        got = bk.fusedSeparableConv2d(tf.ops.tensor(x), tf.ops.tensor(wd), tf.ops.tensor(wp), ci, None, "linear",
                                      None, "linear").dataSync()
        names = [nm for nm, _ in bk.profileEnd()]
        assert not any("fused" in nm for nm in names), names
        assert bk.launchCount() > names_before
        want = _oracle(x, wd, wp, None, None, stride, "linear", "linear")
        got = got.reshape(want.shape)
        np.testing.assert_array_equal(np.isnan(got), np.isnan(want))
        np.testing.assert_array_equal(np.isinf(got), np.isinf(want))
        # a non-finite channel poisons every output channel of its pixel through the pointwise sum
        # (0 * inf), so the finite outputs are the pixels of the last row, where both taps are skipped
        ok = np.isfinite(want)
        assert ok[:, -1].all() and not ok[:, :-1].any()
        assert np.abs(got[ok] - want[ok]).max() <= 1e-3 * np.abs(want[ok]).max()
        # the same filter with the two bad taps made finite runs fused again
        wd[2, 2, 3, 0] = wd[2, 1, 5, 0] = 0.25
        bk.profileBegin()
        bk.fusedSeparableConv2d(tf.ops.tensor(x), tf.ops.tensor(wd), tf.ops.tensor(wp), ci, None, "linear", None,
                                "linear").dataSync()
        assert any("fused" in nm for nm, _ in bk.profileEnd())
    finally:
        bk.setOption("fuse_separable", 1)
        bk.setMathMode("3xtf32")


@pytest.mark.parametrize("b,h,w,n,stride,pad,native", [
    (2, 224, 224, 32, 2, "same", True),    # the network's stem on pixels
    (1, 32, 48, 40, 1, "same", True),      # pad left 1: the window starts 13 bytes past a 16-byte boundary
    (3, 17, 16, 8, 2, "valid", True),
    (1, 20, 24, 32, 2, "same", False),     # rows of 72 bytes cannot be a tensor-map stride: decoded float32 copy
])
@pytest.mark.parametrize("out_storage", ["float32", "float16"])
def test_rgb_stem_conv_on_pixel_bytes(tf, b, h, w, n, stride, pad, native, out_storage):
    """fromPixels-style input: the image is a quantised tensor (one byte per value, x = q / 127.5 - 1)
    and the stem decodes it on chip.  The decoded values are exactly those of the float32 image
    decodeWeights' formula gives, so the result must equal, bit for bit, the same kernel fed that
    float32 image; refilling the tensor with new bytes (the next batch) must be seen."""
    from tfjs_core_b200 import conv_util
    bk = tf.ENGINE.backend
    bk.setMathMode("tf32")
    try:
        rng = _rng(b * h + w + n)
        q = rng.integers(0, 256, (b, h, w, 3), dtype=np.uint8)
        scale, mn = 1.0 / 127.5, -1.0
        x = oracle.dequant_u8(q, scale, mn)
        wt = rng.normal(0, 0.3, (3, 3, 3, n)).astype(np.float32)
        bias = rng.normal(0, 0.1, n).astype(np.float32)
        ci = conv_util.compute_conv2d_info(x.shape, wt.shape, stride, 1, pad)
        wt_t, bias_t = tf.ops.tensor(wt), tf.ops.tensor(bias)
        xq = bk.registerQuantized(list(q.shape), q, scale, mn)
        bk.profileBegin()
        got = bk.fusedConv2d(xq, wt_t, ci, bias_t, "relu6", None, out_storage)
        names = [nm for nm, _ in bk.profileEnd()]
        assert any("uint8 in" in nm for nm in names) == native, names
        ref = bk.fusedConv2d(tf.ops.tensor(x), wt_t, ci, bias_t, "relu6", None, out_storage)
        assert np.array_equal(got.dataSync(), ref.dataSync())
        oci = oracle.compute_conv2d_info(x.shape, wt.shape, stride, 1, pad)
        want = oracle.unary("clip", oracle.binary("add", oracle.conv2d(x, wt, oci), bias), 0, 6)
        assert rel_err(got.dataSync().reshape(want.shape), want) <= (2e-3 if out_storage == "float16" else 1e-3)
        # the next batch of pixels into the same tensor
        q2 = rng.integers(0, 256, q.shape, dtype=np.uint8)
        bk.write(xq.dataId, q2)
        got2 = bk.fusedConv2d(xq, wt_t, ci, bias_t, "relu6", None, out_storage)
        ref2 = bk.fusedConv2d(tf.ops.tensor(oracle.dequant_u8(q2, scale, mn)), wt_t, ci, bias_t, "relu6", None,
                              out_storage)
        assert np.array_equal(got2.dataSync(), ref2.dataSync())
        assert not np.array_equal(got2.dataSync(), got.dataSync())
    finally:
        bk.setMathMode("3xtf32")
