"""16-bit activation storage (setActivationStorage('float16')): the reference's 16-bit precision
class (KernelBackend.floatPrecision() == 16, backends/backend.ts:120-126; its tests then compare at
1e-1 instead of 1e-3, test_util.ts:23-39).  Activations are stored as IEEE half, the arithmetic
stays float32 / tf32 with float32 accumulation, so every kernel is checked against the CPU oracle
run on the SAME half-rounded inputs, at a tolerance that covers one rounding of the operands to
10 mantissa bits and one of the result to half: 2e-3 of the tensor's largest magnitude."""
import numpy as np
import pytest

import oracle
from gpu_util import rel_err, tf  # noqa: F401

pytestmark = pytest.mark.gpu

TOL = 2e-3


def _rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def _half(a):
    return np.asarray(a, np.float32).astype(np.float16).astype(np.float32)


@pytest.fixture()
def half_backend(tf):
    bk = tf.ENGINE.backend
    bk.setMathMode("tf32")
    bk.setActivationStorage("float16")
    yield bk
    bk.setActivationStorage("float32")
    bk.setMathMode("3xtf32")


def _half_tensor(bk, a):
    """A float32 tensor stored as half on the device (what a convolution produces in this mode)."""
    t = bk._out_activation(list(a.shape), "float16")
    bk.write(t.dataId, a)
    assert bk._rec(t.dataId)["dtype"] == "float16"
    return t


def test_storage_round_trip_and_precision_class(tf, half_backend):
    bk = half_backend
    assert bk.floatPrecision() == 16 and bk.epsilon() == 1e-4
    a = _rng(1).uniform(-6, 6, (3, 5, 7, 16)).astype(np.float32)
    t = _half_tensor(bk, a)
    assert np.array_equal(t.dataSync().reshape(a.shape), _half(a))       # rounded once, read back as float32
    assert np.array_equal(t.data().result().reshape(a.shape), _half(a))  # the asynchronous read too
    # a kernel without a half path sees the values through a float32 copy
    r = tf.ops.relu(t)
    assert np.array_equal(r.dataSync().reshape(a.shape), np.maximum(_half(a), 0))
    bk.setActivationStorage("float32")
    assert bk.floatPrecision() == 32


@pytest.mark.parametrize("m_shape,cin,cout", [((2, 14, 14), 512, 512), ((3, 7, 7), 1024, 1024), ((1, 28, 28), 256, 512),
                                              ((5, 9, 11), 40, 72), ((1, 1, 1), 1024, 1000), ((2, 14, 14), 64, 8)])
@pytest.mark.parametrize("out_storage", ["float16", "float32"])
def test_pointwise_conv_on_half_operands(tf, half_backend, m_shape, cin, cout, out_storage):
    """x stored as half -> the tensor cores' f16 path (half A and W tiles, float32 accumulation)."""
    from tfjs_core_b200 import conv_util
    bk = half_backend
    rng = _rng(cin + cout)
    x = rng.uniform(0, 6, m_shape + (cin,)).astype(np.float32)
    w = (rng.uniform(-1, 1, (1, 1, cin, cout)) / np.sqrt(cin)).astype(np.float32)
    b = rng.normal(0, 0.3, cout).astype(np.float32)
    ci = conv_util.compute_conv2d_info(x.shape, w.shape, 1, 1, "same")
    bk.profileBegin()
    out = bk.fusedConv2d(_half_tensor(bk, x), tf.ops.tensor(w), ci, tf.ops.tensor(b), "relu6", None, out_storage)
    names = [n for n, _ in bk.profileEnd()]
    assert any("F16" in n for n in names), names
    assert bk._rec(out.dataId)["dtype"] == out_storage
    oci = oracle.compute_conv2d_info(x.shape, w.shape, 1, 1, "same")
    want = oracle.unary("clip", oracle.binary("add", oracle.conv2d(_half(x), _half(w), oci), b), 0, 6)
    got = out.dataSync().reshape(want.shape)
    assert rel_err(got, want) <= TOL


@pytest.mark.parametrize("shape,stride", [((3, 14, 14, 512), 1), ((2, 7, 7, 1024), 1), ((2, 14, 14, 512), 2),
                                          ((2, 28, 28, 256), 2), ((1, 14, 14, 96), 1)])
def test_depthwise_image_kernel_on_half_storage(tf, half_backend, shape, stride):
    from tfjs_core_b200 import conv_util
    bk = half_backend
    rng = _rng(shape[3] + stride)
    x = rng.uniform(0, 6, shape).astype(np.float32)
    w = rng.normal(0, 0.4, (3, 3, shape[3], 1)).astype(np.float32)
    b = rng.normal(0, 0.3, shape[3]).astype(np.float32)
    ci = conv_util.compute_conv2d_info(shape, w.shape, stride, 1, "same", None, True)
    bk.profileBegin()
    out = bk.fusedDepthwiseConv2D(_half_tensor(bk, x), tf.ops.tensor(w), ci, tf.ops.tensor(b), "relu6")
    names = [n for n, _ in bk.profileEnd()]
    assert any("float16" in n for n in names), names
    assert bk._rec(out.dataId)["dtype"] == "float16"
    oci = oracle.compute_conv2d_info(shape, w.shape, stride, 1, "same", None, True)
    want = oracle.unary("clip", oracle.binary("add", oracle.depthwise_conv2d(_half(x), w, oci), b), 0, 6)
    got = out.dataSync().reshape(want.shape)
    # same float32 tap chain as the float32 kernel, then ONE rounding to half
    assert np.abs(got - want).max() <= 6.0 * 2.0 ** -11 + 1e-6


SEP_SHAPES = [
    # b, h, w, c, n, stride
    (2, 16, 16, 32, 64, 1),
    (2, 20, 23, 64, 96, 1),      # patches overhang right and bottom
    (1, 14, 14, 128, 128, 2),
    (3, 17, 19, 256, 256, 2),
    (2, 28, 28, 256, 256, 1),    # four half-size window stages instead of the in-place tile
    (4, 28, 28, 256, 512, 2),    # two kernels: whole-image depthwise 28 -> 14 + f16 GEMM
    (2, 14, 14, 512, 512, 1),    # two kernels
    (24, 56, 56, 128, 128, 1),   # many patches per CTA
]


@pytest.mark.parametrize("b,h,w,c,n,stride", SEP_SHAPES)
def test_separable_blocks_on_half_storage(tf, half_backend, b, h, w, c, n, stride):
    from tfjs_core_b200 import conv_util
    bk = half_backend
    rng = _rng(b * 1000 + c + n)
    x = rng.uniform(0, 6, (b, h, w, c)).astype(np.float32)
    wd = rng.normal(0, 0.3, (3, 3, c, 1)).astype(np.float32)
    wp = (rng.uniform(-1, 1, (1, 1, c, n)) / np.sqrt(c)).astype(np.float32)
    bd = rng.normal(0, 0.3, c).astype(np.float32)
    bp = rng.normal(0, 0.3, n).astype(np.float32)
    ci = conv_util.compute_conv2d_info(x.shape, wd.shape, stride, 1, "same", None, True)
    out = bk.fusedSeparableConv2d(_half_tensor(bk, x), tf.ops.tensor(wd), tf.ops.tensor(wp), ci, tf.ops.tensor(bd),
                                  "relu6", tf.ops.tensor(bp), "relu6")
    assert bk._rec(out.dataId)["dtype"] == "float16"
    got = out.dataSync()
    if b * h * w * c > 2_000_000:
        # too large for the oracle in a test: the float32-storage path on the same half-rounded input
        bk.setActivationStorage("float32")
        ref = bk.fusedSeparableConv2d(tf.ops.tensor(_half(x)), tf.ops.tensor(wd), tf.ops.tensor(wp), ci,
                                      tf.ops.tensor(bd), "relu6", tf.ops.tensor(bp), "relu6").dataSync()
        bk.setActivationStorage("float16")
        assert rel_err(got, ref) <= TOL
        return
    oci = oracle.compute_conv2d_info(x.shape, wd.shape, stride, 1, "same", None, True)
    mid = oracle.unary("clip", oracle.binary("add", oracle.depthwise_conv2d(_half(x), wd, oci), bd), 0, 6)
    oci2 = oracle.compute_conv2d_info(mid.shape, wp.shape, 1, 1, "valid")
    want = oracle.unary("clip", oracle.binary("add", oracle.conv2d(mid, wp, oci2), bp), 0, 6)
    assert rel_err(got.reshape(want.shape), want) <= TOL


def test_stem_writes_half(tf, half_backend):
    from tfjs_core_b200 import conv_util
    bk = half_backend
    rng = _rng(3)
    x = rng.uniform(-1, 1, (2, 224, 224, 3)).astype(np.float32)
    w = rng.normal(0, 0.3, (3, 3, 3, 32)).astype(np.float32)
    b = rng.normal(0, 0.1, 32).astype(np.float32)
    ci = conv_util.compute_conv2d_info(x.shape, w.shape, 2, 1, "same")
    out = bk.fusedConv2d(tf.ops.tensor(x), tf.ops.tensor(w), ci, tf.ops.tensor(b), "relu6")
    assert bk._rec(out.dataId)["dtype"] == "float16"
    oci = oracle.compute_conv2d_info(x.shape, w.shape, 2, 1, "same")
    want = oracle.unary("clip", oracle.binary("add", oracle.conv2d(x, w, oci), b), 0, 6)
    assert rel_err(out.dataSync().reshape(want.shape), want) <= TOL


def test_shapes_without_a_half_kernel_go_through_float32_copies(tf, half_backend):
    """A 3x3 convolution over 64 channels and a max pool have no half kernel: both still take a
    half-stored input (through a converted copy) and give the float32 path's result on the same
    values, rounded to half where the output is stored as half."""
    from tfjs_core_b200 import conv_util
    bk = half_backend
    rng = _rng(8)
    x = rng.uniform(0, 6, (2, 12, 12, 64)).astype(np.float32)
    w = rng.normal(0, 0.05, (3, 3, 64, 64)).astype(np.float32)
    ci = conv_util.compute_conv2d_info(x.shape, w.shape, 1, 1, "same")
    got = bk.fusedConv2d(_half_tensor(bk, x), tf.ops.tensor(w), ci, None, "relu").dataSync()
    bk.setActivationStorage("float32")
    ref = bk.fusedConv2d(tf.ops.tensor(_half(x)), tf.ops.tensor(w), ci, None, "relu").dataSync()
    bk.setActivationStorage("float16")
    assert np.array_equal(got, _half(ref))
    pooled = tf.ops.max_pool(_half_tensor(bk, x), [3, 3], 2, "same").dataSync()
    oci = oracle.compute_pool2d_info(x.shape, [3, 3], 2, 1, "same")
    assert np.array_equal(pooled.reshape(-1), oracle.pool(_half(x), oci, "max").reshape(-1))


@pytest.mark.parametrize("stored", ["float32", "uint8"])
def test_mobilenet_batch64_in_the_16_bit_precision_class(tf, half_backend, stored):
    """The whole network with half activations, batch 64, against the CPU oracle: logits within
    5e-3 of the largest (the float32-storage TF32 network measures 5.7e-4; storing 27 activation
    tensors as half adds their roundings), probabilities within the reference's own 16-bit
    tolerance of 1e-1 by a wide margin, identical argmax wherever the oracle's two best logits are
    further apart than twice that bound."""
    import threading
    from oracle import mobilenet as oracle_net
    from tfjs_core_b200 import mobilenet
    bk = half_backend
    params = mobilenet.make_weights(3, gain=1.5)
    if stored == "uint8":
        params = mobilenet.quantize_params(params)
    batch = 64
    x = mobilenet.make_input(3, batch)
    want = [None] * batch
    want_p = [None] * batch

    def work(first, step):
        for i in range(first, batch, step):
            want[i], want_p[i] = oracle_net.forward(x[i:i + 1], params)
    import os
    n_thr = min(os.cpu_count() or 1, batch)
    ts = [threading.Thread(target=work, args=(t, n_thr)) for t in range(n_thr)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    want, want_p = np.concatenate(want, 0), np.concatenate(want_p, 0)
    net = mobilenet.MobileNetV1(params, bk)
    try:
        for t in net.forward_separable(tf.ops.tensor(x[:2])):   # prepares the weights' device layouts
            t.dispose()
        before = bk.launchCount()
        logits, probs = net.forward_separable(tf.ops.tensor(x))
        got, got_p = logits.dataSync().reshape(want.shape), probs.dataSync().reshape(want.shape)
        assert bk._rec(logits.dataId)["dtype"] == "float32"
        launches = bk.launchCount() - before
    finally:
        net.dispose()
    err = rel_err(got, want)
    assert err <= 5e-3, err
    assert np.abs(got_p - want_p).max() <= 1e-3       # the reference's 16-bit tolerance is 1e-1
    s = np.sort(want, axis=1)
    decided = (s[:, -1] - s[:, -2]) / np.abs(want).max() > 1e-2
    assert (got.argmax(1) == want.argmax(1))[decided].all() and decided.sum() >= 10
    # and in fact everywhere but on near-ties
    assert np.mean(got.argmax(1) == want.argmax(1)) >= 0.9
    assert launches == 25, launches
    print(f"float16 activations, {stored} weights: logits err {err:.2e}, probabilities err "
          f"{np.abs(got_p - want_p).max():.2e}, argmax agreement {np.mean(got.argmax(1) == want.argmax(1)):.3f}")
