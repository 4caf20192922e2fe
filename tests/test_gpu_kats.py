"""The reference's own known-answer vectors, run through the op layer on the cuda backend.
Tolerance is the reference's: absolute 1e-3 (tfjs-core/src/test_util.ts:23)."""
import numpy as np
import pytest

from gpu_util import tf  # noqa: F401
from kat_util import arr, expect_arrays_close, kat_id, load_kats

pytestmark = pytest.mark.gpu


def _t(tf, k, key):
    return tf.ops.tensor(arr(k[key], [int(v) for v in k[key + "_shape"]]))


@pytest.mark.parametrize("k", load_kats("fused_matmul") + load_kats("matmul"), ids=kat_id)
@pytest.mark.parametrize("tensor_cores", [1, 0])
def test_matmul(tf, k, tensor_cores):
    tf.ENGINE.backend.setOption("use_tensor_cores", tensor_cores)
    try:
        kw = {}
        if k.get("bias") is not None:
            kw["bias"] = _t(tf, k, "bias")
        if k.get("prelu") is not None:
            kw["preluActivationWeights"] = _t(tf, k, "prelu")
        out = tf.ops.fused_matmul(_t(tf, k, "a"), _t(tf, k, "b"), bool(k.get("transpose_a")),
                                  bool(k.get("transpose_b")), activation=k.get("activation", "linear"), **kw)
        expect_arrays_close(out.dataSync(), arr(k["expected"]))
    finally:
        tf.ENGINE.backend.setOption("use_tensor_cores", 1)


@pytest.mark.parametrize("k", load_kats("fused_conv2d") + load_kats("conv2d"), ids=kat_id)
def test_conv2d(tf, k):
    kw = {}
    if k.get("bias") is not None:
        kw["bias"] = _t(tf, k, "bias")
    if k.get("prelu") is not None:
        kw["preluActivationWeights"] = _t(tf, k, "prelu")
    out = tf.ops.fused_conv2d(_t(tf, k, "x"), _t(tf, k, "w"), k["strides"], k["pad"],
                              activation=k.get("activation", "linear"), **kw)
    expect_arrays_close(out.dataSync(), arr(k["expected"]))


@pytest.mark.parametrize("k", load_kats("depthwise"), ids=kat_id)
def test_depthwise(tf, k):
    out = tf.ops.depthwise_conv2d(_t(tf, k, "x"), _t(tf, k, "w"), k["strides"], k["pad"])
    expect_arrays_close(out.dataSync(), arr(k["expected"]))


@pytest.mark.parametrize(
    "k", load_kats("conv2d_dilation_equiv") + load_kats("depthwise_dilation_equiv"), ids=kat_id)
def test_dilation_equivalence(tf, k):
    op = tf.ops.depthwise_conv2d if k["kind"].startswith("depthwise") else tf.ops.conv2d
    got = op(_t(tf, k, "x"), _t(tf, k, "w"), k["strides"], k["pad"], "NHWC", k["dilation"])
    want = op(_t(tf, k, "x"), _t(tf, k, "w_dilated"), k["strides"], k["pad"])
    assert got.shape == want.shape
    expect_arrays_close(got.dataSync(), want.dataSync())


@pytest.mark.parametrize("k", load_kats("separable"), ids=kat_id)
def test_separable(tf, k):
    out = tf.ops.separable_conv2d(_t(tf, k, "x"), _t(tf, k, "dw"), _t(tf, k, "pw"), k["strides"], k["pad"])
    expect_arrays_close(out.dataSync(), arr(k["expected"]))


@pytest.mark.parametrize("k", load_kats("pool"), ids=kat_id)
def test_pool(tf, k):
    op = tf.ops.max_pool if k["pool"] == "max" else tf.ops.avg_pool
    out = op(_t(tf, k, "x"), k["filter"], k["strides"], k["pad"], k["rounding"])
    if "expected_shape" in k:
        assert out.shape == k["expected_shape"]
    else:
        expect_arrays_close(out.dataSync(), arr(k["expected"]))


@pytest.mark.parametrize("k", load_kats("softmax"), ids=kat_id)
@pytest.mark.parametrize("fused", [False, True])
def test_softmax(tf, k, fused):
    x = _t(tf, k, "x")
    out = tf.ops.fused_softmax(x) if fused else tf.ops.softmax(x)
    expect_arrays_close(out.dataSync(), arr(k["expected"]))


@pytest.mark.parametrize("k", load_kats("clip"), ids=kat_id)
def test_clip(tf, k):
    out = tf.ops.clip_by_value(tf.ops.tensor(arr(k["x"])), k["min"], k["max"])
    expect_arrays_close(out.dataSync(), arr(k["expected"]))


@pytest.mark.parametrize("k", load_kats("dequant_u8"), ids=kat_id)
def test_dequant(tf, k):
    t = tf.ENGINE.backend.registerQuantized([len(k["q"])], np.array(k["q"], np.uint8), k["scale"], k["min"])
    expect_arrays_close(t.dataSync(), arr(k["expected"]))
