"""Pins the CPU oracle against the reference's own known-answer vectors
(tests/golden/reference_kats.json, extracted from tfjs-core's spec files)."""
import numpy as np
import pytest

import oracle
from kat_util import arr, expect_arrays_close, kat_id, load_kats


def _epilogue(y, k):
    if k.get("bias") is not None:
        y = oracle.binary("add", y, arr(k["bias"], k["bias_shape"]))
    act = k.get("activation")
    if act == "relu":
        y = oracle.unary("relu", y)
    elif act == "prelu":
        y = oracle.binary("prelu", y, arr(k["prelu"], k["prelu_shape"]))
    return y


@pytest.mark.parametrize("k", load_kats("fused_matmul"), ids=kat_id)
def test_fused_matmul(k):
    a = arr(k["a"], [int(v) for v in k["a_shape"]])
    b = arr(k["b"], [int(v) for v in k["b_shape"]])
    # ops/fused_ops.ts:109-112: operands are reshaped to rank 3 before the backend call
    a3 = a.reshape((-1,) + a.shape[-2:])
    b3 = b.reshape((-1,) + b.shape[-2:])
    y = oracle.batch_matmul(a3, b3, False, bool(k.get("transpose_b")))
    y = y.reshape(a.shape[:-2] + y.shape[-2:])
    expect_arrays_close(_epilogue(y, k), arr(k["expected"]))


@pytest.mark.parametrize("k", load_kats("matmul"), ids=kat_id)
def test_matmul(k):
    a = arr(k["a"], k["a_shape"])
    b = arr(k["b"], k["b_shape"])
    a3 = a.reshape((-1,) + a.shape[-2:])
    b3 = b.reshape((-1,) + b.shape[-2:])
    y = oracle.batch_matmul(a3, b3, k["transpose_a"], k["transpose_b"])
    expect_arrays_close(y, arr(k["expected"]))


def _conv(k, depthwise=False, w_key="w", dilation=None):
    x = arr(k["x"], k["x_shape"])
    w = arr(k[w_key], k[w_key + "_shape"])
    ci = oracle.compute_conv2d_info(x.shape, w.shape, k["strides"],
                                    dilation if dilation else 1, k["pad"], None, depthwise)
    return (oracle.depthwise_conv2d if depthwise else oracle.conv2d)(x, w, ci)


@pytest.mark.parametrize("k", load_kats("fused_conv2d") + load_kats("conv2d"), ids=kat_id)
def test_conv2d(k):
    expect_arrays_close(_epilogue(_conv(k), k), arr(k["expected"]))


@pytest.mark.parametrize("k", load_kats("depthwise"), ids=kat_id)
def test_depthwise(k):
    expect_arrays_close(_conv(k, depthwise=True), arr(k["expected"]))


@pytest.mark.parametrize(
    "k", load_kats("conv2d_dilation_equiv") + load_kats("depthwise_dilation_equiv"), ids=kat_id)
def test_dilation_equivalence(k):
    dw = k["kind"].startswith("depthwise")
    got = _conv(k, depthwise=dw, dilation=k["dilation"])
    want = _conv(k, depthwise=dw, w_key="w_dilated")
    assert got.shape == want.shape
    expect_arrays_close(got, want)


@pytest.mark.parametrize("k", load_kats("separable"), ids=kat_id)
def test_separable(k):
    # ops/conv.ts:643-647: separableConv2d = depthwiseConv2d then a 1x1 stride-1 valid conv2d
    x = arr(k["x"], k["x_shape"])
    dw = arr(k["dw"], k["dw_shape"])
    pw = arr(k["pw"], k["pw_shape"])
    ci = oracle.compute_conv2d_info(x.shape, dw.shape, k["strides"], 1, k["pad"], None, True)
    mid = oracle.depthwise_conv2d(x, dw, ci)
    ci2 = oracle.compute_conv2d_info(mid.shape, pw.shape, 1, 1, "valid")
    expect_arrays_close(oracle.conv2d(mid, pw, ci2), arr(k["expected"]))


@pytest.mark.parametrize("k", load_kats("pool"), ids=kat_id)
def test_pool(k):
    x = arr(k["x"], k["x_shape"])
    ci = oracle.compute_pool2d_info(x.shape, k["filter"], k["strides"], 1, k["pad"], k["rounding"])
    y = oracle.pool(x, ci, k["pool"])
    if "expected_shape" in k:
        assert list(y.shape) == k["expected_shape"]
    else:
        expect_arrays_close(y, arr(k["expected"]))


@pytest.mark.parametrize("k", load_kats("softmax"), ids=kat_id)
def test_softmax(k):
    expect_arrays_close(oracle.softmax_last(arr(k["x"], k["x_shape"])), arr(k["expected"]))


@pytest.mark.parametrize("k", load_kats("clip"), ids=kat_id)
def test_clip(k):
    expect_arrays_close(oracle.unary("clip", arr(k["x"]), k["min"], k["max"]), arr(k["expected"]))


@pytest.mark.parametrize("k", load_kats("dequant_u8"), ids=kat_id)
def test_dequant(k):
    got = oracle.dequant_u8(np.array(k["q"], np.uint8), k["scale"], k["min"])
    expect_arrays_close(got, arr(k["expected"]))
