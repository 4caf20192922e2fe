"""TEST INFRASTRUCTURE ONLY: MobileNetV1 forward on the CPU oracle.

Runs the network the way the reference would on its CPU backend: each layer is the unfused
chain of MathBackendCPU calls (conv2d -> add -> clip, depthwiseConv2D -> add -> clip, pool,
the 8-stage softmax), every call a full pass with its own float32 rounding.  Quantised
weights are dequantised on the host first, as tfjs-core/src/io/io_utils.ts:122-146 does at
load time.  Takes the same parameter dict the device model is built from.
"""
import numpy as np

import oracle

PW_OUT = [64, 128, 128, 256, 256, 512, 512, 512, 512, 512, 512, 1024, 1024]
DW_STRIDE = [1, 2, 1, 2, 1, 2, 1, 1, 1, 1, 1, 2, 1]


def float_weights(params):
    out = {}
    for name, p in params.items():
        w = p["w"] if p.get("q") is None else oracle.dequant_u8(p["q"], p["scale"], p["min"])
        out[name] = (np.asarray(w, np.float32), np.asarray(p["b"], np.float32))
    return out


def _conv_bias_clip(x, w, b, stride, clip=True):
    ci = oracle.compute_conv2d_info(x.shape, w.shape, stride, 1, "same")
    y = oracle.conv2d(x, w, ci)
    y = oracle.binary("add", y, b)
    return oracle.unary("clip", y, 0.0, 6.0) if clip else y


def forward(x, params, return_intermediates=False):
    """Returns (logits [B, 1000], probabilities [B, 1000])."""
    wts = float_weights(params)
    inter = {}
    h = _conv_bias_clip(np.asarray(x, np.float32), *wts["stem"], 2)
    inter["stem"] = h
    for i, s in enumerate(DW_STRIDE, 1):
        w, b = wts[f"dw{i}"]
        ci = oracle.compute_conv2d_info(h.shape, w.shape, s, 1, "same", None, True)
        h = oracle.depthwise_conv2d(h, w, ci)
        h = oracle.binary("add", h, b)
        h = oracle.unary("clip", h, 0.0, 6.0)
        inter[f"dw{i}"] = h
        h = _conv_bias_clip(h, *wts[f"pw{i}"], 1)
        inter[f"pw{i}"] = h
    ci = oracle.compute_pool2d_info(h.shape, [7, 7], 1, 1, "valid")
    h = oracle.pool(h, ci, "avg")
    h = _conv_bias_clip(h, *wts["fc"], 1, clip=False)
    logits = h.reshape(h.shape[0], -1)
    probs = oracle.softmax_last(logits)
    if return_intermediates:
        return logits, probs, inter
    return logits, probs
