"""TEST INFRASTRUCTURE ONLY: float64 numpy implementations of the hot-path operators and of
the MobileNetV1 forward pass, written independently of the CPU oracle.

Two uses.  (1) An independent cross-check of the oracle on the shapes the reference's own
known-answer vectors do not pin (stride-2 SAME depthwise, 3x3 SAME convolution over many input
channels, matMul with K beyond one 48-wide block): the oracle follows MathBackendCPU's loop
nests (tfjs-core/src/backends/cpu/backend_cpu.ts:491-540, 1552-1616, 1979-2035), this file
uses im2col / shifted-slice sums in float64, so a restatement slip in either shows up as a
disagreement far above float32 rounding.  (2) A common yardstick for whole-network error: the
oracle (float32 stores, one rounding per multiply-add) and the device kernels (TF32 or 3xTF32
products, float32 accumulators) both deviate from exact arithmetic on the same weights; comparing
each with this float64 forward separates "the kernels are wrong" from "the network amplifies
rounding".

Padding follows ops/conv_util.ts:399-435 (SAME: out = ceil(in / stride), the smaller half of the
padding on the top / left).
"""
import numpy as np

PW_OUT = [64, 128, 128, 256, 256, 512, 512, 512, 512, 512, 512, 1024, 1024]
DW_STRIDE = [1, 2, 1, 2, 1, 2, 1, 1, 1, 1, 1, 2, 1]


def same_padding(size, filt, stride, dilation=1):
    eff = filt + (filt - 1) * (dilation - 1)
    out = -(-size // stride)
    total = max(0, (out - 1) * stride + eff - size)
    before = total // 2
    return out, before, total - before


def _padded(x, fh, fw, stride, dilation=1):
    _, h, w, _ = x.shape
    oh, pt, pb = same_padding(h, fh, stride, dilation)
    ow, pl, pr = same_padding(w, fw, stride, dilation)
    return np.pad(x, ((0, 0), (pt, pb), (pl, pr), (0, 0))), oh, ow


def conv2d_same(x, w, stride=1, dilation=1):
    """NHWC x [fh, fw, cin, cout], SAME padding, float64 accumulation."""
    x = np.asarray(x, np.float64)
    w = np.asarray(w, np.float64)
    fh, fw, cin, cout = w.shape
    xp, oh, ow = _padded(x, fh, fw, stride, dilation)
    y = np.zeros((x.shape[0], oh, ow, cout), np.float64)
    for r in range(fh):
        for c in range(fw):
            r0, c0 = r * dilation, c * dilation
            patch = xp[:, r0:r0 + (oh - 1) * stride + 1:stride, c0:c0 + (ow - 1) * stride + 1:stride, :]
            y += patch.reshape(-1, cin) .dot(w[r, c]).reshape(y.shape)
    return y


def depthwise_same(x, w, stride=1, dilation=1):
    """NHWC x [fh, fw, c, 1], channel multiplier 1, SAME padding, float64."""
    x = np.asarray(x, np.float64)
    w = np.asarray(w, np.float64)
    fh, fw, c, mult = w.shape
    assert mult == 1
    xp, oh, ow = _padded(x, fh, fw, stride, dilation)
    y = np.zeros((x.shape[0], oh, ow, c), np.float64)
    for r in range(fh):
        for col in range(fw):
            r0, c0 = r * dilation, col * dilation
            y += xp[:, r0:r0 + (oh - 1) * stride + 1:stride, c0:c0 + (ow - 1) * stride + 1:stride, :] * w[r, col, :, 0]
    return y


def matmul(a, b):
    return np.asarray(a, np.float64) @ np.asarray(b, np.float64)


def relu6(x):
    return np.clip(x, 0.0, 6.0)


def softmax(z):
    z = z - z.max(axis=1, keepdims=True)
    e = np.exp(z)
    return e / e.sum(axis=1, keepdims=True)


def float_weights(params):
    """{name: (float32 filter values, bias)}.  uint8 entries are dequantised to the float32 the
    reference's loader produces, float32(float64(q) * scale + min) (io/io_utils.ts:137-143); the
    forward pass below then computes on those float32 VALUES exactly, in float64."""
    out = {}
    for name, p in params.items():
        if p.get("q") is not None:
            w = (p["q"].astype(np.float64) * p["scale"] + p["min"]).astype(np.float32)
        else:
            w = np.asarray(p["w"], np.float32)
        out[name] = (w, np.asarray(p["b"], np.float32))
    return out


def forward(x, params, chunk=8):
    """MobileNetV1-1.0-224 in float64.  Returns (logits [B, 1000], probabilities)."""
    wts = float_weights(params)
    logits = []
    for i in range(0, x.shape[0], chunk):
        h = np.asarray(x[i:i + chunk], np.float64)
        w, b = wts["stem"]
        h = relu6(conv2d_same(h, w, 2) + b)
        for k, s in enumerate(DW_STRIDE, 1):
            w, b = wts[f"dw{k}"]
            h = relu6(depthwise_same(h, w, s) + b)
            w, b = wts[f"pw{k}"]
            n, hh, ww, c = h.shape
            h = relu6(matmul(h.reshape(-1, c), w.reshape(c, -1)) + b).reshape(n, hh, ww, -1)
        h = h.mean(axis=(1, 2))
        w, b = wts["fc"]
        logits.append(matmul(h, w.reshape(w.shape[2], -1)) + b)
    logits = np.concatenate(logits, 0)
    return logits, softmax(logits)


def quantize_params(params):
    """The uint8-stored form of a float parameter dict (the product's own helper)."""
    from tfjs_core_b200 import mobilenet
    return mobilenet.quantize_params(params)
