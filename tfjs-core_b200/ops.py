"""The slice of tfjs-core's op layer that the MobileNet inference path goes through.

Each function restates the checks and shape arithmetic of the TypeScript op (cited per
function) and then calls the backend method through ENGINE.runKernel, exactly as the real op
layer does; the real op layer is unchanged TypeScript and would sit above the same backend.
Used by the model driver and by the tests, which read like the reference's specs
(`tf.fused.conv2d({x, filter, ...})` becomes `ops.fused_conv2d(x=x, filter=w, ...)`).
"""
import numpy as np

from . import conv_util
from .backend_cuda import assert_and_get_broadcast_shape
from .engine import ENGINE, NP_DTYPE, Tensor, size_from_shape


def _assert(cond, msg):
    if not cond:
        raise ValueError(msg() if callable(msg) else msg)


def tensor(values, shape=None, dtype="float32"):
    """tf.tensor (ops/tensor_ops.ts:55-113)."""
    arr = np.asarray(values)
    if shape is None:
        shape = list(arr.shape)
    _assert(size_from_shape(shape) == arr.size,
            f"Based on the provided shape, {list(shape)}, the tensor should have "
            f"{size_from_shape(shape)} values but has {arr.size}")
    return Tensor(shape, dtype, np.ascontiguousarray(arr.reshape(-1), dtype=NP_DTYPE[dtype]))


def scalar(value, dtype="float32"):
    return tensor([value], [], dtype)


def _convert(x, name, op):
    """convertToTensor (tensor_util_env.ts)."""
    if isinstance(x, Tensor):
        return x
    _assert(x is not None and not isinstance(x, (str, dict)),
            f"Argument '{name}' passed to '{op}' must be a Tensor or TensorLike")
    return tensor(x)


def reshape(x, shape):
    """ops/array_ops.ts reshape: metadata only, dispatched through runKernel."""
    shape = list(shape)
    if -1 in shape:
        known = size_from_shape([s for s in shape if s != -1])
        shape[shape.index(-1)] = x.size // known if known else 0
    _assert(size_from_shape(shape) == x.size, "new shape and old shape must have the same number of elements.")
    return ENGINE.runKernel(lambda b: b.reshape(x, shape), "reshape")


def cast(x, dtype):
    return ENGINE.runKernel(lambda b: b.cast(x, dtype), "cast")


# ---- matMul ------------------------------------------------------------------------------
def fused_matmul(a, b, transposeA=False, transposeB=False, bias=None, activation="linear",
                 preluActivationWeights=None):
    """tf.fused.matMul (ops/fused_ops.ts:52-218)."""
    a = _convert(a, "a", "fused matMul")
    b = _convert(b, "b", "fused matMul")
    inner_a = a.shape[-2] if transposeA else a.shape[-1]
    inner_b = b.shape[-1] if transposeB else b.shape[-2]
    outer_a = a.shape[-1] if transposeA else a.shape[-2]
    outer_b = b.shape[-2] if transposeB else b.shape[-1]
    _assert(a.rank >= 2 and b.rank >= 2 and a.rank == b.rank,
            f"Error in fused matMul: inputs must have the same rank of at least 2, got ranks "
            f"{a.rank} and {b.rank}.")
    _assert(a.shape[:-2] == b.shape[:-2],
            f"Error in fused matMul: outer dimensions ({a.shape[:-2]}) and ({b.shape[:-2]}) of "
            f"Tensors with shapes {a.shape} and {b.shape} must match.")
    _assert(inner_a == inner_b,
            f"Error in fused matMul: inner shapes ({inner_a}) and ({inner_b}) of Tensors with "
            f"shapes {a.shape} and {b.shape} and transposeA={transposeA} and "
            f"transposeB={transposeB} must match.")
    out_shape = a.shape[:-2] + [outer_a, outer_b]
    batch = size_from_shape(a.shape[:-2])
    a3 = reshape(a, [batch] + a.shape[-2:])
    b3 = reshape(b, [batch] + b.shape[-2:])
    if bias is not None:
        bias = _convert(bias, "bias", "fused matMul")
        assert_and_get_broadcast_shape(out_shape, bias.shape)
    if preluActivationWeights is not None:
        preluActivationWeights = _convert(preluActivationWeights, "prelu weights", "fused matMul")
    res = ENGINE.runKernel(lambda bk: bk.fusedBatchMatMul(
        a=a3, b=b3, transposeA=transposeA, transposeB=transposeB, bias=bias, activation=activation,
        preluActivationWeights=preluActivationWeights), "fusedBatchMatMul")
    out = reshape(res, out_shape)
    for t in (a3, b3, res):
        t.dispose()
    return out


def matmul(a, b, transposeA=False, transposeB=False):
    """tf.matMul (ops/matmul.ts:43-118)."""
    return fused_matmul(a, b, transposeA, transposeB)


# ---- convolutions ------------------------------------------------------------------------
def _as4d(x):
    if x.rank == 3:
        return reshape(x, [1] + x.shape), True
    return x, False


def _conv_checks(x4, filt, strides, dilations, name):
    _assert(x4.rank == 4, f"Error in {name}: input must be rank 4, but got rank {x4.rank}.")
    _assert(filt.rank == 4, f"Error in {name}: filter must be rank 4, but got rank {filt.rank}.")
    _assert(conv_util.either_strides_or_dilations_are_one(strides, dilations),
            f"Error in {name}: Either strides or dilations must be 1. Got strides {strides} and "
            f"dilations '{dilations}'")


def fused_conv2d(x, filter, strides, pad, dataFormat="NHWC", dilations=(1, 1), dimRoundingMode=None,
                 bias=None, activation="linear", preluActivationWeights=None):
    """tf.fused.conv2d (ops/fused_ops.ts:276-425)."""
    x = _convert(x, "x", "conv2d")
    filter = _convert(filter, "filter", "conv2d")
    x4, reshaped = _as4d(x)
    _conv_checks(x4, filter, strides, dilations, "fused conv2d")
    if dimRoundingMode is not None:
        _assert(isinstance(pad, int), "Error in fused conv2d: pad must be an integer when using "
                f"dimRoundingMode {dimRoundingMode} but got pad {pad}.")
    _assert(x4.shape[3] == filter.shape[2],
            f"Error in conv2d: depth of input ({x4.shape[3]}) must match input depth for filter "
            f"{filter.shape[2]}.")
    _assert(dataFormat == "NHWC",
            f"Error in conv2d: got dataFormat of {dataFormat} but only NHWC is currently supported.")
    ci = conv_util.compute_conv2d_info(x4.shape, filter.shape, strides, dilations, pad, dimRoundingMode)
    if bias is not None:
        bias = _convert(bias, "bias", "fused conv2d")
        assert_and_get_broadcast_shape(ci.outShape, bias.shape)
    if preluActivationWeights is not None:
        preluActivationWeights = _convert(preluActivationWeights, "prelu weights", "fused conv2d")
    res = ENGINE.runKernel(lambda b: b.fusedConv2d(x4, filter, ci, bias, activation,
                                                   preluActivationWeights), "fusedConv2d")
    if reshaped:
        out = reshape(res, res.shape[1:])
        res.dispose()
        x4.dispose()
        return out
    return res


def conv2d(x, filter, strides, pad, dataFormat="NHWC", dilations=(1, 1), dimRoundingMode=None):
    """tf.conv2d (ops/conv.ts:145-215)."""
    x = _convert(x, "x", "conv2d")
    filter = _convert(filter, "filter", "conv2d")
    x4, reshaped = _as4d(x)
    _conv_checks(x4, filter, strides, dilations, "conv2d")
    _assert(dataFormat == "NHWC", "the cuda backend supports conv2d in NHWC only")
    _assert(x4.shape[3] == filter.shape[2],
            f"Error in conv2d: depth of input ({x4.shape[3]}) must match input depth for filter "
            f"{filter.shape[2]}.")
    ci = conv_util.compute_conv2d_info(x4.shape, filter.shape, strides, dilations, pad, dimRoundingMode)
    res = ENGINE.runKernel(lambda b: b.conv2d(x4, filter, ci), "conv2d")
    if reshaped:
        out = reshape(res, res.shape[1:])
        res.dispose()
        x4.dispose()
        return out
    return res


def depthwise_conv2d(x, filter, strides, pad, dataFormat="NHWC", dilations=(1, 1), dimRoundingMode=None):
    """tf.depthwiseConv2d (ops/conv.ts:470-542)."""
    x = _convert(x, "x", "depthwiseConv2d")
    filter = _convert(filter, "filter", "depthwiseConv2d")
    x4, reshaped = _as4d(x)
    _assert(x4.rank == 4, f"Error in depthwiseConv2d: input must be rank 4, but got rank {x4.rank}.")
    _assert(filter.rank == 4, f"Error in depthwiseConv2d: filter must be rank 4, but got rank {filter.rank}.")
    _assert(x4.shape[3] == filter.shape[2],
            f"Error in depthwiseConv2d: number of input channels ({x4.shape[3]}) must match the "
            f"inChannels dimension in filter {filter.shape[2]}.")
    _assert(conv_util.either_strides_or_dilations_are_one(strides, dilations),
            f"Error in depthwiseConv2d: Either strides or dilations must be 1. Got strides {strides} "
            f"and dilations '{dilations}'")
    ci = conv_util.compute_conv2d_info(x4.shape, filter.shape, strides, dilations, pad, dimRoundingMode, True)
    res = ENGINE.runKernel(lambda b: b.depthwiseConv2D(x4, filter, ci), "depthwiseConv2D")
    if reshaped:
        out = reshape(res, res.shape[1:])
        res.dispose()
        x4.dispose()
        return out
    return res


def separable_conv2d(x, depthwiseFilter, pointwiseFilter, strides, pad, dilation=(1, 1)):
    """tf.separableConv2d (ops/conv.ts:582-650): depthwise, then a 1x1 stride-1 valid conv2d."""
    _assert(pointwiseFilter.shape[0] == 1 and pointwiseFilter.shape[1] == 1,
            "Error in separableConv2d: the pointwise filter must be 1x1")
    dw = depthwise_conv2d(x, depthwiseFilter, strides, pad, "NHWC", dilation)
    out = conv2d(dw, pointwiseFilter, 1, "valid")
    dw.dispose()
    return out


# ---- pooling (ops/pool.ts:53-231) ---------------------------------------------------------
def _pool(x, filterSize, strides, pad, dimRoundingMode, kind):
    x = _convert(x, "x", kind + "Pool")
    x4, reshaped = _as4d(x)
    _assert(x4.rank == 4, f"Error in {kind}Pool: x must be rank 4 but got rank {x4.rank}.")
    if kind == "avg":
        _assert(x4.dtype == "float32", "The input dtype to avgPool must be float32")
    if dimRoundingMode is not None:
        _assert(isinstance(pad, int), f"Error in {kind}Pool: pad must be an integer when using, "
                f"dimRoundingMode {dimRoundingMode} but got pad {pad}.")
    ci = conv_util.compute_pool2d_info(x4.shape, filterSize, strides, 1, pad, dimRoundingMode)
    res = ENGINE.runKernel(lambda b: b.avgPool(x4, ci) if kind == "avg" else b.maxPool(x4, ci),
                           kind + "Pool")
    if reshaped:
        out = reshape(res, res.shape[1:])
        res.dispose()
        x4.dispose()
        return out
    return res


def max_pool(x, filterSize, strides, pad, dimRoundingMode=None):
    return _pool(x, filterSize, strides, pad, dimRoundingMode, "max")


def avg_pool(x, filterSize, strides, pad, dimRoundingMode=None):
    return _pool(x, filterSize, strides, pad, dimRoundingMode, "avg")


# ---- element-wise (ops/binary_ops.ts, ops/unary_ops.ts, ops/relu_ops.ts) -------------------
def _binary(name, method, a, b):
    a = _convert(a, "a", name)
    b = _convert(b, "b", name)
    assert_and_get_broadcast_shape(a.shape, b.shape)
    return ENGINE.runKernel(lambda bk: getattr(bk, method)(a, b), method)


def add(a, b):
    return _binary("add", "add", a, b)


def sub(a, b):
    return _binary("sub", "subtract", a, b)


def mul(a, b):
    return _binary("mul", "multiply", a, b)


def div(a, b):
    return _binary("div", "realDivide", a, b)


def relu(x):
    x = _convert(x, "x", "relu")
    return ENGINE.runKernel(lambda b: b.relu(x), "relu")


def prelu(x, alpha):
    return _binary("prelu", "prelu", x, alpha)


def clip_by_value(x, clipValueMin, clipValueMax):
    """tf.clipByValue (ops/unary_ops.ts:442-465); relu6 in this API is clipByValue(x, 0, 6)."""
    x = _convert(x, "x", "clipByValue")
    _assert(clipValueMin <= clipValueMax,
            f"Error in clip: min ({clipValueMin}) must be less than or equal to max ({clipValueMax}).")
    return ENGINE.runKernel(lambda b: b.clip(x, clipValueMin, clipValueMax), "clip")


def exp(x):
    return ENGINE.runKernel(lambda b: b.exp(_convert(x, "x", "exp")), "exp")


def log(x):
    return ENGINE.runKernel(lambda b: b.log(_convert(x, "x", "log")), "log")


# ---- reductions (ops/reduction_ops.ts; inner-most axes only on this path) ------------------
def _parse_axes(axis, rank):
    if axis is None:
        return list(range(rank))
    axes = [axis] if isinstance(axis, int) else list(axis)
    return [a + rank if a < 0 else a for a in axes]


def _reduce(x, axis, keepDims, method):
    x = _convert(x, "x", method)
    axes = _parse_axes(axis, x.rank)
    res = ENGINE.runKernel(lambda b: getattr(b, method)(x, axes), method)
    if keepDims:
        shape = [1 if i in axes else s for i, s in enumerate(x.shape)]
        out = reshape(res, shape)
        res.dispose()
        return out
    return res


def sum(x, axis=None, keepDims=False):
    return _reduce(x, axis, keepDims, "sum")


def max(x, axis=None, keepDims=False):
    return _reduce(x, axis, keepDims, "max")


def arg_max(x, axis=0):
    x = _convert(x, "x", "argMax")
    return ENGINE.runKernel(lambda b: b.argMax(x, axis % x.rank if x.rank else 0), "argMax")


def log_sum_exp(x, axis=None, keepDims=False):
    """ops/reduction_ops.ts:56-73: max, sub, exp, sum, log, add."""
    x = _convert(x, "x", "logSumExp")
    axes = _parse_axes(axis, x.rank)
    x_max = max(x, axes, True)
    a = sub(x, x_max)
    b = exp(a)
    c = sum(b, axes)
    d = log(c)
    xm2 = reshape(x_max, d.shape)
    res = add(xm2, d)
    for t in (x_max, a, b, c, d, xm2):
        t.dispose()
    if keepDims:
        shape = [1 if i in axes else s for i, s in enumerate(x.shape)]
        out = reshape(res, shape)
        res.dispose()
        return out
    return res


def softmax(logits, dim=-1):
    """tf.softmax (ops/softmax.ts:45-76) as the op layer composes it: exp(x - logSumExp(x)),
    i.e. eight backend kernels."""
    logits = _convert(logits, "logits", "softmax")
    if dim == -1:
        dim = logits.rank - 1
    if dim != logits.rank - 1:
        raise ValueError("Softmax along a non-last dimension is not yet supported. "
                         f"Logits was rank {logits.rank} and dim was {dim}")
    lse = log_sum_exp(logits, [dim], True)
    lf = cast(logits, "float32")
    log_result = sub(lf, lse)
    y = exp(log_result)
    for t in (lse, lf, log_result):
        t.dispose()
    return y


def fused_softmax(logits):
    """Extension: the same function as softmax() in one kernel."""
    logits = _convert(logits, "logits", "softmax")
    return ENGINE.runKernel(lambda b: b.softmax(logits), "softmax")
