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
    x_shape = list(x.shape)
    return ENGINE.runKernel(lambda b: b.reshape(x, shape), "reshape", {"x": x},
                            lambda dy, saved: {"x": lambda: reshape(dy, x_shape)})


def cast(x, dtype):
    # array_ops.ts:412-419: the gradient passes through unchanged
    return ENGINE.runKernel(lambda b: b.cast(x, dtype), "cast", {"x": x},
                            lambda dy, saved: {"x": lambda: dy.clone()})


def clone(x):
    """tf.clone (ops/tensor_ops.ts): a new Tensor over the same storage; gradient passes through."""
    x = _convert(x, "x", "clone")
    return ENGINE.runKernel(lambda b: x.clone(), "clone", {"x": x}, lambda dy, saved: {"x": lambda: dy.clone()})


def square(x):
    """tf.square (unary_ops.ts:621-633): x * x with gradient 2 * x * dy."""
    x = _convert(x, "x", "square")

    def forward(b, save):
        save([x])
        return b.multiply(x, x)

    def backward(dy, saved):
        def dx():
            two = scalar(2.0)
            t = mul(saved[0], two)
            out = mul(dy, t)
            two.dispose()
            t.dispose()
            return out
        return {"x": dx}
    return ENGINE.runKernel(forward, "square", {"x": x}, backward)


def ones(shape):
    return tensor(np.ones(shape, np.float32), shape)


def zeros(shape):
    return tensor(np.zeros(shape, np.float32), shape)


def neg(x):
    """tf.neg (unary_ops.ts): -x, here as x * -1 (exact)."""
    m = scalar(-1.0)
    out = mul(x, m)
    m.dispose()
    return out


def step(x, alpha=0.0):
    """tf.step (unary_ops.ts:484-497)."""
    x = _convert(x, "x", "step")
    return ENGINE.runKernel(lambda b: b.step(x, alpha), "step", {"x": x},
                            lambda dy, saved: {"x": lambda: zeros(dy.shape)})


def transpose(x, perm=None):
    """tf.transpose (ops/transpose.ts)."""
    x = _convert(x, "x", "transpose")
    perm = list(range(x.rank))[::-1] if perm is None else [int(p) for p in perm]
    _assert(len(perm) == x.rank, f"Error in transpose: rank of input {x.rank} must match length of perm {perm}.")
    if x.rank <= 1:
        return x.clone()
    undo = [perm.index(i) for i in range(len(perm))]
    return ENGINE.runKernel(lambda b: b.transpose(x, perm), "transpose", {"x": x},
                            lambda dy, saved: {"x": lambda: transpose(dy, undo)})


def _reduce_to_shape(grad, shape, owns):
    """The tail of every broadcasting binary gradient (binary_ops.ts:62-80): sum over the
    broadcast axes (broadcast_util.ts getReductionAxes), then reshape to the operand's shape."""
    in_rank, out_rank = len(shape), grad.rank
    axes = []
    for i in range(in_rank):
        dim = in_rank - 1 - i
        out_axis = out_rank - 1 - i
        if shape[dim] == 1 and grad.shape[out_axis] > 1:
            axes.insert(0, out_axis)
    axes = list(range(out_rank - in_rank)) + axes
    res = grad
    if axes:
        res = sum(grad, axes)
        if owns:
            grad.dispose()
        owns = True
    out = reshape(res, list(shape))
    if owns:
        res.dispose()
    return out


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
    def forward(bk, save):
        y = bk.fusedBatchMatMul(a=a3, b=b3, transposeA=transposeA, transposeB=transposeB, bias=bias,
                                activation=activation, preluActivationWeights=preluActivationWeights)
        save([a3, b3, y])
        return y

    def backward(dy, saved):
        # fused_ops.ts:134-196 (linear and relu only, as in the reference); matmul.ts:92-115
        sa, sb, sy = saved
        _assert(activation in (None, "linear", "relu"),
                f"Gradient for activation {activation} has not been implemented yet.")
        state = {}

        def dy_act():
            if "v" not in state:
                if activation == "relu":
                    st = step(sy)
                    state["v"] = mul(dy, st)
                    st.dispose()
                else:
                    state["v"] = dy.clone()
            return state["v"]
        grads = {}
        if not transposeA and not transposeB:
            grads["a"] = lambda: fused_matmul(dy_act(), sb, False, True)
            grads["b"] = lambda: fused_matmul(sa, dy_act(), True, False)
        elif not transposeA and transposeB:
            grads["a"] = lambda: fused_matmul(dy_act(), sb, False, False)
            grads["b"] = lambda: fused_matmul(dy_act(), sa, True, False)
        elif transposeA and not transposeB:
            grads["a"] = lambda: fused_matmul(sb, dy_act(), False, True)
            grads["b"] = lambda: fused_matmul(sa, dy_act(), False, False)
        else:
            grads["a"] = lambda: fused_matmul(sb, dy_act(), True, True)
            grads["b"] = lambda: fused_matmul(dy_act(), sa, True, True)
        if bias is not None:
            grads["bias"] = lambda: _reduce_to_shape(dy_act(), bias.shape, False)
        return grads
    inputs = {"a": a3, "b": b3}
    if bias is not None:
        inputs["bias"] = bias
    res = ENGINE.runKernel(forward, "fusedBatchMatMul", inputs, backward)
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
    def forward(b, save):
        y = b.fusedConv2d(x4, filter, ci, bias, activation, preluActivationWeights)
        save([x4, filter, y])
        return y

    def backward(dy, saved):
        # fused_ops.ts:358-402 (linear and relu, dilation 1); conv.ts:187-206
        sx, sf, sy = saved
        _assert(activation in (None, "linear", "relu"),
                f"Gradient for activation {activation} has not been implemented yet.")
        _assert(ci.dilationHeight == 1 and ci.dilationWidth == 1,
                "Error in gradient of fused conv2D: dilation rates greater than 1 are not yet supported "
                f"in gradients. Got dilations '{dilations}'")
        state = {}

        def dy_act():
            if "v" not in state:
                if activation == "relu":
                    st = step(sy)
                    state["v"] = mul(dy, st)
                    st.dispose()
                else:
                    state["v"] = dy.clone()
            return state["v"]
        grads = {"x": lambda: ENGINE.runKernel(lambda b: b.conv2dDerInput(dy_act(), sf, ci), "conv2dDerInput"),
                 "filter": lambda: ENGINE.runKernel(lambda b: b.conv2dDerFilter(sx, dy_act(), ci), "conv2dDerFilter")}
        if bias is not None:
            grads["bias"] = lambda: _reduce_to_shape(dy_act(), bias.shape, False)
        return grads
    inputs = {"x": x4, "filter": filter}
    if bias is not None:
        inputs["bias"] = bias
    res = ENGINE.runKernel(forward, "fusedConv2d", inputs, backward)
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
    def forward(b, save):
        save([x4, filter])
        return b.conv2d(x4, filter, ci)

    def backward(dy, saved):
        # conv.ts:187-206
        sx, sf = saved
        _assert(ci.dilationHeight == 1 and ci.dilationWidth == 1,
                "Error in gradient of conv2D: dilation rates greater than 1 are not yet supported in "
                f"gradients. Got dilations '{dilations}'")
        return {"x": lambda: ENGINE.runKernel(lambda b: b.conv2dDerInput(dy, sf, ci), "conv2dDerInput"),
                "filter": lambda: ENGINE.runKernel(lambda b: b.conv2dDerFilter(sx, dy, ci), "conv2dDerFilter")}
    res = ENGINE.runKernel(forward, "conv2d", {"x": x4, "filter": filter}, backward)
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
    def forward(b, save):
        save([x4, filter])
        return b.depthwiseConv2D(x4, filter, ci)

    def backward(dy, saved):
        # conv.ts:519-530
        sx, sf = saved
        _assert(ci.dilationHeight == 1 and ci.dilationWidth == 1,
                "Error in gradient of depthwiseConv2d: dilation rates greater than 1 are not yet "
                f"supported. Got dilations '{dilations}'")
        return {"x": lambda: ENGINE.runKernel(lambda b: b.depthwiseConv2DDerInput(dy, sf, ci),
                                              "depthwiseConv2DDerInput"),
                "filter": lambda: ENGINE.runKernel(lambda b: b.depthwiseConv2DDerFilter(sx, dy, ci),
                                                   "depthwiseConv2DDerFilter")}
    res = ENGINE.runKernel(forward, "depthwiseConv2D", {"x": x4, "filter": filter}, backward)
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
    def forward(b, save):
        y = b.avgPool(x4, ci) if kind == "avg" else b.maxPool(x4, ci)
        save([x4, y])
        return y

    def backward(dy, saved):
        # pool.ts:104-112 (max), :217-221 (avg)
        sx, sy = saved
        if kind == "avg":
            return {"x": lambda: ENGINE.runKernel(lambda b: b.avgPoolBackprop(dy, sx, ci), "avgPoolBackprop")}
        return {"x": lambda: ENGINE.runKernel(lambda b: b.maxPoolBackprop(dy, sx, sy, ci), "maxPoolBackprop")}
    res = ENGINE.runKernel(forward, kind + "Pool", {"x": x4}, backward)
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

    def forward(bk, save):
        save([a, b])
        return getattr(bk, method)(a, b)

    def backward(dy, saved):
        sa, sb = saved
        if method == "add":          # binary_ops.ts:62-80
            return {"a": lambda: _reduce_to_shape(dy, sa.shape, False),
                    "b": lambda: _reduce_to_shape(dy, sb.shape, False)}
        if method == "subtract":     # binary_ops.ts:211-229
            return {"a": lambda: _reduce_to_shape(dy, sa.shape, False),
                    "b": lambda: _reduce_to_shape(neg(dy), sb.shape, True)}
        if method == "multiply":     # binary_ops.ts:353-369
            return {"a": lambda: _reduce_to_shape(mul(dy, sb), sa.shape, True),
                    "b": lambda: _reduce_to_shape(mul(dy, sa), sb.shape, True)}
        if method == "realDivide":   # binary_ops.ts:448-466: da = dy / b, db = -(dy * a) / b^2
            def db():
                num = mul(dy, sa)
                sq = mul(sb, sb)
                q = div(num, sq)
                out = _reduce_to_shape(neg(q), sb.shape, True)
                for t in (num, sq, q):
                    t.dispose()
                return out
            return {"a": lambda: _reduce_to_shape(div(dy, sb), sa.shape, True), "b": db}
        raise NotImplementedError(f"gradient of {method} is not defined on this path")
    return ENGINE.runKernel(forward, method, {"a": a, "b": b}, backward)


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

    def forward(b, save):
        save([x])
        return b.relu(x)

    def backward(dy, saved):
        # relu_ops.ts:43-49: dy * step(x)
        def dx():
            st = step(saved[0])
            out = mul(dy, st)
            st.dispose()
            return out
        return {"x": dx}
    return ENGINE.runKernel(forward, "relu", {"x": x}, backward)


def prelu(x, alpha):
    return _binary("prelu", "prelu", x, alpha)


def clip_by_value(x, clipValueMin, clipValueMax):
    """tf.clipByValue (ops/unary_ops.ts:442-465); relu6 in this API is clipByValue(x, 0, 6)."""
    x = _convert(x, "x", "clipByValue")
    _assert(clipValueMin <= clipValueMax,
            f"Error in clip: min ({clipValueMin}) must be less than or equal to max ({clipValueMax}).")
    def forward(b, save):
        save([x])
        return b.clip(x, clipValueMin, clipValueMax)

    def backward(dy, saved):
        # unary_ops.ts:456-462: dy where min <= x <= max, zero elsewhere
        return {"x": lambda: ENGINE.runKernel(
            lambda b: b.clipBackprop(dy, saved[0], clipValueMin, clipValueMax), "clipBackprop")}
    return ENGINE.runKernel(forward, "clip", {"x": x}, backward)


def exp(x):
    x = _convert(x, "x", "exp")

    def forward(b, save):
        y = b.exp(x)
        save([y])
        return y
    # unary_ops.ts:233-236: dy * y
    return ENGINE.runKernel(forward, "exp", {"x": x}, lambda dy, saved: {"x": lambda: mul(dy, saved[0])})


def log(x):
    x = _convert(x, "x", "log")

    def forward(b, save):
        save([x])
        return b.log(x)
    # unary_ops.ts:275-278: dy / x
    return ENGINE.runKernel(forward, "log", {"x": x}, lambda dy, saved: {"x": lambda: div(dy, saved[0])})


# ---- reductions (ops/reduction_ops.ts; inner-most axes only on this path) ------------------
def _parse_axes(axis, rank):
    if axis is None:
        return list(range(rank))
    axes = [axis] if isinstance(axis, int) else list(axis)
    return [a + rank if a < 0 else a for a in axes]


def _reduce(x, axis, keepDims, method):
    x = _convert(x, "x", method)
    axes = sorted(_parse_axes(axis, x.rank))
    x_shape = list(x.shape)
    # axis_util.ts getAxesPermutation: the backend reduces inner-most axes only
    inner = list(range(x.rank - len(axes), x.rank))
    permuted, red_axes = x, axes
    if axes != inner:
        perm = [i for i in range(x.rank) if i not in axes] + axes
        permuted = transpose(x, perm)
        red_axes = inner
    if method == "sum":
        def backward(dy, saved):
            # reduction_ops.ts:122-135: dy broadcast back over the reduced axes
            def dx():
                expanded = reshape(dy, [1 if i in red_axes else s for i, s in enumerate(permuted.shape)])
                one = ones(permuted.shape)
                out = mul(expanded, one)
                expanded.dispose()
                one.dispose()
                return out
            return {"x": dx}
        res = ENGINE.runKernel(lambda b: b.sum(permuted, red_axes), "sum", {"x": permuted}, backward)
    else:
        res = ENGINE.runKernel(lambda b: getattr(b, method)(permuted, red_axes), method)
    if permuted is not x:
        permuted.dispose()
    if keepDims:
        shape = [1 if i in axes else s for i, s in enumerate(x_shape)]
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
    def forward(backend, save):
        # nested ops run below kernel depth 1, so the tape records this op as one node whose
        # gradient is the custom one below (softmax.ts:57-73, customGrad)
        lse = log_sum_exp(logits, [dim], True)
        lf = cast(logits, "float32")
        log_result = sub(lf, lse)
        y = exp(log_result)
        for t in (lse, lf, log_result):
            t.dispose()
        save([y])
        return y
    return ENGINE.runKernel(forward, None, {"logits": logits}, _softmax_grad(dim))


def _softmax_grad(dim):
    def backward(dy, saved):
        y = saved[0]

        def dlogits():
            dy_times_y = mul(dy, y)
            s_ = sum(dy_times_y, [dim], True)
            sy = mul(s_, y)
            out = sub(dy_times_y, sy)
            for t in (dy_times_y, s_, sy):
                t.dispose()
            return out
        return {"logits": dlogits}
    return backward


def fused_softmax(logits):
    """Extension: the same function as softmax() in one kernel."""
    logits = _convert(logits, "logits", "softmax")

    def forward(b, save):
        y = b.softmax(logits)
        save([y])
        return y
    return ENGINE.runKernel(forward, "softmax", {"logits": logits}, _softmax_grad(logits.rank - 1))


# ---- gradients (ops/gradients.ts) ----------------------------------------------------------------
def grad(f):
    """tf.grad(f)(x, dy?) -> df/dx."""
    def g(x, dy=None):
        x = _convert(x, "x", "tf.grad")

        def run():   # gradients.ts:68-80: tidy, so that the value of f and its temporaries go
            _, grads = ENGINE.gradients(lambda: f(x), [x], dy)
            return grads[0]
        return ENGINE.tidy(run)
    return g


def grads(f):
    """tf.grads(f)([x1, x2, ...], dy?) -> [df/dx1, ...]."""
    def g(xs, dy=None):
        xs = [_convert(x, "args", "tf.grads") for x in xs]

        def run():   # gradients.ts:117-127
            _, out = ENGINE.gradients(lambda: f(*xs), xs, dy)
            return out
        return ENGINE.tidy(run)
    return g


def value_and_grads(f):
    """tf.valueAndGrads(f)([x1, ...], dy?) -> (value, [grads])."""
    def g(xs, dy=None):
        xs = [_convert(x, "args", "tf.valueAndGrads") for x in xs]
        return ENGINE.gradients(lambda: f(*xs), xs, dy)
    return g
