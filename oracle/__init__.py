"""TEST INFRASTRUCTURE ONLY: numpy front-end of the CPU oracle (oracle.c).

The oracle restates tfjs-core's ``MathBackendCPU`` loops
(tfjs-core/src/backends/cpu/backend_cpu.ts) with JavaScript number semantics.  Only the
tests, the smoke check and the bench's cpu-baseline leg may import this module; the
shipped backend never does.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

PAD_VALID, PAD_SAME, PAD_NUMBER = 0, 1, 2
ROUND = {None: 0, "floor": 1, "round": 2, "ceil": 3}
ACT = {None: 0, "linear": 0, "relu": 1, "prelu": 2}
BINARY = {"add": 0, "sub": 1, "mul": 2, "div": 3, "prelu": 4}
UNARY = {"relu": 0, "clip": 1, "exp": 2, "log": 3}


class ConvInfo(C.Structure):
    """Mirror of Conv2DInfo (tfjs-core/src/ops/conv_util.ts:43-64), channelsLast."""

    _fields_ = [(n, C.c_int32) for n in (
        "batchSize", "inHeight", "inWidth", "inChannels", "outHeight", "outWidth",
        "outChannels", "strideHeight", "strideWidth", "dilationHeight", "dilationWidth",
        "filterHeight", "filterWidth", "effectiveFilterHeight", "effectiveFilterWidth",
        "padTop", "padBottom", "padLeft", "padRight")]

    @property
    def outShape(self):
        return (self.batchSize, self.outHeight, self.outWidth, self.outChannels)

    @property
    def inShape(self):
        return [self.batchSize, self.inHeight, self.inWidth, self.inChannels]

    def as_dict(self):
        return {n: getattr(self, n) for n, _ in self._fields_}


def build(force=False):
    """Compile liboracle.so with the flags the Makefile states."""
    if force or not os.path.exists(_LIB_PATH) or (
            os.path.getmtime(_LIB_PATH) < max(os.path.getmtime(os.path.join(_HERE, f))
                                              for f in ("oracle.c", "oracle_backward.c", "oracle.h"))):
        subprocess.check_call(["make", "-s", "-C", _HERE, "liboracle.so"])
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.tfo_binary.restype = C.c_int64
    return _lib


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _tuple2(v):
    return (v, v) if isinstance(v, int) else (int(v[0]), int(v[1]))


def compute_conv2d_info(in_shape, filter_shape, strides, dilations, pad,
                        rounding_mode=None, depthwise=False):
    sh, sw = _tuple2(strides)
    dh, dw = _tuple2(dilations)
    if pad == "same":
        mode, pv = PAD_SAME, 0
    elif pad == "valid":
        mode, pv = PAD_VALID, 0
    else:
        mode, pv = (PAD_NUMBER, int(pad)) if int(pad) != 0 else (PAD_NUMBER, 0)
    ci = ConvInfo()
    ins = (C.c_int32 * 4)(*in_shape)
    fs = (C.c_int32 * 4)(*filter_shape)
    rc = lib().tfo_compute_conv2d_info(ins, fs, sh, sw, dh, dw, mode, pv,
                                       ROUND[rounding_mode], int(depthwise), C.byref(ci))
    if rc != 0:
        raise ValueError("output size must be an integer; change stride and/or zero pad")
    return ci


def compute_pool2d_info(in_shape, filter_size, strides, dilations, pad, rounding_mode=None):
    """conv_util.ts:66-86 computePool2DInfo."""
    fh, fw = _tuple2(filter_size)
    return compute_conv2d_info(in_shape, (fh, fw, in_shape[3], in_shape[3]), strides,
                               dilations, pad, rounding_mode, False)


def batch_matmul(a, b, transpose_a=False, transpose_b=False):
    a, b = _f32(a), _f32(b)
    assert a.ndim == 3 and b.ndim == 3
    left = a.shape[2] if transpose_a else a.shape[1]
    right = b.shape[1] if transpose_b else b.shape[2]
    out = np.empty((a.shape[0], left, right), np.float32)
    lib().tfo_batch_matmul(_p(a), _p(b), _p(out), a.shape[0], a.shape[1], a.shape[2],
                           b.shape[1], b.shape[2], int(transpose_a), int(transpose_b))
    return out


def conv2d(x, w, ci):
    x, w = _f32(x), _f32(w)
    y = np.empty(ci.outShape, np.float32)
    lib().tfo_conv2d(_p(x), _p(w), _p(y), C.byref(ci))
    return y


def depthwise_conv2d(x, w, ci):
    x, w = _f32(x), _f32(w)
    y = np.empty(ci.outShape, np.float32)
    lib().tfo_depthwise_conv2d(_p(x), _p(w), _p(y), C.byref(ci))
    return y


def pool(x, ci, kind):
    x = _f32(x)
    y = np.empty(ci.outShape, np.float32)
    lib().tfo_pool(_p(x), _p(y), C.byref(ci), int(kind == "avg"))
    return y


def broadcast_shape(sa, sb):
    a = np.zeros(sa, np.float32)
    b = np.zeros(sb, np.float32)
    return np.broadcast(a, b).shape


def binary(op, a, b):
    a, b = _f32(a), _f32(b)
    ash = (C.c_int32 * max(a.ndim, 1))(*a.shape)
    bsh = (C.c_int32 * max(b.ndim, 1))(*b.shape)
    n = lib().tfo_binary(BINARY[op], _p(a), ash, a.ndim, _p(b), bsh, b.ndim, None)
    if n < 0:
        raise ValueError("Operands could not be broadcast together")
    out = np.empty(broadcast_shape(a.shape, b.shape), np.float32)
    assert out.size == n
    lib().tfo_binary(BINARY[op], _p(a), ash, a.ndim, _p(b), bsh, b.ndim, _p(out))
    return out


def unary(op, x, p0=0.0, p1=0.0):
    x = _f32(x)
    out = np.empty_like(x)
    lib().tfo_unary(UNARY[op], _p(x), _p(out), C.c_int64(x.size), C.c_double(p0), C.c_double(p1))
    return out


def _outer_inner(x):
    inner = x.shape[-1]
    return x.size // max(inner, 1), inner


def sum_last(x):
    x = _f32(x)
    o, i = _outer_inner(x)
    out = np.empty(x.shape[:-1], np.float32)
    lib().tfo_sum_last(_p(x), _p(out), C.c_int64(o), C.c_int64(i))
    return out


def max_last(x):
    x = _f32(x)
    o, i = _outer_inner(x)
    out = np.empty(x.shape[:-1], np.float32)
    lib().tfo_max_last(_p(x), _p(out), C.c_int64(o), C.c_int64(i))
    return out


def argmax_last(x):
    x = _f32(x)
    o, i = _outer_inner(x)
    out = np.empty(x.shape[:-1], np.int32)
    lib().tfo_argmax_last(_p(x), _p(out), C.c_int64(o), C.c_int64(i))
    return out


def softmax_last(x):
    x = _f32(x)
    o, i = _outer_inner(x)
    out = np.empty_like(x)
    lib().tfo_softmax_last(_p(x), _p(out), C.c_int64(o), C.c_int64(i))
    return out


def dequant_u8(q, scale, mn):
    q = np.ascontiguousarray(q, dtype=np.uint8)
    out = np.empty(q.shape, np.float32)
    lib().tfo_dequant_u8(_p(q), C.c_int64(q.size), C.c_double(scale), C.c_double(mn), _p(out))
    return out


def _epilogue_args(bias, prelu):
    bias = None if bias is None else _f32(bias)
    prelu = None if prelu is None else _f32(prelu)
    return (bias, prelu, _p(bias) if bias is not None else None,
            C.c_int64(bias.size if bias is not None else 0),
            _p(prelu) if prelu is not None else None,
            C.c_int64(prelu.size if prelu is not None else 0))


def fused_matmul(a, b, transpose_a=False, transpose_b=False, bias=None, activation=None,
                 prelu=None):
    """fusedBatchMatMul (backend_cpu.ts:542-555) for a bias/prelu broadcast over the
    inner-most axis only; compose batch_matmul + binary for other shapes."""
    a, b = _f32(a), _f32(b)
    left = a.shape[2] if transpose_a else a.shape[1]
    right = b.shape[1] if transpose_b else b.shape[2]
    out = np.empty((a.shape[0], left, right), np.float32)
    bias, prelu, bp, bn, pp, pn = _epilogue_args(bias, prelu)
    lib().tfo_fused_matmul(_p(a), _p(b), _p(out), a.shape[0], a.shape[1], a.shape[2],
                           b.shape[1], b.shape[2], int(transpose_a), int(transpose_b),
                           bp, bn, ACT[activation], pp, pn)
    return out


def fused_conv2d(x, w, ci, bias=None, activation=None, prelu=None):
    x, w = _f32(x), _f32(w)
    y = np.empty(ci.outShape, np.float32)
    bias, prelu, bp, bn, pp, pn = _epilogue_args(bias, prelu)
    lib().tfo_fused_conv2d(_p(x), _p(w), _p(y), C.byref(ci), bp, bn, ACT[activation], pp, pn)
    return y


# ---- gradient kernels (oracle_backward.c) ---------------------------------------------------------
def conv2d_der_input(dy, w, ci):
    """backend_cpu.ts:1686-1762"""
    dy, w = _f32(dy), _f32(w)
    dx = np.empty(ci.inShape, np.float32)
    lib().tfo_conv2d_der_input(_p(dy), _p(w), _p(dx), C.byref(ci))
    return dx


def conv2d_der_filter(x, dy, ci):
    """backend_cpu.ts:1849-1898"""
    x, dy = _f32(x), _f32(dy)
    dw = np.empty((ci.filterHeight, ci.filterWidth, ci.inChannels, ci.outChannels), np.float32)
    lib().tfo_conv2d_der_filter(_p(x), _p(dy), _p(dw), C.byref(ci))
    return dw


def depthwise_der_input(dy, w, ci):
    """backend_cpu.ts:2037-2102"""
    dy, w = _f32(dy), _f32(w)
    dx = np.empty(ci.inShape, np.float32)
    lib().tfo_depthwise_der_input(_p(dy), _p(w), _p(dx), C.byref(ci))
    return dx


def depthwise_der_filter(x, dy, ci):
    """backend_cpu.ts:2104-2150"""
    x, dy = _f32(x), _f32(dy)
    dw = np.empty((ci.filterHeight, ci.filterWidth, ci.inChannels, ci.outChannels // ci.inChannels), np.float32)
    lib().tfo_depthwise_der_filter(_p(x), _p(dy), _p(dw), C.byref(ci))
    return dw


def pool_backprop(dy, x, ci, kind):
    """backend_cpu.ts:2400-2509 maxPoolBackprop / avgPoolBackprop"""
    dy, x = _f32(dy), _f32(x)
    dx = np.empty(ci.inShape, np.float32)
    pos = np.empty(ci.outShape, np.int32)
    lib().tfo_pool_backprop(_p(dy), _p(x), _p(dx), pos.ctypes.data_as(C.c_void_p), C.byref(ci),
                            int(kind == "avg"))
    return dx


def step(x, alpha=0.0):
    """backend_cpu.ts:1520-1534"""
    x = _f32(x)
    out = np.empty(x.shape, np.float32)
    lib().tfo_step(_p(x), _p(out), C.c_int64(x.size), C.c_double(alpha))
    return out
