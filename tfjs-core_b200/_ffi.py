"""ctypes binding of the C ABI declared in include/tfjs_cuda.h.

The same entry points are what a Node N-API shim binds; Python is the
host language here because no JavaScript toolchain exists on the build or GPU machines.
There is no fallback: if the shared library is missing this module raises.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtfjs_cuda.so")

OK = 0
ERR_INVALID_ARG, ERR_OOM, ERR_CUDA, ERR_TIMEOUT, ERR_UNSUPPORTED, ERR_NOT_FOUND = -1, -2, -3, -4, -5, -6
F32, I32, BOOL, F16 = 0, 1, 2, 3
ACT = {None: 0, "linear": 0, "relu": 1, "prelu": 2, "clip": 3}
MATH = {"3xtf32": 0, "tf32": 1}
BINARY = {"add": 0, "sub": 1, "mul": 2, "div": 3, "prelu": 4, "notEqual": 5}
UNARY = {"relu": 0, "clip": 1, "exp": 2, "log": 3, "int": 4, "step": 5}
REDUCE = {"sum": 0, "max": 1, "argMax": 2}


class ConvInfo(C.Structure):
    """tfjs_conv2d_info: Conv2DInfo of tfjs-core/src/ops/conv_util.ts:43-64, channelsLast."""
    _fields_ = [(n, C.c_int32) for n in (
        "batchSize", "inHeight", "inWidth", "inChannels", "outHeight", "outWidth", "outChannels",
        "strideHeight", "strideWidth", "dilationHeight", "dilationWidth", "filterHeight",
        "filterWidth", "effectiveFilterHeight", "effectiveFilterWidth", "padTop", "padBottom",
        "padLeft", "padRight")]

    @property
    def outShape(self):
        return [self.batchSize, self.outHeight, self.outWidth, self.outChannels]

    @property
    def inShape(self):
        return [self.batchSize, self.inHeight, self.inWidth, self.inChannels]


class Epilogue(C.Structure):
    _fields_ = [("bias", C.c_int64), ("bias_len", C.c_int64), ("activation", C.c_int32),
                ("prelu", C.c_int64), ("prelu_len", C.c_int64), ("clip_lo", C.c_float),
                ("clip_hi", C.c_float)]


class MemStats(C.Structure):
    _fields_ = [(n, C.c_int64) for n in ("num_tensors", "bytes_in_use", "bytes_reserved",
                                         "num_buffers_cached", "num_device_allocs")]


# name -> (restype, argtypes); mirrors include/tfjs_cuda.h one to one
_P = C.c_void_p
_I64P = C.POINTER(C.c_int64)
SIGNATURES = {
    "tfjs_cuda_ctx_create": (C.c_int, [C.c_int, C.POINTER(_P)]),
    "tfjs_cuda_device_count": (C.c_int, [C.POINTER(C.c_int)]),
    "tfjs_cuda_ctx_destroy": (C.c_int, [_P]),
    "tfjs_cuda_last_error": (C.c_char_p, [_P]),
    "tfjs_cuda_ctx_set_option": (C.c_int, [_P, C.c_char_p, C.c_double]),
    "tfjs_cuda_ctx_sync": (C.c_int, [_P, C.c_int]),
    "tfjs_cuda_ctx_memory": (C.c_int, [_P, C.POINTER(MemStats)]),
    "tfjs_cuda_ctx_time_begin": (C.c_int, [_P]),
    "tfjs_cuda_ctx_time_end": (C.c_int, [_P, C.POINTER(C.c_float), _I64P]),
    "tfjs_cuda_profile_begin": (C.c_int, [_P, C.c_int]),
    "tfjs_cuda_profile_end": (C.c_int, [_P, C.POINTER(C.c_int)]),
    "tfjs_cuda_profile_get": (C.c_int, [_P, C.c_int, C.POINTER(C.c_char_p), C.POINTER(C.c_float)]),
    "tfjs_cuda_ctx_launch_count": (C.c_int64, [_P]),
    "tfjs_cuda_ctx_stream": (_P, [_P]),
    "tfjs_cuda_tensor_register": (C.c_int, [_P, _I64P, C.c_int, _I64P, C.c_int]),
    "tfjs_cuda_tensor_write": (C.c_int, [_P, C.c_int64, _P, C.c_size_t]),
    "tfjs_cuda_tensor_read": (C.c_int, [_P, C.c_int64, _P, C.c_size_t]),
    "tfjs_cuda_tensor_write_async": (C.c_int, [_P, C.c_int64, _P, C.c_size_t]),
    "tfjs_cuda_tensor_wait": (C.c_int, [_P, C.c_int64]),
    "tfjs_cuda_tensor_read_async": (C.c_int, [_P, C.c_int64, _P, C.c_size_t, C.POINTER(_P)]),
    "tfjs_cuda_event_query": (C.c_int, [_P]),
    "tfjs_cuda_event_wait": (C.c_int, [_P, C.c_int]),
    "tfjs_cuda_event_destroy": (C.c_int, [_P]),
    "tfjs_cuda_tensor_dispose": (C.c_int, [_P, C.c_int64]),
    "tfjs_cuda_tensor_device_ptr": (C.c_int, [_P, C.c_int64, C.POINTER(_P), C.POINTER(C.c_size_t)]),
    "tfjs_cuda_host_alloc": (C.c_int, [C.POINTER(_P), C.c_size_t]),
    "tfjs_cuda_host_free": (C.c_int, [_P]),
    "tfjs_cuda_tensor_register_quantized": (C.c_int, [_P, _I64P, C.c_int, _I64P, _P, C.c_double,
                                                      C.c_double]),
    "tfjs_cuda_batch_matmul": (C.c_int, [_P, C.c_int64, C.c_int64, C.c_int64, C.c_int32, C.c_int32,
                                         C.c_int32, C.c_int32, C.c_int32, C.c_int, C.c_int,
                                         C.POINTER(Epilogue)]),
    "tfjs_cuda_conv2d": (C.c_int, [_P, C.c_int64, C.c_int64, C.c_int64, C.POINTER(ConvInfo),
                                   C.POINTER(Epilogue)]),
    "tfjs_cuda_depthwise_conv2d": (C.c_int, [_P, C.c_int64, C.c_int64, C.c_int64, C.POINTER(ConvInfo),
                                             C.POINTER(Epilogue)]),
    "tfjs_cuda_separable_conv2d": (C.c_int, [_P, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                                             C.POINTER(ConvInfo), C.c_int32, C.POINTER(Epilogue),
                                             C.POINTER(Epilogue)]),
    "tfjs_cuda_conv2d_der_input": (C.c_int, [_P, C.c_int64, C.c_int64, C.c_int64, C.POINTER(ConvInfo)]),
    "tfjs_cuda_conv2d_der_filter": (C.c_int, [_P, C.c_int64, C.c_int64, C.c_int64, C.POINTER(ConvInfo)]),
    "tfjs_cuda_depthwise_conv2d_der_input": (C.c_int, [_P, C.c_int64, C.c_int64, C.c_int64,
                                                       C.POINTER(ConvInfo)]),
    "tfjs_cuda_depthwise_conv2d_der_filter": (C.c_int, [_P, C.c_int64, C.c_int64, C.c_int64,
                                                        C.POINTER(ConvInfo)]),
    "tfjs_cuda_pool2d_backprop": (C.c_int, [_P, C.c_int64, C.c_int64, C.c_int64, C.POINTER(ConvInfo), C.c_int]),
    "tfjs_cuda_clip_backprop": (C.c_int, [_P, C.c_int64, C.c_int64, C.c_int64, C.c_float, C.c_float]),
    "tfjs_cuda_transpose": (C.c_int, [_P, C.c_int64, C.c_int64, C.c_int, _I64P, C.POINTER(C.c_int32)]),
    "tfjs_cuda_pool2d": (C.c_int, [_P, C.c_int64, C.c_int64, C.POINTER(ConvInfo), C.c_int]),
    "tfjs_cuda_binary": (C.c_int, [_P, C.c_int, C.c_int64, C.c_int, _I64P, C.c_int64, C.c_int, _I64P,
                                   C.c_int64]),
    "tfjs_cuda_unary": (C.c_int, [_P, C.c_int, C.c_int64, C.c_int64, C.c_float, C.c_float]),
    "tfjs_cuda_reduce_last": (C.c_int, [_P, C.c_int, C.c_int64, C.c_int64, C.c_int64, C.c_int64]),
    "tfjs_cuda_softmax_last": (C.c_int, [_P, C.c_int64, C.c_int64, C.c_int64, C.c_int64]),
    "tfjs_cuda_cast": (C.c_int, [_P, C.c_int64, C.c_int64]),
    "tfjs_cuda_matmul_static_scratch": (C.c_int, [_P, _P, _P, _P, _P, C.c_int64, C.c_int64, C.c_int64,
                                                  C.c_int, C.c_float, C.c_float]),
    "tfjs_cuda_graph_begin": (C.c_int, [_P]),
    "tfjs_cuda_graph_end": (C.c_int, [_P, C.POINTER(_P)]),
    "tfjs_cuda_graph_launch": (C.c_int, [_P, _P]),
    "tfjs_cuda_graph_destroy": (C.c_int, [_P, _P]),
}

_lib = None


def load():
    """Loads libtfjs_cuda.so and types every entry point.  Raises if the library is absent:
    the backend has no other implementation to fall back to."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python tfjs-core_b200/build.py` "
                "(the cuda backend has no CPU fallback)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def shape_array(shape):
    return (C.c_int64 * max(len(shape), 1))(*[int(s) for s in shape])
