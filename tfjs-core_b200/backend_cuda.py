"""`BackendCuda`: the KernelBackend implementation for B200, host side.

Mirrors the plugin class a TypeScript `class BackendCuda extends KernelBackend`
(tfjs-core/src/backends/backend.ts:91-649) would be: same method names, argument order and
error behaviour, each method a thin marshalling layer over the C ABI (include/tfjs_cuda.h)
that only enqueues device work.  Tensor data lives in device memory owned by the library and
moves to the host only in readSync()/read().

Methods outside the reference's surface are extensions and are named in their docstrings:
a clip/relu6 activation for the fused ops, fusedDepthwiseConv2D, softmax, quantised weight
registration and CUDA-graph capture.  Each has an unfused equivalent through the plain
methods, which is what unmodified tf.* code reaches.
"""
import ctypes as C
import time as _time
import weakref

import numpy as np

from . import _ffi
from .engine import ENGINE, NP_DTYPE, Tensor, size_from_shape

EPSILON_FLOAT32 = 1e-7  # backends/backend.ts:23
EPSILON_FLOAT16 = 1e-4  # backends/backend.ts:24
_DTYPE_CODE = {"float32": _ffi.F32, "int32": _ffi.I32, "bool": _ffi.BOOL, "float16": _ffi.F16}
# host-side element type per STORAGE dtype: half-stored tensors travel as float32 (the library converts)
_HOST_DTYPE = dict(NP_DTYPE, float16=np.float32)


class CudaError(RuntimeError):
    pass


class _ReadHandle:
    """Result of BackendCuda.read(): the promise of backend.ts:95-97."""

    def __init__(self, backend, event, host_ptr, nbytes, dtype, shape):
        self._b, self._ev, self._ptr, self._n = backend, event, host_ptr, nbytes
        self._dtype, self._shape = dtype, shape
        self._value = None

    def done(self):
        return self._value is not None or self._b._lib.tfjs_cuda_event_query(self._ev) == 1

    def result(self, timeout_ms=-1):
        if self._value is None:
            rc = self._b._lib.tfjs_cuda_event_wait(self._ev, timeout_ms)
            if rc != 0:
                raise CudaError(f"read failed with status {rc}")
            buf = (C.c_uint8 * self._n).from_address(self._ptr.value) if self._n else b""
            self._value = np.frombuffer(bytes(buf), dtype=self._dtype).reshape(-1).copy()
            self._b._lib.tfjs_cuda_event_destroy(self._ev)
            self._b._lib.tfjs_cuda_host_free(self._ptr)
        return self._value


class BackendCuda:
    """KernelBackend for one CUDA device.  `device` selects the GPU; one instance per GPU is
    how a batch is sharded (registered as 'cuda:0' ... 'cuda:7')."""

    def __init__(self, device=0, math_mode="3xtf32"):
        self._lib = _ffi.load()
        ctx = C.c_void_p()
        rc = self._lib.tfjs_cuda_ctx_create(int(device), C.byref(ctx))
        if rc != 0:
            msg = self._lib.tfjs_cuda_last_error(None).decode()
            raise CudaError(f"cuda backend initialisation failed ({rc}): {msg}")
        self._ctx = ctx
        self.device = int(device)
        self._data = weakref.WeakKeyDictionary()  # DataStorage (backend.ts:47-70): dataId -> record
        self.activation_storage = "float32"
        self._pending_storage = None
        self.setMathMode(math_mode)

    # ---- helpers -------------------------------------------------------------------------
    def _check(self, rc):
        if rc != 0:
            msg = self._lib.tfjs_cuda_last_error(self._ctx).decode()
            if rc == _ffi.ERR_UNSUPPORTED:
                raise NotImplementedError(msg)
            raise CudaError(f"[{rc}] {msg}")

    def _rec(self, data_id):
        rec = self._data.get(data_id)
        if rec is None:
            # DataStorage.get miss (backend.ts:52-57): the tensor lives on another backend;
            # the engine moves it here through host memory.
            ENGINE.moveData(self, data_id)
            rec = self._data[data_id]
        return rec

    def _id(self, t, want="float32"):
        """Device tensor id of `t`, converting when the stored dtype differs from the dtype
        the tensor claims (cast-up aliases share storage, backend_util.ts:50-54)."""
        rec = self._rec(t.dataId)
        if rec["dtype"] == want:
            return rec["id"], None
        tmp = self._new_id(t.shape, want)
        self._check(self._lib.tfjs_cuda_cast(self._ctx, rec["id"], tmp))
        return tmp, tmp

    def _new_id(self, shape, dtype):
        out = C.c_int64()
        self._check(self._lib.tfjs_cuda_tensor_register(self._ctx, C.byref(out), len(shape),
                                                        _ffi.shape_array(shape), _DTYPE_CODE[dtype]))
        return out.value

    def _free_tmp(self, *ids):
        for i in ids:
            if i is not None:
                self._lib.tfjs_cuda_tensor_dispose(self._ctx, i)

    def _out(self, shape, dtype="float32"):
        return Tensor.make(shape, {}, dtype, self)

    def _out_activation(self, shape, storage=None):
        """Output of a convolution: a float32 tensor whose storage follows the activation-storage
        mode (or `storage` when the caller names one)."""
        self._pending_storage = storage or self.activation_storage
        try:
            return Tensor.make(shape, {}, "float32", self)
        finally:
            self._pending_storage = None

    def _activation_id(self, t):
        """Device id of an activation operand for the kernels that read float32 and half storage
        alike; any other storage is converted to float32 first."""
        rec = self._rec(t.dataId)
        if rec["dtype"] in ("float32", "float16"):
            return rec["id"], None
        return self._id(t)

    @staticmethod
    def _assert_numeric(tensors, op):
        for t in tensors if isinstance(tensors, (list, tuple)) else [tensors]:
            if t is not None and t.dtype not in ("float32", "int32", "bool"):
                raise ValueError(f"{op}: cuda backend does not support {t.dtype} tensors")

    # ---- storage (backend.ts:92-126; CPU backend_cpu.ts:102-129, 199-254) ----------------
    def register(self, dataId, shape, dtype):
        if dataId in self._data:
            raise ValueError("Data buffer is already registered")  # backend_cpu.ts:119-121
        if dtype not in _DTYPE_CODE:
            raise ValueError(f"cuda backend does not support dtype {dtype}")
        storage = dtype
        if self._pending_storage == "float16" and dtype == "float32":
            storage = "float16"   # a float32 tensor stored as IEEE half (16-bit activation storage)
        self._data[dataId] = {"id": self._new_id(shape, storage), "dtype": storage,
                              "shape": list(shape)}

    def write(self, dataId, values):
        if values is None:
            raise ValueError("MathBackendCUDA.write(): values can not be null")
        rec = self._rec(dataId)
        # a quantised tensor is refilled with its raw bytes (e.g. the next batch of pixels)
        host_dtype = np.uint8 if rec.get("quantized") else _HOST_DTYPE[rec["dtype"]]
        arr = np.ascontiguousarray(np.asarray(values).reshape(-1), dtype=host_dtype)
        self._check(self._lib.tfjs_cuda_tensor_write(self._ctx, rec["id"], arr.ctypes.data_as(C.c_void_p),
                                                     arr.nbytes))

    def writeFromHostPointer(self, dataId, ptr, nbytes):
        """Extension: upload from caller-owned (pinned) host memory without a numpy copy."""
        rec = self._rec(dataId)
        self._check(self._lib.tfjs_cuda_tensor_write(self._ctx, rec["id"], ptr, nbytes))

    def writeAsync(self, dataId, ptr, nbytes):
        """Extension: upload from pinned host memory on the copy stream, overlapping the kernels
        enqueued next; consumers wait for it (pass the tensor to graphLaunch(inputs=...))."""
        rec = self._rec(dataId)
        self._check(self._lib.tfjs_cuda_tensor_write_async(self._ctx, rec["id"], ptr, nbytes))

    def readSync(self, dataId):
        rec = self._rec(dataId)
        n = size_from_shape(rec["shape"])
        out = np.empty(n, dtype=np.float32 if rec.get("quantized") else _HOST_DTYPE[rec["dtype"]])
        self._check(self._lib.tfjs_cuda_tensor_read(self._ctx, rec["id"], out.ctypes.data_as(C.c_void_p),
                                                    out.nbytes))
        return out

    def read(self, dataId):
        rec = self._rec(dataId)
        dtype = np.float32 if rec.get("quantized") else _HOST_DTYPE[rec["dtype"]]
        nbytes = size_from_shape(rec["shape"]) * np.dtype(dtype).itemsize
        host = C.c_void_p()
        if self._lib.tfjs_cuda_host_alloc(C.byref(host), nbytes) != 0:
            raise CudaError("pinned host allocation failed")
        ev = C.c_void_p()
        self._check(self._lib.tfjs_cuda_tensor_read_async(self._ctx, rec["id"], host, nbytes, C.byref(ev)))
        return _ReadHandle(self, ev, host, nbytes, dtype, rec["shape"])

    def disposeData(self, dataId):
        rec = self._data.pop(dataId, None)
        if rec is not None and self._ctx:
            self._lib.tfjs_cuda_tensor_dispose(self._ctx, rec["id"])

    def memory(self):
        st = _ffi.MemStats()
        self._check(self._lib.tfjs_cuda_ctx_memory(self._ctx, C.byref(st)))
        return {"unreliable": False, "numBytesInGPU": st.bytes_in_use,
                "numBytesInGPUAllocated": st.bytes_reserved, "numBuffersFree": st.num_buffers_cached,
                "numDeviceAllocs": st.num_device_allocs, "numDeviceTensors": st.num_tensors}

    def time(self, f):
        """backend.ts:92-94 / BackendTimingInfo: device time between two events around f()."""
        t0 = _time.perf_counter()
        self._check(self._lib.tfjs_cuda_ctx_time_begin(self._ctx))
        f()
        ms, n = C.c_float(), C.c_int64()
        self._check(self._lib.tfjs_cuda_ctx_time_end(self._ctx, C.byref(ms), C.byref(n)))
        return {"kernelMs": ms.value, "wallMs": (_time.perf_counter() - t0) * 1e3,
                "getExtraProfileInfo": lambda: f"{n.value} kernel launches"}

    def floatPrecision(self):
        """backend.ts:120-126: 16 while activations are stored as IEEE half, else 32."""
        return 16 if self.activation_storage == "float16" else 32

    def epsilon(self):
        return EPSILON_FLOAT32 if self.floatPrecision() == 32 else EPSILON_FLOAT16

    def dispose(self):
        if self._ctx:
            self._lib.tfjs_cuda_ctx_destroy(self._ctx)
            self._ctx = None
            self._data = weakref.WeakKeyDictionary()

    def fromPixels(self, pixels, numChannels):
        raise NotImplementedError("Not yet implemented.")

    # ---- options / diagnostics (extensions) ----------------------------------------------
    def setMathMode(self, mode):
        """'3xtf32' (default, float32-level accuracy) or 'tf32' (one tensor-core pass)."""
        self.math_mode = mode
        self._check(self._lib.tfjs_cuda_ctx_set_option(self._ctx, b"math_mode", float(_ffi.MATH[mode])))

    def setActivationStorage(self, storage):
        """Extension: 'float32' (default) or 'float16'.  With 'float16' the outputs of the
        convolution methods (fusedConv2d, fusedDepthwiseConv2D, fusedSeparableConv2d) are stored as
        IEEE half, which halves the bytes every layer moves; the arithmetic stays float32 /
        tf32 with float32 accumulation.  This is the reference's 16-bit precision class
        (floatPrecision() == 16, test tolerance 1e-1: test_util.ts:23-39)."""
        if storage not in ("float32", "float16"):
            raise ValueError("activation storage must be 'float32' or 'float16'")
        self.activation_storage = storage

    def setOption(self, key, value):
        self._check(self._lib.tfjs_cuda_ctx_set_option(self._ctx, key.encode(), float(value)))

    def sync(self, timeout_ms=-1):
        self._check(self._lib.tfjs_cuda_ctx_sync(self._ctx, int(timeout_ms)))

    def profileBegin(self, max_launches=4096):
        """Extension: start recording one device-time row per kernel launch."""
        self._check(self._lib.tfjs_cuda_profile_begin(self._ctx, int(max_launches)))

    def profileEnd(self):
        """Returns [(kernel name, milliseconds)] for every launch since profileBegin()."""
        n = C.c_int()
        self._check(self._lib.tfjs_cuda_profile_end(self._ctx, C.byref(n)))
        rows = []
        for i in range(n.value):
            name, ms = C.c_char_p(), C.c_float()
            self._check(self._lib.tfjs_cuda_profile_get(self._ctx, i, C.byref(name), C.byref(ms)))
            rows.append((name.value.decode(), ms.value))
        return rows

    def launchCount(self):
        return self._lib.tfjs_cuda_ctx_launch_count(self._ctx)

    def stream(self):
        return self._lib.tfjs_cuda_ctx_stream(self._ctx)

    def registerQuantized(self, shape, q, scale, min_):
        """Extension: a float32 tensor stored as uint8 affine-quantised bytes, w = q*scale + min
        (io/io_utils.ts:122-146).  Usable as the filter / b operand of the contractions and as a
        depthwise filter; readSync returns the dequantised float32 values."""
        q = np.ascontiguousarray(np.asarray(q).reshape(-1), dtype=np.uint8)
        if q.size != size_from_shape(shape):
            raise ValueError("quantised byte count does not match the shape")
        # The engine creates and tracks the tensor like any other backend output (Tensor.make
        # re-enters register(), which allocates a float32 buffer); that buffer is then swapped
        # for the uint8 storage, so that id, refcount, scopes and the tape all see a normal tensor.
        t = Tensor.make([int(s) for s in shape], {}, "float32", self)
        rec = self._data[t.dataId]
        out = C.c_int64()
        try:
            self._check(self._lib.tfjs_cuda_tensor_register_quantized(
                self._ctx, C.byref(out), len(shape), _ffi.shape_array(shape),
                q.ctypes.data_as(C.c_void_p), float(scale), float(min_)))
        except Exception:
            t.dispose()
            raise
        self._lib.tfjs_cuda_tensor_dispose(self._ctx, rec["id"])
        self._data[t.dataId] = {"id": out.value, "dtype": "float32", "shape": list(t.shape),
                                "quantized": True}
        return t

    # ---- fused epilogue marshalling ------------------------------------------------------
    @staticmethod
    def _is_channel_vector(t, channels):
        """True when `t` broadcasts along the inner-most axis only: a scalar, or [.., 1, C]."""
        if t.size == 1:
            return True
        return t.size == channels and t.shape[-1] == channels

    def _epilogue(self, bias, activation, prelu, channels):
        """Returns (Epilogue | None, temporaries, needs_compose).  `activation` is 'linear' |
        'relu' | 'prelu' (ops/fused_util.ts:20) or the extensions 'relu6' and ('clip', lo, hi)."""
        tmps = []
        epi = _ffi.Epilogue()
        clip = None
        if activation == "relu6":
            activation, clip = "clip", (0.0, 6.0)
        elif isinstance(activation, tuple):
            activation, clip = "clip", (float(activation[1]), float(activation[2]))
        if activation not in _ffi.ACT:
            raise ValueError(f"Activation {activation} has not been implemented for the cuda backend.")
        fusable = True
        if bias is not None and not self._is_channel_vector(bias, channels):
            fusable = False
        if activation == "prelu":
            if prelu is None:
                raise ValueError("prelu activation needs preluActivationWeights")
            if not self._is_channel_vector(prelu, channels):
                fusable = False
        if not fusable:
            return None, tmps, True
        if bias is not None:
            bid, tmp = self._id(bias)
            tmps.append(tmp)
            epi.bias, epi.bias_len = bid, bias.size
        epi.activation = _ffi.ACT[activation]
        if activation == "prelu":
            pid, tmp = self._id(prelu)
            tmps.append(tmp)
            epi.prelu, epi.prelu_len = pid, prelu.size
        if clip:
            epi.clip_lo, epi.clip_hi = clip
        return epi, tmps, False

    def _compose_epilogue(self, result, bias, activation, prelu):
        """The unfused order of MathBackendCPU (backend_cpu.ts:542-555, 1536-1550)."""
        if bias is not None:
            r2 = self.add(result, bias)
            result.dispose()
            result = r2
        if activation in (None, "linear"):
            return result
        if activation == "relu":
            r2 = self.relu(result)
        elif activation == "prelu":
            r2 = self.prelu(result, prelu)
        elif activation == "relu6":
            r2 = self.clip(result, 0.0, 6.0)
        elif isinstance(activation, tuple):
            r2 = self.clip(result, activation[1], activation[2])
        else:
            raise ValueError(f"Activation {activation} has not been implemented for the cuda backend.")
        result.dispose()
        return r2

    # ---- contractions --------------------------------------------------------------------
    def batchMatMul(self, a, b, transposeA, transposeB):
        return self.fusedBatchMatMul(a=a, b=b, transposeA=transposeA, transposeB=transposeB)

    def fusedBatchMatMul(self, a, b, transposeA=False, transposeB=False, bias=None, activation=None,
                         preluActivationWeights=None):
        """backend.ts:134-138; CPU backend_cpu.ts:542-555."""
        self._assert_numeric([a, b, bias], "matMul")
        batch = a.shape[0]
        M = a.shape[2] if transposeA else a.shape[1]
        N = b.shape[1] if transposeB else b.shape[2]
        epi, tmps, compose = self._epilogue(bias, activation, preluActivationWeights, N)
        aid, ta = self._id(a)
        bid, tb = self._id(b)
        out = self._out([batch, M, N])
        oid = self._rec(out.dataId)["id"]
        self._check(self._lib.tfjs_cuda_batch_matmul(
            self._ctx, aid, bid, oid, batch, a.shape[1], a.shape[2], b.shape[1], b.shape[2],
            int(bool(transposeA)), int(bool(transposeB)), C.byref(epi) if epi is not None else None))
        self._free_tmp(ta, tb, *tmps)
        if compose:
            out = self._compose_epilogue(out, bias, activation, preluActivationWeights)
        return out

    def conv2d(self, x, filter, convInfo):
        return self.fusedConv2d(x, filter, convInfo)

    def fusedConv2d(self, x, filter, convInfo, bias=None, activation=None, preluActivationWeights=None,
                    outputStorage=None):
        """backend.ts:414-418; CPU backend_cpu.ts:1536-1616.  `outputStorage` (extension) overrides
        the activation-storage mode for this result, e.g. 'float32' for a network's logits."""
        self._assert_numeric([x, filter, bias], "conv2d")
        epi, tmps, compose = self._epilogue(bias, activation, preluActivationWeights, convInfo.outChannels)
        xid, tx = self._activation_id(x)
        fid, tf_ = self._id(filter)
        out = self._out_activation(convInfo.outShape, outputStorage)
        oid = self._rec(out.dataId)["id"]
        self._check(self._lib.tfjs_cuda_conv2d(self._ctx, xid, fid, oid, C.byref(convInfo),
                                               C.byref(epi) if epi is not None else None))
        self._free_tmp(tx, tf_, *tmps)
        if compose:
            out = self._compose_epilogue(out, bias, activation, preluActivationWeights)
        return out

    def depthwiseConv2D(self, x, filter, convInfo):
        """backend.ts:431-434; CPU backend_cpu.ts:1979-2035."""
        return self.fusedDepthwiseConv2D(x, filter, convInfo)

    def fusedDepthwiseConv2D(self, x, filter, convInfo, bias=None, activation=None):
        """Extension: depthwiseConv2D + add(bias) + activation in one kernel."""
        self._assert_numeric([x, filter, bias], "depthwiseConv2D")
        epi, tmps, compose = self._epilogue(bias, activation, None, convInfo.outChannels)
        xid, tx = self._activation_id(x)
        fid, tf_ = self._id(filter)
        out = self._out_activation(convInfo.outShape)
        oid = self._rec(out.dataId)["id"]
        self._check(self._lib.tfjs_cuda_depthwise_conv2d(self._ctx, xid, fid, oid, C.byref(convInfo),
                                                         C.byref(epi) if epi is not None else None))
        self._free_tmp(tx, tf_, *tmps)
        if compose:
            out = self._compose_epilogue(out, bias, activation, None)
        return out

    def fusedSeparableConv2d(self, x, depthwiseFilter, pointwiseFilter, convInfo, dwBias=None,
                             dwActivation=None, pwBias=None, pwActivation=None):
        """Extension: tf.separableConv2d's op pair (ops/conv.ts:574-654) with bias + activation
        after each half, `convInfo` being the depthwise Conv2DInfo and pointwiseFilter
        [1, 1, convInfo.outChannels, outDepth].  Eligible shapes run as one kernel that never
        writes the depthwise result to device memory; results equal the two separate calls."""
        self._assert_numeric([x, depthwiseFilter, pointwiseFilter, dwBias, pwBias], "separableConv2d")
        out_depth = pointwiseFilter.shape[3]
        if pointwiseFilter.shape[:3] != [1, 1, convInfo.outChannels]:
            raise ValueError(
                f"Error in separableConv2d: the third dimension of pointwise filter must be "
                f"{convInfo.outChannels}, but got {pointwiseFilter.shape[2]}.")
        dw_epi, tmps1, compose1 = self._epilogue(dwBias, dwActivation, None, convInfo.outChannels)
        pw_epi, tmps2, compose2 = self._epilogue(pwBias, pwActivation, None, out_depth)
        if compose1 or compose2:
            # a bias that is not a channel vector: the two-call form handles the broadcast
            self._free_tmp(*tmps1, *tmps2)
            mid = self.fusedDepthwiseConv2D(x, depthwiseFilter, convInfo, dwBias, dwActivation)
            from . import conv_util
            ci = conv_util.compute_conv2d_info(mid.shape, pointwiseFilter.shape, 1, 1, "valid")
            out = self.fusedConv2d(mid, pointwiseFilter, ci, pwBias, pwActivation)
            mid.dispose()
            return out
        xid, tx = self._activation_id(x)
        did, td = self._id(depthwiseFilter)
        pid, tp = self._id(pointwiseFilter)
        out = self._out_activation([convInfo.batchSize, convInfo.outHeight, convInfo.outWidth, out_depth])
        oid = self._rec(out.dataId)["id"]
        self._check(self._lib.tfjs_cuda_separable_conv2d(
            self._ctx, xid, did, pid, oid, C.byref(convInfo), int(out_depth), C.byref(dw_epi), C.byref(pw_epi)))
        self._free_tmp(tx, td, tp, *tmps1, *tmps2)
        return out

    # ---- pooling -------------------------------------------------------------------------
    def _pool(self, x, convInfo, is_avg):
        self._assert_numeric(x, "pool")
        xid, tx = self._activation_id(x)
        out = self._out(convInfo.outShape)
        self._check(self._lib.tfjs_cuda_pool2d(self._ctx, xid, self._rec(out.dataId)["id"],
                                               C.byref(convInfo), int(is_avg)))
        self._free_tmp(tx)
        return out

    def maxPool(self, x, convInfo):
        return self._pool(x, convInfo, False)

    def avgPool(self, x, convInfo):
        return self._pool(x, convInfo, True)

    # ---- element-wise --------------------------------------------------------------------
    def _binary(self, op, a, b, out_dtype="float32"):
        self._assert_numeric([a, b], op)
        shape = assert_and_get_broadcast_shape(a.shape, b.shape)
        aid, ta = self._id(a)
        bid, tb = self._id(b)
        out = self._out(shape, out_dtype)
        self._check(self._lib.tfjs_cuda_binary(
            self._ctx, _ffi.BINARY[op], aid, len(a.shape), _ffi.shape_array(a.shape), bid,
            len(b.shape), _ffi.shape_array(b.shape), self._rec(out.dataId)["id"]))
        self._free_tmp(ta, tb)
        return out

    def add(self, a, b):
        return self._binary("add", a, b)

    def subtract(self, a, b):
        return self._binary("sub", a, b)

    def multiply(self, a, b):
        return self._binary("mul", a, b)

    def realDivide(self, a, b):
        return self._binary("div", a, b)

    def prelu(self, x, a):
        return self._binary("prelu", x, a)

    def notEqual(self, a, b):
        return self._binary("notEqual", a, b, "bool")

    def _unary(self, op, x, p0=0.0, p1=0.0, out_dtype="float32"):
        self._assert_numeric(x, op)
        xid, tx = self._id(x)
        out = self._out(x.shape, out_dtype)
        self._check(self._lib.tfjs_cuda_unary(self._ctx, _ffi.UNARY[op], xid, self._rec(out.dataId)["id"],
                                              float(p0), float(p1)))
        self._free_tmp(tx)
        return out

    def relu(self, x):
        return self._unary("relu", x)

    def clip(self, x, min, max):
        return self._unary("clip", x, min, max)

    def exp(self, x):
        return self._unary("exp", x)

    def log(self, x):
        return self._unary("log", x)

    def int(self, x):
        return self._unary("int", x, out_dtype="int32")

    def step(self, x, alpha=0.0):
        """backend.ts:401; CPU backend_cpu.ts:1520-1534 (the gradient of relu)."""
        return self._unary("step", x, alpha)

    # ---- gradient kernels (backend.ts:424-442, 456-466, 216) ------------------------------
    def _conv_gradient(self, fn, first, second, out_shape, convInfo, name):
        self._assert_numeric([first, second], name)
        aid, ta = self._id(first)
        bid, tb = self._id(second)
        out = self._out(out_shape)
        self._check(fn(self._ctx, aid, bid, self._rec(out.dataId)["id"], C.byref(convInfo)))
        self._free_tmp(ta, tb)
        return out

    def conv2dDerInput(self, dy, filter, convInfo):
        return self._conv_gradient(self._lib.tfjs_cuda_conv2d_der_input, dy, filter, convInfo.inShape,
                                   convInfo, "conv2dDerInput")

    def conv2dDerFilter(self, x, dy, convInfo):
        shape = [convInfo.filterHeight, convInfo.filterWidth, convInfo.inChannels, convInfo.outChannels]
        return self._conv_gradient(self._lib.tfjs_cuda_conv2d_der_filter, x, dy, shape, convInfo,
                                   "conv2dDerFilter")

    def depthwiseConv2DDerInput(self, dy, filter, convInfo):
        return self._conv_gradient(self._lib.tfjs_cuda_depthwise_conv2d_der_input, dy, filter,
                                   convInfo.inShape, convInfo, "depthwiseConv2DDerInput")

    def depthwiseConv2DDerFilter(self, x, dy, convInfo):
        shape = [convInfo.filterHeight, convInfo.filterWidth, convInfo.inChannels,
                 convInfo.outChannels // max(convInfo.inChannels, 1)]
        return self._conv_gradient(self._lib.tfjs_cuda_depthwise_conv2d_der_filter, x, dy, shape, convInfo,
                                   "depthwiseConv2DDerFilter")

    def _pool_backprop(self, dy, x, convInfo, is_avg):
        self._assert_numeric([dy, x], "poolBackprop")
        did, td = self._id(dy)
        xid, tx = self._id(x)
        out = self._out(x.shape)
        self._check(self._lib.tfjs_cuda_pool2d_backprop(self._ctx, did, xid, self._rec(out.dataId)["id"],
                                                        C.byref(convInfo), int(is_avg)))
        self._free_tmp(td, tx)
        return out

    def maxPoolBackprop(self, dy, x, y, convInfo):
        return self._pool_backprop(dy, x, convInfo, False)

    def avgPoolBackprop(self, dy, x, convInfo):
        return self._pool_backprop(dy, x, convInfo, True)

    def clipBackprop(self, dy, x, lo, hi):
        """Extension: dy where lo <= x <= hi, else 0 (the gradient of clip as one kernel)."""
        self._assert_numeric([dy, x], "clipBackprop")
        did, td = self._id(dy)
        xid, tx = self._id(x)
        out = self._out(x.shape)
        self._check(self._lib.tfjs_cuda_clip_backprop(self._ctx, did, xid, self._rec(out.dataId)["id"],
                                                      float(lo), float(hi)))
        self._free_tmp(td, tx)
        return out

    def transpose(self, x, perm):
        self._assert_numeric(x, "transpose")
        xid, tx = self._id(x)
        out = self._out([x.shape[p] for p in perm])
        perm_arr = (C.c_int32 * max(len(perm), 1))(*[int(p) for p in perm])
        self._check(self._lib.tfjs_cuda_transpose(self._ctx, xid, self._rec(out.dataId)["id"], len(perm),
                                                  _ffi.shape_array(x.shape), perm_arr))
        self._free_tmp(tx)
        return out

    # ---- reductions over the inner-most axes (backend.ts:183, 198, 255) ------------------
    def _reduce(self, op, x, axes, out_dtype):
        self._assert_numeric(x, op)
        rank = len(x.shape)
        axes = sorted(a % rank if rank else 0 for a in axes)
        if axes != list(range(rank - len(axes), rank)):
            # axis_util.ts assertAxesAreInnerMostDims
            raise ValueError(f"{op} requires inner-most axes; got axes {axes} and rank-{rank} input")
        out_shape = x.shape[:rank - len(axes)]
        inner = size_from_shape(x.shape[rank - len(axes):])
        outer = size_from_shape(out_shape)
        xid, tx = self._id(x)
        out = self._out(out_shape, out_dtype)
        self._check(self._lib.tfjs_cuda_reduce_last(self._ctx, _ffi.REDUCE[op], xid,
                                                    self._rec(out.dataId)["id"], outer, inner))
        self._free_tmp(tx)
        return out

    def sum(self, x, axes):
        return self._reduce("sum", x, axes, "float32")

    def max(self, x, axes):
        return self._reduce("max", x, axes, "float32")

    def argMax(self, x, axis):
        return self._reduce("argMax", x, [axis], "int32")

    def softmax(self, logits):
        """Extension: tf.softmax over the last axis in one kernel (same per-stage rounding as
        the op-layer chain max, sub, exp, sum, log, add, sub, exp)."""
        self._assert_numeric(logits, "softmax")
        inner = logits.shape[-1] if logits.shape else 1
        outer = logits.size // inner if inner else 0
        xid, tx = self._id(logits)
        out = self._out(logits.shape)
        self._check(self._lib.tfjs_cuda_softmax_last(self._ctx, xid, self._rec(out.dataId)["id"],
                                                     outer, inner))
        self._free_tmp(tx)
        return out

    # ---- metadata ops (backend.ts:480-486; backend_util.ts:36-76) ------------------------
    def reshape(self, x, shape):
        """Free: a new Tensor sharing the dataId (backend_util.reshapeTensor)."""
        return Tensor.make(shape, {"dataId": x.dataId}, x.dtype)

    def cast(self, x, dtype):
        """backend_util.castTensor: up-casts alias the storage, float->int32 goes through
        int(), ->bool through notEqual(x, 0)."""
        if dtype == x.dtype:
            return Tensor.make(x.shape, {"dataId": x.dataId}, x.dtype)
        order = {"bool": 0, "int32": 1, "float32": 2}
        if order[dtype] > order[x.dtype]:
            return Tensor.make(x.shape, {"dataId": x.dataId}, dtype)
        if dtype == "int32":
            return self.int(x)
        zero = Tensor([], x.dtype, np.zeros(1, NP_DTYPE[x.dtype]), backend=self)
        out = self.notEqual(x, zero)
        zero.dispose()
        return out

    # ---- CUDA graph capture (extension) --------------------------------------------------
    def graphBegin(self):
        self._check(self._lib.tfjs_cuda_graph_begin(self._ctx))

    def graphEnd(self):
        g = C.c_void_p()
        self._check(self._lib.tfjs_cuda_graph_end(self._ctx, C.byref(g)))
        return g

    def graphLaunch(self, graph, inputs=()):
        """Replays a captured graph.  `inputs`: tensors the graph reads that may have an
        asynchronous upload (writeAsync) in flight; the replay is ordered after those uploads."""
        for t in inputs:
            self._check(self._lib.tfjs_cuda_tensor_wait(self._ctx, self._rec(t.dataId)["id"]))
        self._check(self._lib.tfjs_cuda_graph_launch(self._ctx, graph))

    def graphDestroy(self, graph):
        self._lib.tfjs_cuda_graph_destroy(self._ctx, graph)


def assert_and_get_broadcast_shape(shape_a, shape_b):
    """ops/broadcast_util.ts:58-87."""
    result = []
    la, lb = len(shape_a), len(shape_b)
    for i in range(max(la, lb)):
        a = shape_a[la - i - 1] if i < la else 1
        b = shape_b[lb - i - 1] if i < lb else 1
        if a == 1:
            result.insert(0, b)
        elif b == 1:
            result.insert(0, a)
        elif a != b:
            raise ValueError(f"Operands could not be broadcast together with shapes "
                             f"{list(shape_a)} and {list(shape_b)}.")
        else:
            result.insert(0, a)
    return result
