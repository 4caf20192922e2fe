"""CPU-only tests of the host side: op-layer shape arithmetic, the engine stand-in's backend
registry and tensor bookkeeping (with fake backends, as tfjs-core/src/engine_test.ts:25-305 does
with TestKernelBackend), and the C-ABI library's exports.  No compute call needs a GPU."""
import ctypes
import os
import re
import warnings

import numpy as np
import pytest

import oracle
import tfjs_core_b200 as tf
from tfjs_core_b200 import _ffi, conv_util, mobilenet
from tfjs_core_b200.engine import Engine, Tensor

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


# ---- conv_util ----------------------------------------------------------------------------------
def test_conv_info_matches_oracle_on_random_geometry():
    rng = np.random.Generator(np.random.PCG64(0))
    fields = [n for n, _ in _ffi.ConvInfo._fields_]
    for _ in range(500):
        in_shape = [int(rng.integers(1, 4)), int(rng.integers(1, 40)), int(rng.integers(1, 40)), int(rng.integers(1, 9))]
        f = [int(rng.integers(1, 6)), int(rng.integers(1, 6)), in_shape[3], int(rng.integers(1, 5))]
        stride = [int(rng.integers(1, 4)), int(rng.integers(1, 4))]
        dil = [int(rng.integers(1, 3)), int(rng.integers(1, 3))]
        pad = ["same", "valid"][int(rng.integers(0, 2))]
        dw = bool(rng.integers(0, 2))
        a = conv_util.compute_conv2d_info(in_shape, f, stride, dil, pad, None, dw)
        b = oracle.compute_conv2d_info(in_shape, f, stride, dil, pad, None, dw)
        if b.outHeight < 0 or b.outWidth < 0:
            continue
        for n in fields:
            assert getattr(a, n) == getattr(b, n), (n, in_shape, f, stride, dil, pad)


def test_conv_info_reference_cases():
    # ops/conv_util_test.ts:82-99: 3x3 stride 2 'same' on an odd-sized input
    ci = conv_util.compute_conv2d_info([1, 5, 5, 3], [3, 3, 3, 7], 2, 1, "same")
    assert ci.outShape == [1, 3, 3, 7] and (ci.padTop, ci.padBottom, ci.padLeft, ci.padRight) == (1, 1, 1, 1)
    # even input: padding is asymmetric, bottom/right only
    ci = conv_util.compute_conv2d_info([64, 224, 224, 3], [3, 3, 3, 32], 2, 1, "same")
    assert ci.outShape == [64, 112, 112, 32] and (ci.padTop, ci.padBottom, ci.padLeft, ci.padRight) == (0, 1, 0, 1)
    # depthwise out channels = chMul * inChannels (conv_util.ts:151)
    ci = conv_util.compute_conv2d_info([1, 8, 8, 4], [3, 3, 4, 2], 1, 1, "valid", None, True)
    assert ci.outChannels == 8 and ci.outShape == [1, 6, 6, 8]
    # numeric pad with rounding (pool_test.ts:104-110)
    ci = conv_util.compute_pool2d_info([1, 2, 2, 3], 1, 2, 1, 1, "floor")
    assert ci.outShape == [1, 2, 2, 3]
    with pytest.raises(ValueError):
        conv_util.compute_conv2d_info([1, 4, 4, 1], [2, 2, 1, 1], 3, 1, 1)  # non-integer output
    # dilation enlarges the effective filter (conv_util.ts:391-397)
    ci = conv_util.compute_conv2d_info([1, 9, 9, 1], [3, 3, 1, 1], 1, 2, "valid")
    assert (ci.effectiveFilterHeight, ci.outHeight) == (5, 5)


def test_mobilenet_accounting_matches_layer_table():
    # fp32, fused epilogues, every tensor once: 41.228 MB per image, 16.88 MB of weights,
    # 1.1375 GFLOP per image
    assert mobilenet.algorithmic_bytes_per_image() * 64 + mobilenet.weight_bytes() == 2638567840
    assert mobilenet.weight_bytes() == 16884128
    assert mobilenet.flops_per_image() == 1137530880
    # per-launch accounting: the layer-wise forward has 30 launches; with four depthwise +
    # pointwise pairs fused (the accounting of this example; the default forward fuses five) there
    # are 26, and the four intermediates (1.6 + 0.8 + 1.6 + 0.4 MB per image, written once and read
    # once) drop out of the byte count
    layerwise = mobilenet.layer_algorithmic_bytes(64, True)
    names = (["conv2d_tcgen05 (3-channel 3x3, window TMA, TF32)"] +
             ["separableConv2d (fused dw3x3 s1 + pw, TF32)"] * 4 +
             ["depthwiseConv2D (3x3 strip)", "gemm_tcgen05 (TF32)"] * 9 +
             ["avgPool (global)", "gemm_tcgen05 (TF32)", "softmax_last"])
    fused = mobilenet.launch_algorithmic_bytes(64, True, names)
    assert len(layerwise) == 30 and len(fused) == 26
    mid = 4 * 64 * (112 * 112 * 32 + 56 * 56 * 64 + 56 * 56 * 128 + 28 * 28 * 128)
    assert sum(layerwise) - sum(fused) == 2 * mid
    with pytest.raises(AssertionError):
        mobilenet.launch_algorithmic_bytes(64, True, names[:-1])
    specs = mobilenet.layer_specs()
    assert len(specs) == 28 and specs[0][2] == (3, 3, 3, 32) and specs[-1][2] == (1, 1, 1024, 1000)


def test_synthetic_weights_are_seeded():
    a = mobilenet.make_weights(4, quantized=True)
    b = mobilenet.make_weights(4, quantized=True)
    assert all(np.array_equal(a[k]["q"], b[k]["q"]) and a[k]["scale"] == b[k]["scale"] for k in a)
    assert all(abs(a[k]["min"] + 128 * a[k]["scale"]) < 1e-12 for k in a)
    assert a["pw13"]["q"].dtype == np.uint8 and a["pw13"]["q"].shape == (1, 1, 1024, 1024)


# ---- engine stand-in with fake backends -----------------------------------------------------------
class FakeBackend:
    def __init__(self):
        self.data = {}
        self.disposed = False

    def register(self, data_id, shape, dtype):
        if data_id in self.data:
            raise ValueError("Data buffer is already registered")
        self.data[data_id] = None

    def write(self, data_id, values):
        self.data[data_id] = np.array(values)

    def readSync(self, data_id):
        return self.data[data_id]

    def disposeData(self, data_id):
        self.data.pop(data_id, None)

    def memory(self):
        return {"unreliable": True}

    def dispose(self):
        self.disposed = True


def test_backend_registry_priority_and_fallback():
    e = Engine()
    assert e.registerBackend("low", FakeBackend, 1)
    assert e.registerBackend("high", FakeBackend, 5)

    def failing():
        raise RuntimeError("no device")
    assert e.registerBackend("broken", failing, 100)
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        assert e.registerBackend("low", FakeBackend, 9) is False      # engine.ts:221-226
        name, inst = e.initializeBackendsAndReturnBest()               # engine.ts:334-359
    assert name == "high" and isinstance(inst, FakeBackend)
    assert any("already registered" in str(x.message) for x in w)
    assert any("Initialization of backend broken failed" in str(x.message) for x in w)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        assert e.setBackend("broken") is False
    assert e.setBackend("low") and e.backendName == "low"
    with pytest.raises(ValueError):
        e.setBackend("missing")
    e.removeBackend("low")
    assert e.findBackend("low") is None


def test_cuda_backend_fails_loudly_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(tf.CudaError):
        tf.BackendCuda(0)


def test_tensor_refcounts_scopes_and_cross_backend_move(monkeypatch):
    import tfjs_core_b200.engine as eng
    e = Engine()
    b1, b2 = FakeBackend(), FakeBackend()
    e.registerBackend("cpu1", lambda: b1, 1)
    e.registerBackend("cpu2", lambda: b2, 1)
    e.setBackend("cpu1")
    monkeypatch.setattr(eng, "ENGINE", e)
    t = Tensor([2], "float32", np.array([1, 2], np.float32))
    alias = Tensor.make([2, 1], {"dataId": t.dataId}, "float32")    # reshape: shares the dataId
    assert e.numTensors == 2 and e.numDataBuffers == 1 and len(b1.data) == 1
    t.dispose()
    assert e.numDataBuffers == 1 and len(b1.data) == 1                # still referenced
    assert np.array_equal(alias.dataSync(), [1, 2])
    e.moveData(b2, alias.dataId)                                       # engine.ts:361-363
    assert len(b1.data) == 0 and np.array_equal(b2.data[alias.dataId], [1, 2])
    alias.dispose()
    assert e.numTensors == 0 and e.numDataBuffers == 0 and e.numBytes == 0 and len(b2.data) == 0
    kept = e.tidy(lambda: [Tensor([1], "float32", [1.0]), Tensor([1], "float32", [2.0])][1])
    assert e.numTensors == 1 and not kept.isDisposed


# ---- the C-ABI library ------------------------------------------------------------------------------
def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "tfjs_cuda.h")).read()
    declared = set(re.findall(r"\b(tfjs_cuda_[a-z0-9_]+)\s*\(", header))
    declared -= {"tfjs_cuda_status"}
    assert len(declared) >= 38
    lib = ctypes.CDLL(_ffi.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in tfjs_cuda.h but not exported"
    assert declared == set(_ffi.SIGNATURES), declared ^ set(_ffi.SIGNATURES)


def test_struct_layouts_match_the_header():
    assert ctypes.sizeof(_ffi.ConvInfo) == 19 * 4
    assert ctypes.sizeof(_ffi.Epilogue) == 48 and _ffi.Epilogue.activation.offset == 16
    assert _ffi.Epilogue.prelu.offset == 24 and _ffi.Epilogue.clip_lo.offset == 40
    assert ctypes.sizeof(_ffi.MemStats) == 40
    assert ctypes.sizeof(oracle.ConvInfo) == ctypes.sizeof(_ffi.ConvInfo)


def test_context_creation_reports_errors_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib = _ffi.load()
    ctx = ctypes.c_void_p()
    rc = lib.tfjs_cuda_ctx_create(0, ctypes.byref(ctx))
    assert rc == _ffi.ERR_CUDA and not ctx.value
    assert b"CUDA device" in lib.tfjs_cuda_last_error(None)


def test_bench_groups_every_hot_path_kernel_name_into_a_family():
    """bench.py reports per-family times (`kernels{}`, `roofline.kernel`) by the names the library
    gives its launches: every name of a kernel on the inference path that the sources can report
    must be in its table, or a new variant would show up as a family of its own."""
    import importlib.util
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_for_test", os.path.join(root, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    names = set()
    csrc = os.path.join(root, "tfjs-core_b200", "csrc")
    for fn in os.listdir(csrc):
        text = open(os.path.join(csrc, fn)).read()
        names.update(re.findall(r'"((?:gemm_tcgen05|conv2d_tcgen05|separableConv2d|depthwiseConv2D \(3x3|avgPool \(global|softmax_last)[^"]*)"', text))
    names = {n for n in names if "(" in n}   # kernel names carry their variant in parentheses; error texts do not
    assert len(names) >= 20, names
    missing = sorted(n for n in names if n not in bench.KERNEL_FAMILY)
    assert not missing, missing
