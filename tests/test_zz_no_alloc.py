"""tfjs_cuda_matmul_static_scratch, the matMul entry point for callers that may not allocate.

Some hosts of this library are not allowed to obtain device memory while they run: a serving
loop whose buffers were all sized at start-up, or a plugin that a framework hands raw device
pointers and whose pool it must leave alone.  For them the library offers one matMul variant
whose only scratch (the repacked b operand) is a fixed array inside the library image.  This
file checks, through the C ABI, that the variant returns what the regular entry point returns,
on two calls in a row with different operands (the shared array still holds the first call's
data when the second starts), that the calls leave the context's allocator untouched, and that
operands beyond the fixed size are refused with an explanation.

The file name sorts last on purpose: a run that stops at the first failure has then already
exercised every other test.
"""
import ctypes as C

import numpy as np
import pytest

from gpu_util import rel_err, tf  # noqa: F401
from tfjs_core_b200 import _ffi

pytestmark = pytest.mark.gpu


def _device_ptr(bk, tensor):
    ptr, nbytes = C.c_void_p(), C.c_size_t()
    rc = bk._lib.tfjs_cuda_tensor_device_ptr(bk._ctx, bk._rec(tensor.dataId)["id"], C.byref(ptr), C.byref(nbytes))
    assert rc == 0
    return ptr


def _both_ways(tf, m, k, n, seed, activation):
    """Returns (regular entry point's result, static-scratch entry point's result)."""
    bk = tf.ENGINE.backend
    rng = np.random.Generator(np.random.PCG64(seed))
    a = rng.uniform(-1, 1, (1, m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (1, k, n)).astype(np.float32)
    bias = rng.normal(0, 1, n).astype(np.float32)
    ta, tb, tbias = tf.ops.tensor(a), tf.ops.tensor(b), tf.ops.tensor(bias)
    want = bk.fusedBatchMatMul(a=ta, b=tb, bias=tbias, activation=activation)
    out = tf.ops.tensor(np.full((m, n), np.nan, np.float32))     # the caller owns the output buffer
    allocs_before = bk.memory()["numDeviceAllocs"]
    tensors_before = bk.memory()["numDeviceTensors"]
    act = {"linear": 0, "relu": 1, "relu6": 3}[activation]
    rc = bk._lib.tfjs_cuda_matmul_static_scratch(
        bk._ctx, _device_ptr(bk, ta), _device_ptr(bk, tb), _device_ptr(bk, tbias), _device_ptr(bk, out),
        m, k, n, act, 0.0, 6.0)
    assert rc == 0, bk._lib.tfjs_cuda_last_error(bk._ctx).decode()
    got = out.dataSync().reshape(m, n)
    after = bk.memory()
    assert after["numDeviceAllocs"] == allocs_before and after["numDeviceTensors"] == tensors_before
    return want.dataSync().reshape(m, n), got


def test_static_scratch_matmul_matches_regular_entry_point_twice(tf):
    # Both entry points run the same two kernels (repack b, tensor-core GEMM) on the same values,
    # so the results must agree bit for bit, not merely within a tolerance.
    # first call: a 1024-wide b fills the whole fixed array
    want, got = _both_ways(tf, 256, 1024, 1024, seed=1, activation="relu")
    assert np.array_equal(got, want)
    # second call straight after, smaller operands with a ragged tile edge: the array still
    # holds the first call's planes and must not leak into this result
    want, got = _both_ways(tf, 130, 68, 72, seed=2, activation="relu6")
    assert np.array_equal(got, want)
    assert np.isfinite(got).all()
    # and against the CPU oracle, so that the pair is not merely self-consistent
    import oracle
    rng = np.random.Generator(np.random.PCG64(2))
    a = rng.uniform(-1, 1, (1, 130, 68)).astype(np.float32)
    b = rng.uniform(-1, 1, (1, 68, 72)).astype(np.float32)
    bias = rng.normal(0, 1, 72).astype(np.float32)
    ref = oracle.unary("clip", oracle.fused_matmul(a, b, bias=bias)[0], 0.0, 6.0)
    assert rel_err(got, ref) <= 1e-5


def test_static_scratch_matmul_in_tf32_mode(tf):
    """The entry point follows the context's math mode: one tensor-core pass on operands rounded
    to tf32, again identical to the regular entry point and within 1e-3 of the oracle."""
    import oracle
    bk = tf.ENGINE.backend
    bk.setMathMode("tf32")
    try:
        want, got = _both_ways(tf, 200, 96, 64, seed=3, activation="linear")
        assert np.array_equal(got, want)
        rng = np.random.Generator(np.random.PCG64(3))
        a = rng.uniform(-1, 1, (1, 200, 96)).astype(np.float32)
        b = rng.uniform(-1, 1, (1, 96, 64)).astype(np.float32)
        bias = rng.normal(0, 1, 64).astype(np.float32)
        assert rel_err(got, oracle.fused_matmul(a, b, bias=bias)[0]) <= 1e-3
    finally:
        bk.setMathMode("3xtf32")


def test_static_scratch_matmul_refuses_oversized_operands(tf):
    bk = tf.ENGINE.backend
    a = tf.ops.tensor(np.zeros((8, 2048), np.float32))
    b = tf.ops.tensor(np.zeros((2048, 1024), np.float32))
    out = tf.ops.tensor(np.zeros((8, 1024), np.float32))
    rc = bk._lib.tfjs_cuda_matmul_static_scratch(
        bk._ctx, _device_ptr(bk, a), _device_ptr(bk, b), None, _device_ptr(bk, out), 8, 2048, 1024, 0, 0.0, 0.0)
    assert rc == _ffi.ERR_INVALID_ARG
    assert "limit" in bk._lib.tfjs_cuda_last_error(bk._ctx).decode()
