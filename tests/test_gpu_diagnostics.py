"""Failure detection without a GPU fault: the bounded device-side waits and the allocator's
guard patterns.  Neither test traps, faults or hangs the device: the wait is made to run out by
withholding a load on the host's request (nothing is left in flight, the kernel returns by
itself after the configured limit), and the buffer overrun stays inside the allocation."""
import ctypes as C

import numpy as np
import pytest

import oracle
from gpu_util import rel_err, tf  # noqa: F401
from tfjs_core_b200 import _ffi
from tfjs_core_b200.backend_cuda import CudaError

pytestmark = pytest.mark.gpu


def _matmul(tf, a, b):
    out = tf.ENGINE.backend.fusedBatchMatMul(tf.ops.tensor(a), tf.ops.tensor(b))
    return out


@pytest.mark.parametrize("mode", ["tf32", "3xtf32"])
def test_bounded_wait_reports_timeout_and_context_survives(tf, mode):
    """Every mbarrier wait of the tensor-core kernels is bounded.  With the last load withheld the
    consumers' wait runs out after the limit (2 ms here), the kernel frees its tensor memory and
    returns, the next synchronisation reports TFJS_CUDA_ERR_TIMEOUT, and the context goes on
    working."""
    bk = tf.ENGINE.backend
    rng = np.random.Generator(np.random.PCG64(5))
    a = rng.uniform(-1, 1, (1, 128, 64)).astype(np.float32)
    b = rng.uniform(-1, 1, (1, 64, 32)).astype(np.float32)
    bk.setMathMode(mode)
    warm = _matmul(tf, a, b)           # prepares b's tensor-core layout
    warm.dataSync()
    bk.setOption("wait_limit_us", 2000)
    bk.setOption("test_withhold_last_load", 1)
    try:
        broken = _matmul(tf, a, b)
        with pytest.raises(CudaError, match=r"\[-4\].*bounded wait"):
            bk.sync()
        broken.dispose()
    finally:
        bk.setOption("test_withhold_last_load", 0)
        bk.setOption("wait_limit_us", 2_000_000)
        bk.setMathMode("3xtf32")
    bk.sync()                          # the status word was cleared: no stale error
    bk.setMathMode(mode)
    try:
        good = _matmul(tf, a, b).dataSync().reshape(128, 32)
    finally:
        bk.setMathMode("3xtf32")
    assert np.array_equal(good, warm.dataSync().reshape(128, 32))
    assert rel_err(good, oracle.batch_matmul(a, b)[0]) <= (1e-3 if mode == "tf32" else 1e-5)


@pytest.mark.parametrize("mode", ["tf32", "3xtf32"])
def test_bounded_wait_on_cta_pairs(tf, mode):
    """The same on the CTA-pair kernel, whose two CTAs wait on each other's barriers: with the last
    loads of both producers withheld, every role of both CTAs gives up within the limit, both take
    part in the closing cluster barrier, the pair frees its tensor memory, and the context goes on
    working (tf32: the variant whose converter warps round A; 3xtf32: the split variant)."""
    bk = tf.ENGINE.backend
    rng = np.random.Generator(np.random.PCG64(6))
    a = rng.uniform(-1, 1, (1, 300, 512)).astype(np.float32)
    b = (rng.uniform(-1, 1, (1, 512, 256)) / 22.0).astype(np.float32)
    bk.setMathMode(mode)
    bk.setOption("gemm_pair", 2)
    try:
        bk.profileBegin(8)
        warm = _matmul(tf, a, b)
        want = warm.dataSync().reshape(300, 256)
        assert any("CTA pairs" in name for name, _ in bk.profileEnd())
        bk.setOption("wait_limit_us", 2000)
        bk.setOption("test_withhold_last_load", 1)
        try:
            broken = _matmul(tf, a, b)
            with pytest.raises(CudaError, match=r"\[-4\].*bounded wait"):
                bk.sync()
            broken.dispose()
        finally:
            bk.setOption("test_withhold_last_load", 0)
            bk.setOption("wait_limit_us", 2_000_000)
        bk.sync()
        good = _matmul(tf, a, b).dataSync().reshape(300, 256)
        assert np.array_equal(good, want)
        assert rel_err(good, oracle.batch_matmul(a, b)[0]) <= (1e-3 if mode == "tf32" else 1e-5)
    finally:
        bk.setOption("gemm_pair", 1)
        bk.setMathMode("3xtf32")


def test_wait_limit_bounds_are_checked(tf):
    bk = tf.ENGINE.backend
    with pytest.raises(CudaError, match="wait_limit_us"):
        bk.setOption("wait_limit_us", 1)


def test_guard_pattern_detects_a_write_past_the_end(tf):
    """Option debug_canary: a kernel that writes beyond the end of its output buffer is reported
    when the buffer is released.  The overrun is produced on purpose and harmlessly: the raw-pointer
    matMul is told that `out` has 130 rows while the tensor behind it has 128, so its last two rows
    (256 bytes) land on the guard, which still lies inside the buffer's allocation."""
    bk = tf.ENGINE.backend
    lib = bk._lib

    def ptr(t):
        p, n = C.c_void_p(), C.c_size_t()
        assert lib.tfjs_cuda_tensor_device_ptr(bk._ctx, bk._rec(t.dataId)["id"], C.byref(p), C.byref(n)) == 0
        return p

    rng = np.random.Generator(np.random.PCG64(6))
    a = tf.ops.tensor(rng.uniform(-1, 1, (130, 64)).astype(np.float32))
    b = tf.ops.tensor(rng.uniform(-1, 1, (64, 32)).astype(np.float32))
    bk.setOption("debug_canary", 1)
    try:
        # a clean run first: guards intact, nothing reported
        ok = tf.ops.tensor(np.zeros((130, 32), np.float32))
        assert lib.tfjs_cuda_matmul_static_scratch(bk._ctx, ptr(a), ptr(b), None, ptr(ok), 130, 64, 32, 0, 0, 0) == 0
        ok.dispose()
        bk.sync()
        small = tf.ops.tensor(np.zeros((128, 32), np.float32))
        assert lib.tfjs_cuda_matmul_static_scratch(bk._ctx, ptr(a), ptr(b), None, ptr(small), 130, 64, 32, 0, 0, 0) == 0
        small.dispose()                # the guard is verified here, on the stream
        with pytest.raises(CudaError, match="guard pattern"):
            bk.sync()
    finally:
        bk.setOption("debug_canary", 0)
    bk.sync()
    a.dispose()
    b.dispose()
