"""The TF32 GEMM on pairs of CTAs (256 x 256 tiles, tcgen05 cta_group::2).

It serves the pointwise convolution of a separable block whose depthwise result has already been
rounded to tf32 (KernelBackend.fusedConv2d with a 1x1 filter, tfjs-core/src/backends/backend.ts:
414-418).  The pair kernel issues the same tensor-core instructions over the same k-slices as the
single-CTA kernel, so the two must agree bit for bit; against the CPU oracle the block is held to
the TF32 tolerance.  Shapes cover whole tiles, a last row tile whose second CTA lies entirely
beyond M, one and several column tiles, one to many k-blocks, and every epilogue.
"""
import numpy as np
import pytest

import oracle
from gpu_util import rel_err, tf  # noqa: F401

pytestmark = pytest.mark.gpu


def _block(tf, b, h, w, c, n, seed, pw_act, bias, pair):
    """depthwise 3x3 + pointwise through fusedSeparableConv2d's two-kernel form."""
    from tfjs_core_b200 import conv_util
    bk = tf.ENGINE.backend
    rng = np.random.Generator(np.random.PCG64(seed))
    x = rng.uniform(-1, 1, (b, h, w, c)).astype(np.float32)
    wd = rng.normal(0, 0.5, (3, 3, c, 1)).astype(np.float32)
    wp = (rng.uniform(-1, 1, (1, 1, c, n)) / np.sqrt(c)).astype(np.float32)
    bd = rng.normal(0, 0.3, c).astype(np.float32)
    bp = rng.normal(0, 0.3, n).astype(np.float32) if bias else None
    ci = conv_util.compute_conv2d_info(x.shape, wd.shape, 1, 1, "same", None, True)
    t = lambda a: None if a is None else tf.ops.tensor(a)  # noqa: E731
    bk.setOption("gemm_pair", pair)
    before = bk.launchCount()
    y = bk.fusedSeparableConv2d(t(x), t(wd), t(wp), ci, t(bd), "relu6", t(bp), pw_act)
    out = y.dataSync().reshape(y.shape)
    return x, wd, wp, bd, bp, out, bk.launchCount() - before


def _oracle_block(x, wd, wp, bd, bp, pw_act):
    ci = oracle.compute_conv2d_info(x.shape, wd.shape, 1, 1, "same", None, True)
    mid = oracle.unary("clip", oracle.binary("add", oracle.depthwise_conv2d(x, wd, ci), bd), 0, 6)
    ci2 = oracle.compute_conv2d_info(mid.shape, wp.shape, 1, 1, "valid")
    y = oracle.conv2d(mid, wp, ci2)
    if bp is not None:
        y = oracle.binary("add", y, bp)
    if pw_act == "relu6":
        y = oracle.unary("clip", y, 0, 6)
    elif pw_act == "relu":
        y = oracle.unary("relu", y)
    return y


SHAPES = [
    # b, h, w, c (= K), n, pointwise activation, bias
    (8, 14, 14, 512, 512, "relu6", True),    # M = 1568: 6 whole row tiles + 32 rows, two column tiles
    (3, 14, 14, 512, 256, "relu", True),     # M = 588: the last tile's second CTA is all padding
    (2, 16, 16, 288, 1024, "linear", False), # M = 512: whole tiles, 9 k-blocks, four column tiles
    (6, 7, 7, 1024, 1024, "relu6", True),    # M = 294: one tile and a sliver, 32 k-blocks
    (4, 16, 16, 128, 256, "linear", True),   # 4 k-blocks: shorter than the ring
]


@pytest.mark.parametrize("b,h,w,c,n,act,bias", SHAPES)
def test_pair_kernel_equals_single_cta_kernel_and_matches_the_oracle(tf, b, h, w, c, n, act, bias):
    bk = tf.ENGINE.backend
    bk.setMathMode("tf32")
    bk.setOption("fuse_separable", 0)
    try:
        seed = b * 1000 + c + n
        x, wd, wp, bd, bp, single, _ = _block(tf, b, h, w, c, n, seed, act, bias, pair=0)
        bk.profileBegin(16)
        _, _, _, _, _, paired, _ = _block(tf, b, h, w, c, n, seed, act, bias, pair=2)
        names = [name for name, _ in bk.profileEnd()]
        assert any("CTA pairs" in name for name in names), names   # the pair kernel did run
        assert np.array_equal(paired, single)
        want = _oracle_block(x, wd, wp, bd, bp, act)
        assert rel_err(paired, want) <= 1e-3   # TF32 contraction tolerance
    finally:
        bk.setOption("gemm_pair", 1)
        bk.setOption("fuse_separable", 1)
        bk.setMathMode("3xtf32")


@pytest.mark.parametrize("b,h,w,c,n,act,bias", SHAPES)
def test_pair_kernel_3xtf32_equals_single_cta_kernel_and_matches_the_oracle(tf, b, h, w, c, n, act, bias):
    """3xTF32: each CTA's converter warps split its A stages into tf32 hi / lo, the weight halves
    arrive as hi and lo planes, three MMAs per k-step into a main and a correction accumulator.
    Same instruction sequence per output element as the single-CTA kernel: bit-identical, and within
    1e-5 of the oracle."""
    bk = tf.ENGINE.backend
    bk.setMathMode("3xtf32")
    bk.setOption("fuse_separable", 0)
    try:
        seed = b * 1000 + c + n + 1
        x, wd, wp, bd, bp, single, _ = _block(tf, b, h, w, c, n, seed, act, bias, pair=0)
        bk.profileBegin(16)
        _, _, _, _, _, paired, _ = _block(tf, b, h, w, c, n, seed, act, bias, pair=2)
        names = [name for name, _ in bk.profileEnd()]
        assert any("3xTF32, CTA pairs" in name for name in names), names
        assert np.array_equal(paired, single)
        want = _oracle_block(x, wd, wp, bd, bp, act)
        assert rel_err(paired, want) <= 1e-5   # 3xTF32 contraction tolerance
    finally:
        bk.setOption("gemm_pair", 1)
        bk.setOption("fuse_separable", 1)


@pytest.mark.parametrize("mode,tol", [("tf32", 1e-3), ("3xtf32", 1e-5)])
def test_pair_kernel_on_a_plain_matmul(tf, mode, tol):
    """fusedBatchMatMul on operands straight from the host: in TF32 mode nothing has rounded A, so
    the converter warps of both CTAs round each A stage in shared memory (as the single-CTA kernel's
    do); ragged M, relu epilogue."""
    bk = tf.ENGINE.backend
    bk.setMathMode(mode)
    try:
        rng = np.random.Generator(np.random.PCG64(99))
        m, k, n = 1000, 256, 512
        a = rng.uniform(-1, 1, (1, m, k)).astype(np.float32)
        b = (rng.uniform(-1, 1, (1, k, n)) / np.sqrt(k)).astype(np.float32)
        bias = rng.normal(0, 0.3, n).astype(np.float32)
        outs = {}
        for pair in (0, 2):
            bk.setOption("gemm_pair", pair)
            bk.profileBegin(16)
            y = bk.fusedBatchMatMul(a=tf.ops.tensor(a), b=tf.ops.tensor(b), bias=tf.ops.tensor(bias), activation="relu")
            outs[pair] = y.dataSync().reshape(m, n)
            names = [name for name, _ in bk.profileEnd()]
            assert any("CTA pairs" in name for name in names) == (pair == 2), names
        assert np.array_equal(outs[2], outs[0])
        want = oracle.unary("relu", oracle.fused_matmul(a, b, bias=bias)[0])
        assert rel_err(outs[2], want) <= tol
    finally:
        bk.setOption("gemm_pair", 1)
        bk.setMathMode("3xtf32")


def test_pair_kernel_twice_in_a_row_and_after_other_kernels(tf):
    """Tensor memory and barriers are set up per launch: back-to-back launches with different
    shapes, with a single-CTA tensor-core kernel in between, leave nothing behind."""
    bk = tf.ENGINE.backend
    bk.setMathMode("tf32")
    bk.setOption("fuse_separable", 0)
    try:
        outs = []
        for rep in range(2):
            for (b, h, w, c, n, act, bias) in (SHAPES[0], SHAPES[1]):
                outs.append(_block(tf, b, h, w, c, n, 7, act, bias, pair=2)[5])
                _block(tf, 2, 8, 8, 64, 64, 8, "relu", True, pair=0)
        assert np.array_equal(outs[0], outs[2]) and np.array_equal(outs[1], outs[3])
    finally:
        bk.setOption("gemm_pair", 1)
        bk.setOption("fuse_separable", 1)
        bk.setMathMode("3xtf32")


def test_default_dispatch_takes_the_pair_kernel_only_for_large_problems(tf):
    bk = tf.ENGINE.backend
    bk.setMathMode("tf32")
    try:
        bk.profileBegin(16)
        _block(tf, 2, 14, 14, 512, 512, 1, "relu6", True, pair=1)        # 2 x 2 tiles: single-CTA kernel
        small = [name for name, _ in bk.profileEnd()]
        bk.profileBegin(16)
        _block(tf, 128, 14, 14, 512, 512, 1, "relu6", True, pair=1)      # 98 x 2 tiles: pairs
        large = [name for name, _ in bk.profileEnd()]
        assert not any("CTA pairs" in name for name in small), small
        assert any("CTA pairs" in name for name in large), large
    finally:
        bk.setMathMode("3xtf32")


def test_pair_kernel_writes_nothing_past_its_output(tf):
    """The pair kernel stores its rows with ordinary 128-bit stores (no tensor map clips them): with
    guard patterns behind every buffer (option debug_canary), a ragged M whose last tile is mostly
    padding leaves the guards intact, in all three precisions."""
    bk = tf.ENGINE.backend
    bk.setOption("debug_canary", 1)
    bk.setOption("fuse_separable", 0)
    try:
        for mode in ("tf32", "3xtf32"):
            bk.setMathMode(mode)
            out = _block(tf, 3, 14, 14, 512, 256, 5, "relu", True, pair=2)[5]      # M = 588
            assert np.isfinite(out).all()
            bk.sync()                                                               # guards checked on release
        bk.setMathMode("tf32")
        rng = np.random.Generator(np.random.PCG64(5))
        a = tf.ops.tensor(rng.uniform(-1, 1, (1, 300, 512)).astype(np.float32))    # rounding variant, M = 300
        b = tf.ops.tensor(rng.uniform(-1, 1, (1, 512, 256)).astype(np.float32))
        bk.setOption("gemm_pair", 2)
        y = bk.fusedBatchMatMul(a=a, b=b, bias=None, activation="linear")
        y.dataSync()
        y.dispose()
        bk.sync()
    finally:
        bk.setOption("debug_canary", 0)
        bk.setOption("gemm_pair", 1)
        bk.setOption("fuse_separable", 1)
        bk.setMathMode("3xtf32")


@pytest.mark.parametrize("scale,mn", [(0.0078125, -1.0), (0.013731, -1.7576)])
def test_pair_kernel_dequantises_uint8_weights_in_the_main_loop(tf, scale, mn):
    """Option dequant_in_gemm on CTA pairs: the pointwise filter stays uint8 in device memory, each
    CTA loads its 128 rows x 32 bytes per k-block and its converter warps expand them into the
    tensor cores' operand tile.  Bit-identical to the cached-plane path on pairs and on single CTAs."""
    from tfjs_core_b200 import conv_util
    bk = tf.ENGINE.backend
    bk.setMathMode("tf32")
    bk.setOption("fuse_separable", 0)
    try:
        rng = np.random.Generator(np.random.PCG64(77))
        b, hw, c, n = 5, 14, 512, 512                       # M = 980: three whole pair tiles + 212 rows
        x = rng.uniform(-1, 1, (b, hw, hw, c)).astype(np.float32)
        wd = rng.normal(0, 0.5, (3, 3, c, 1)).astype(np.float32)
        q = rng.integers(0, 256, (1, 1, c, n), dtype=np.uint8)
        bd = rng.normal(0, 0.3, c).astype(np.float32)
        bp = rng.normal(0, 0.3, n).astype(np.float32)
        ci = conv_util.compute_conv2d_info(x.shape, wd.shape, 1, 1, "same", None, True)
        wq = bk.registerQuantized(list(q.shape), q, scale, mn)
        outs = {}
        for pair, in_loop in ((0, 0), (2, 0), (0, 1), (2, 1)):
            bk.setOption("gemm_pair", pair)
            bk.setOption("dequant_in_gemm", in_loop)
            bk.profileBegin(16)
            y = bk.fusedSeparableConv2d(tf.ops.tensor(x), tf.ops.tensor(wd), wq, ci, tf.ops.tensor(bd), "relu6",
                                        tf.ops.tensor(bp), "linear")
            outs[(pair, in_loop)] = y.dataSync().reshape(y.shape)
            names = [name for name, _ in bk.profileEnd()]
            if pair == 2 and in_loop == 1:
                assert any("uint8 weights, CTA pairs" in name for name in names), names
        for key in outs:
            assert np.array_equal(outs[key], outs[(0, 0)]), key
        w = oracle.dequant_u8(q, scale, mn)
        want = _oracle_block(x, wd, w, bd, bp, "linear")
        assert rel_err(outs[(2, 1)], want) <= 1e-3
    finally:
        bk.setOption("gemm_pair", 1)
        bk.setOption("dequant_in_gemm", 0)
        bk.setOption("fuse_separable", 1)
        bk.setMathMode("3xtf32")
