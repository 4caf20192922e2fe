#!/usr/bin/env python3
"""Device times of BASELINE configs 1-3 (the single-op parity cases) and of the memory-bound
operators of the unfused tf.* path.

    python profile_configs.py [tf32|3xtf32]          # configs 1-3
    python profile_configs.py ops [batch] [reps]     # add / clip / exp / sum / max / pooling
    python profile_configs.py block B HW C N [stride] [key=value ...]
                                                     # one depthwise 3x3 + pointwise block on its own
    python profile_configs.py stem B                 # the 3x3x3->32 stride-2 first convolution on its own
    python profile_configs.py matmul M K N [tf32|3xtf32] [key=value ...]   # one fused matMul + bias, graph replay

For each config: the device time of one call launched eagerly and replayed from a CUDA graph, and
the bandwidth / FLOP rate the algorithmic figures correspond to (parity with the CPU oracle is
the tests' business, tests/test_gpu_parity.py).  The tensors of these configs (6-16 MB) fit in L2, so the replay numbers are
L2-resident rates; a second column repeats the replay with a 256 MB write between calls
(cold L2), timed by per-kernel events.  These are table rows, not the benchmark: bench.py
measures the whole network.
"""
import os
import sys
import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import tfjs_core_b200 as tf  # noqa: E402
from tfjs_core_b200 import conv_util, ops  # noqa: E402


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def make_config(n):
    """name, flop, bytes, host tensors, device call."""
    if n == 1:
        r = rng(0)
        a = r.uniform(-1, 1, (256, 1024)).astype(np.float32)
        lim = np.sqrt(6.0 / 2048)
        b = r.uniform(-lim, lim, (1024, 1024)).astype(np.float32)
        bias = r.normal(0, 0.01, 1024).astype(np.float32)
        return dict(name="1 fused matMul 256x1024x1024 + bias + relu", flop=536870912, bytes=6295552,
                    host=(a, b, bias),
                    dev=lambda t: ops.fused_matmul(t[0], t[1], bias=t[2], activation="relu"))
    if n == 2:
        r = rng(1)
        x = r.uniform(0, 1, (8, 56, 56, 64)).astype(np.float32)
        w = r.normal(0, np.sqrt(2.0 / 576), (3, 3, 64, 64)).astype(np.float32)
        bias = r.normal(0, 0.01, 64).astype(np.float32)
        return dict(name="2 fused conv2d 8x56x56x64 * 3x3x64x64 same + bias + relu", flop=1849688064,
                    bytes=12992768, host=(x, w, bias),
                    dev=lambda t: ops.fused_conv2d(t[0], t[1], 1, "same", bias=t[2], activation="relu"))
    r = rng(2)
    x = r.uniform(0, 1, (8, 112, 112, 32)).astype(np.float32)
    w = r.normal(0, np.sqrt(2.0 / 9), (3, 3, 32, 1)).astype(np.float32)
    bias = r.normal(0, 0.01, 32).astype(np.float32)

    def dev(t):
        ci = conv_util.compute_conv2d_info(x.shape, w.shape, 2, 1, "same", None, True)
        return tf.ENGINE.backend.fusedDepthwiseConv2D(t[0], t[1], ci, t[2], "relu6")

    return dict(name="3 depthwise 8x112x112x32 * 3x3 s2 same + bias + relu6 (fused)", flop=14450688,
                bytes=16057600, host=(x, w, bias), dev=dev)


def run_ops(batch, reps=5):
    """The memory-bound operators as the unfused tf.* path issues them, on MobileNet-sized tensors
    larger than L2: bias add ([B,H,W,C] + [C]), clipByValue, exp, sum and max over the last axis,
    a 3x3 stride-2 max pool and a 2x2 average pool.  Per-kernel device time from events between
    launches; bytes = every tensor once."""
    bk = tf.BackendCuda(0, "tf32")
    tf.ENGINE.registerBackend("profile-cuda", lambda: bk, 10)
    tf.ENGINE.setBackend("profile-cuda")
    r = rng(11)
    x = ops.tensor(r.uniform(-3, 9, (batch, 112, 112, 64)).astype(np.float32))   # 3.2 MB per image
    bias = ops.tensor(r.normal(0, 1, 64).astype(np.float32))
    rows2d = ops.tensor(r.uniform(-3, 3, (batch * 112, 1000)).astype(np.float32))
    n = x.size
    cases = [
        ("add [B,112,112,64] + [64]", lambda: ops.add(x, bias), 8 * n),
        ("clipByValue(0, 6)", lambda: ops.clip_by_value(x, 0, 6), 8 * n),
        ("exp", lambda: ops.exp(x), 8 * n),
        ("sum over the last axis [B*112, 1000]", lambda: ops.sum(rows2d, -1), 4 * rows2d.size + 4 * rows2d.shape[0]),
        ("max over the last axis [B*112, 1000]", lambda: ops.max(rows2d, -1), 4 * rows2d.size + 4 * rows2d.shape[0]),
        ("maxPool 3x3 s2 same", lambda: ops.max_pool(x, [3, 3], 2, "same"), 4 * n + n),
        ("avgPool 2x2 s2 valid", lambda: ops.avg_pool(x, [2, 2], 2, "valid"), 4 * n + n),
    ]
    for name, fn, nbytes in cases:
        fn().dispose()
        bk.profileBegin(4 * reps)
        for _ in range(reps):
            fn().dispose()
        rows = bk.profileEnd()
        best = min(ms for _, ms in rows)
        print(f"{name:42s} {rows[0][0]:24s} {best * 1e3:9.1f} us  {nbytes / best / 1e6:8.0f} GB/s", flush=True)


def run_block(batch, hw, c, n, stride, options, reps=5):
    """One separable block (depthwise 3x3 + bias + relu6, pointwise + bias + relu6) of a MobileNet
    layer's shape, alone on the device: input, intermediate and output are the only large buffers
    (1.2 GB for pw7-pw11 at batch 1024), which keeps a profiler capture of a full-size launch small.
    `options` are context options (e.g. gemm_pair=0, fuse_separable=0)."""
    bk = tf.BackendCuda(0, "tf32")
    tf.ENGINE.registerBackend("profile-cuda", lambda: bk, 10)
    tf.ENGINE.setBackend("profile-cuda")
    for key, value in options.items():
        bk.setOption(key, value)
    r = rng(21)
    x = ops.tensor(r.uniform(0, 6, (batch, hw, hw, c)).astype(np.float32))
    wd = ops.tensor(r.normal(0, 0.5, (3, 3, c, 1)).astype(np.float32))
    wp = ops.tensor((r.uniform(-1, 1, (1, 1, c, n)) / np.sqrt(c)).astype(np.float32))
    bd = ops.tensor(r.normal(0, 0.3, c).astype(np.float32))
    bp = ops.tensor(r.normal(0, 0.3, n).astype(np.float32))
    ci = conv_util.compute_conv2d_info(x.shape, wd.shape, stride, 1, "same", None, True)
    call = lambda: bk.fusedSeparableConv2d(x, wd, wp, ci, bd, "relu6", bp, "relu6")  # noqa: E731
    call().dispose()
    bk.profileBegin(4 * reps)
    for _ in range(reps):
        call().dispose()
    rows = bk.profileEnd()
    per_call = len(rows) // reps
    out_pixels = batch * ci.outHeight * ci.outWidth
    nbytes = {"depthwise": 4 * (x.size + out_pixels * c), "pointwise": 4 * out_pixels * (c + n),
              "fused": 4 * (x.size + out_pixels * n)}
    for i in range(per_call):
        name = rows[i][0]
        best = min(rows[i + k * per_call][1] for k in range(reps))
        kind = "fused" if name.startswith("separableConv2d") else ("depthwise" if name.startswith("depthwise") else "pointwise")
        print(f"{name:62s} {best * 1e3:9.1f} us {nbytes[kind] / 1e6:9.1f} MB {nbytes[kind] / best / 1e6:7.0f} GB/s", flush=True)


def run_stem(batch, reps=5):
    """MobileNet's first layer (3x3x3 -> 32, stride 2, + bias + relu6) alone on the device."""
    bk = tf.BackendCuda(0, "tf32")
    tf.ENGINE.registerBackend("profile-cuda", lambda: bk, 10)
    tf.ENGINE.setBackend("profile-cuda")
    r = rng(22)
    x = ops.tensor(r.uniform(-1, 1, (batch, 224, 224, 3)).astype(np.float32))
    w = ops.tensor(r.normal(0, 0.3, (3, 3, 3, 32)).astype(np.float32))
    b = ops.tensor(r.normal(0, 0.3, 32).astype(np.float32))
    call = lambda: ops.fused_conv2d(x, w, 2, "same", bias=b, activation="relu6")  # noqa: E731
    call().dispose()
    bk.profileBegin(4 * reps)
    for _ in range(reps):
        call().dispose()
    rows = bk.profileEnd()
    per_call = len(rows) // reps
    nbytes = 4 * (x.size + batch * 112 * 112 * 32)
    for i in range(per_call):
        best = min(rows[i + k * per_call][1] for k in range(reps))
        print(f"{rows[i][0]:62s} {best * 1e3:9.1f} us {nbytes / 1e6:9.1f} MB {nbytes / best / 1e6:7.0f} GB/s", flush=True)


def run_matmul(m, k, n, mode, options, reps=50):
    """One fusedBatchMatMul [m, k] x [k, n] + bias on its own, replayed from a CUDA graph (device time
    per call without host launch gaps)."""
    bk = tf.BackendCuda(0, mode)
    tf.ENGINE.registerBackend("profile-cuda", lambda: bk, 10)
    tf.ENGINE.setBackend("profile-cuda")
    for key, value in options.items():
        bk.setOption(key, value)
    r = rng(23)
    a = ops.tensor(r.uniform(-1, 1, (m, k)).astype(np.float32))
    b = ops.tensor((r.uniform(-1, 1, (k, n)) / np.sqrt(k)).astype(np.float32))
    bias = ops.tensor(r.normal(0, 0.1, n).astype(np.float32))
    call = lambda: ops.fused_matmul(a, b, bias=bias)  # noqa: E731
    call().dispose()
    bk.graphBegin()
    call().dispose()
    g = bk.graphEnd()
    bk.graphLaunch(g)

    def replay():
        for _ in range(reps):
            bk.graphLaunch(g)
    us = bk.time(replay)["kernelMs"] * 1e3 / reps
    bk.profileBegin(4)
    call().dispose()
    name = bk.profileEnd()[-1][0]
    nbytes = 4 * (m * k + k * n + m * n + n)
    print(f"matMul {m} x {k} x {n} {mode} {options}: {name}  {us:.1f} us  {nbytes / us / 1e3:.0f} GB/s  "
          f"{2.0 * m * k * n / us / 1e6:.1f} TFLOP/s", flush=True)


def main():
    if len(sys.argv) > 1 and sys.argv[1] == "matmul":
        nums = [int(a) for a in sys.argv[2:] if a.isdigit()]
        mode = "3xtf32" if "3xtf32" in sys.argv else "tf32"
        options = {a.split("=")[0]: int(a.split("=")[1]) for a in sys.argv[2:] if "=" in a}
        return run_matmul(nums[0], nums[1], nums[2], mode, options)
    if len(sys.argv) > 1 and sys.argv[1] == "stem":
        return run_stem(int(sys.argv[2]) if len(sys.argv) > 2 else 64)
    if len(sys.argv) > 1 and sys.argv[1] == "block":
        nums = [int(a) for a in sys.argv[2:] if "=" not in a]
        options = {a.split("=")[0]: int(a.split("=")[1]) for a in sys.argv[2:] if "=" in a}
        return run_block(nums[0], nums[1], nums[2], nums[3], nums[4] if len(nums) > 4 else 1, options)
    if len(sys.argv) > 1 and sys.argv[1] == "ops":
        return run_ops(int(sys.argv[2]) if len(sys.argv) > 2 else 64, int(sys.argv[3]) if len(sys.argv) > 3 else 5)
    mode = sys.argv[1] if len(sys.argv) > 1 and not sys.argv[1].startswith("-") else "tf32"
    bk = tf.BackendCuda(0, mode)
    tf.ENGINE.registerBackend("profile-cuda", lambda: bk, 10)
    tf.ENGINE.setBackend("profile-cuda")
    flush = ops.tensor(np.zeros(64 << 20, np.float32))  # 256 MB > L2
    reps = 20
    for n in (1, 2, 3):
        c = make_config(n)
        t = [ops.tensor(h) for h in c["host"]]
        out = c["dev"](t)
        got = out.dataSync()
        out.dispose()
        assert np.isfinite(got).all()

        def eager():
            for _ in range(reps):
                c["dev"](t).dispose()
        eager()
        eager_us = bk.time(eager)["kernelMs"] * 1e3 / reps
        bk.graphBegin()
        c["dev"](t).dispose()
        g = bk.graphEnd()
        bk.graphLaunch(g)

        def replay():
            for _ in range(reps):
                bk.graphLaunch(g)
        replay_us = bk.time(replay)["kernelMs"] * 1e3 / reps
        # cold L2: a 256 MB pass between calls; per-kernel events give the op's own time
        bk.profileBegin(8 * reps)
        for _ in range(reps):
            ops.relu(flush).dispose()
            c["dev"](t).dispose()
        rows = bk.profileEnd()
        cold = [ms for name, ms in rows if not name.startswith("unary")]
        per_call = len(cold) // reps
        cold_us = min(sum(cold[i * per_call:(i + 1) * per_call]) for i in range(reps)) * 1e3
        bk.graphDestroy(g)
        print(f"config {c['name']}\n"
              f"   eager {eager_us:.1f} us   graph replay {replay_us:.1f} us "
              f"({c['bytes'] / replay_us / 1e3:.0f} GB/s, {c['flop'] / replay_us / 1e6:.1f} TFLOP/s, L2-resident)   "
              f"cold L2 {cold_us:.1f} us ({c['bytes'] / cold_us / 1e3:.0f} GB/s, "
              f"{c['flop'] / cold_us / 1e6:.1f} TFLOP/s)", flush=True)
        for x in t:
            x.dispose()


if __name__ == "__main__":
    main()
