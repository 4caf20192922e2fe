#!/usr/bin/env python3
"""Device and CPU times of BASELINE configs 1-3 (the single-op parity cases).

    python tfjs-core_b200/profile_configs.py [tf32|3xtf32] [--no-cpu]

For each config: the error against the CPU oracle, the oracle's own time on one host thread
(the same unfused passes the reference executes), the device time of one call launched
eagerly and replayed from a CUDA graph, and the bandwidth / FLOP rate the algorithmic figures
correspond to.  The tensors of these configs (6-16 MB) fit in L2, so the replay numbers are
L2-resident rates; a second column repeats the replay with a 256 MB write between calls
(cold L2), timed by per-kernel events.  These are table rows, not the benchmark: bench.py
measures the whole network.
"""
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import tfjs_core_b200 as tf  # noqa: E402
from tfjs_core_b200 import conv_util, ops  # noqa: E402


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def make_config(n):
    """(name, flop, bytes, host tensors, device call, oracle call)."""
    if n == 1:
        r = rng(0)
        a = r.uniform(-1, 1, (256, 1024)).astype(np.float32)
        lim = np.sqrt(6.0 / 2048)
        b = r.uniform(-lim, lim, (1024, 1024)).astype(np.float32)
        bias = r.normal(0, 0.01, 1024).astype(np.float32)
        return dict(name="1 fused matMul 256x1024x1024 + bias + relu", flop=536870912, bytes=6295552,
                    host=(a, b, bias),
                    dev=lambda t: ops.fused_matmul(t[0], t[1], bias=t[2], activation="relu"),
                    cpu=lambda o: o.fused_matmul(a[None], b[None], bias=bias, activation="relu")[0])
    if n == 2:
        r = rng(1)
        x = r.uniform(0, 1, (8, 56, 56, 64)).astype(np.float32)
        w = r.normal(0, np.sqrt(2.0 / 576), (3, 3, 64, 64)).astype(np.float32)
        bias = r.normal(0, 0.01, 64).astype(np.float32)
        return dict(name="2 fused conv2d 8x56x56x64 * 3x3x64x64 same + bias + relu", flop=1849688064,
                    bytes=12992768, host=(x, w, bias),
                    dev=lambda t: ops.fused_conv2d(t[0], t[1], 1, "same", bias=t[2], activation="relu"),
                    cpu=lambda o: o.fused_conv2d(x, w, o.compute_conv2d_info(x.shape, w.shape, 1, 1, "same"),
                                                 bias=bias, activation="relu"))
    r = rng(2)
    x = r.uniform(0, 1, (8, 112, 112, 32)).astype(np.float32)
    w = r.normal(0, np.sqrt(2.0 / 9), (3, 3, 32, 1)).astype(np.float32)
    bias = r.normal(0, 0.01, 32).astype(np.float32)

    def dev(t):
        ci = conv_util.compute_conv2d_info(x.shape, w.shape, 2, 1, "same", None, True)
        return tf.ENGINE.backend.fusedDepthwiseConv2D(t[0], t[1], ci, t[2], "relu6")

    def cpu(o):
        ci = o.compute_conv2d_info(x.shape, w.shape, 2, 1, "same", None, True)
        return o.unary("clip", o.binary("add", o.depthwise_conv2d(x, w, ci), bias), 0, 6)

    return dict(name="3 depthwise 8x112x112x32 * 3x3 s2 same + bias + relu6 (fused)", flop=14450688,
                bytes=16057600, host=(x, w, bias), dev=dev, cpu=cpu)


def main():
    mode = sys.argv[1] if len(sys.argv) > 1 and not sys.argv[1].startswith("-") else "tf32"
    with_cpu = "--no-cpu" not in sys.argv
    bk = tf.BackendCuda(0, mode)
    tf.ENGINE.registerBackend("profile-cuda", lambda: bk, 10)
    tf.ENGINE.setBackend("profile-cuda")
    flush = ops.tensor(np.zeros(64 << 20, np.float32))  # 256 MB > L2
    if with_cpu:
        import oracle
    reps = 20
    for n in (1, 2, 3):
        c = make_config(n)
        t = [ops.tensor(h) for h in c["host"]]
        out = c["dev"](t)
        got = out.dataSync()
        out.dispose()
        err = cpu_ms = float("nan")
        if with_cpu:
            t0 = time.perf_counter()
            want = c["cpu"](oracle)
            cpu_ms = (time.perf_counter() - t0) * 1e3
            err = np.abs(got.reshape(want.shape).astype(np.float64) - want).max() / np.abs(want).max()

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
              f"   max err / max|want| {err:.2e}   oracle (1 thread) {cpu_ms:.1f} ms\n"
              f"   eager {eager_us:.1f} us   graph replay {replay_us:.1f} us "
              f"({c['bytes'] / replay_us / 1e3:.0f} GB/s, {c['flop'] / replay_us / 1e6:.1f} TFLOP/s, L2-resident)   "
              f"cold L2 {cold_us:.1f} us ({c['bytes'] / cold_us / 1e3:.0f} GB/s, "
              f"{c['flop'] / cold_us / 1e6:.1f} TFLOP/s)", flush=True)
        for x in t:
            x.dispose()


if __name__ == "__main__":
    main()
