#!/usr/bin/env python3
"""Per-layer device times of one fused MobileNetV1 forward on the cuda backend.

    python profile_layers.py [batch] [tf32|3xtf32] [f|q|q-in-loop] [separable|layerwise|separable-all] [f32|f16]

Prints, for each launch of one forward pass (25 with the fused depthwise + pointwise blocks,
30 with `layerwise`), the kernel name, the best device time over a few passes
(events recorded between launches on the context's stream), the layer's algorithmic bytes and
the bandwidth that corresponds to.  `q` stores the filters as uint8 (BASELINE config 5); `q-in-loop` also keeps the GEMM weights uint8 and dequantises them inside the GEMM main loop;
`separable-all` fuses every block the fused kernel can take (up to 256 channels), not only those
where fusion pays.  At a small batch this is also a convenient command to capture single
kernels of the network with ncu.
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import tfjs_core_b200 as tf  # noqa: E402
from tfjs_core_b200 import mobilenet, ops  # noqa: E402


def main():
    batch = int(sys.argv[1]) if len(sys.argv) > 1 else 64
    mode = sys.argv[2] if len(sys.argv) > 2 else "tf32"
    quantized = len(sys.argv) > 3 and sys.argv[3] in ("q", "q-in-loop")
    in_loop = len(sys.argv) > 3 and sys.argv[3] == "q-in-loop"
    layerwise = len(sys.argv) > 4 and sys.argv[4] == "layerwise"
    half = len(sys.argv) > 5 and sys.argv[5] == "f16"   # activations stored as IEEE half
    reps = 4
    bk = tf.BackendCuda(0, mode)
    tf.ENGINE.registerBackend("profile-cuda", lambda: bk, 10)
    tf.ENGINE.setBackend("profile-cuda")
    bk.setOption("dequant_in_gemm", 1 if in_loop else 0)
    if half:
        bk.setActivationStorage("float16")
    if len(sys.argv) > 4 and sys.argv[4] == "separable-all":
        bk.setOption("fuse_separable", 2)
    params = mobilenet.make_weights(4 if quantized else 3, quantized=quantized, gain=1.5)
    net = mobilenet.MobileNetV1(params, bk)
    forward = net.forward_fused if layerwise else net.forward_separable
    x = ops.tensor(mobilenet.make_input(3, batch))
    for _ in range(2):
        before = bk.launchCount()
        logits, probs = forward(x)
        n = bk.launchCount() - before
        probs.dataSync()
        logits.dispose()
        probs.dispose()
    bk.profileBegin((n + 2) * reps)
    for _ in range(reps):
        logits, probs = forward(x)
        logits.dispose()
        probs.dispose()
    rows = bk.profileEnd()
    kernel_names = [name for name, _ in rows[:n]]
    layer_bytes = mobilenet.launch_algorithmic_bytes(batch, quantized, kernel_names, half)
    names = [s[0] for s in mobilenet.layer_specs()][:-1] + ["avgpool", "fc", "softmax"]
    total, layer = 0.0, 0
    for i in range(n):
        ms = min(rows[i + n * r][1] for r in range(reps))
        total += ms
        fused = kernel_names[i].startswith("separableConv2d (fused")
        label = names[layer] + "+" + names[layer + 1] if fused else names[layer]
        layer += 2 if fused else 1
        print(f"{label:9s} {kernel_names[i]:62s} {ms * 1e3:9.1f} us {layer_bytes[i] / 1e6:9.1f} MB "
              f"{layer_bytes[i] / ms / 1e6:7.0f} GB/s")
    print(f"total {total:.3f} ms  {batch / total * 1e3:.0f} img/s  "
          f"{sum(layer_bytes) / total / 1e6:.0f} GB/s algorithmic")


if __name__ == "__main__":
    main()
