"""MobileNetV1 (alpha 1.0, 224x224) inference written against the tfjs-core op surface.

The reference repository holds no model code (models live in @tensorflow-models); this driver
expresses the network with the ops an application would call (tf.fused.conv2d,
tf.depthwiseConv2d, tf.add, tf.clipByValue, tf.avgPool, tf.softmax), which is 77 backend
kernel calls per forward, and alternatively with the backend's fused extensions (relu6
epilogues, fused depthwise, fused softmax), which is 30 launches.

Weights are synthetic (seeded numpy PCG64): Glorot-uniform filters, N(0, 0.01) biases with
batch-norm assumed folded; optionally every filter is stored as uint8 affine-quantised bytes
(w = q*scale + min, the tfjs weights-manifest quantisation).
"""
import numpy as np

from . import conv_util, ops
from .engine import ENGINE

PW_OUT = [64, 128, 128, 256, 256, 512, 512, 512, 512, 512, 512, 1024, 1024]
DW_STRIDE = [1, 2, 1, 2, 1, 2, 1, 1, 1, 1, 1, 2, 1]
NUM_CLASSES = 1000


def layer_specs():
    """[(name, kind, filter_shape, stride)] in execution order."""
    specs = [("stem", "conv", (3, 3, 3, 32), 2)]
    c = 32
    for i, (co, s) in enumerate(zip(PW_OUT, DW_STRIDE), 1):
        specs.append((f"dw{i}", "dw", (3, 3, c, 1), s))
        specs.append((f"pw{i}", "conv", (1, 1, c, co), 1))
        c = co
    specs.append(("fc", "conv", (1, 1, c, NUM_CLASSES), 1))
    return specs


def _glorot(rng, shape, depthwise):
    fh, fw, cin, cout = shape
    if depthwise:
        fan_in = fan_out = fh * fw
    else:
        fan_in, fan_out = fh * fw * cin, fh * fw * cout
    lim = np.sqrt(6.0 / (fan_in + fan_out))
    return rng.uniform(-lim, lim, size=shape)


def make_weights(seed, quantized=False, gain=1.0):
    """Host-side synthetic parameters.  Returns {name: {'w': float32 array | None, 'q': uint8
    array | None, 'scale', 'min', 'b': float32 bias}} drawn in layer order."""
    rng = np.random.Generator(np.random.PCG64(seed))
    params = {}
    for name, kind, shape, _ in layer_specs():
        cout = shape[2] if kind == "dw" else shape[3]
        if quantized:
            q = rng.integers(0, 256, size=shape, dtype=np.uint8)
            scale = float(rng.uniform(1e-3, 2e-2))
            entry = {"w": None, "q": q, "scale": scale, "min": -128.0 * scale}
        else:
            entry = {"w": (gain * _glorot(rng, shape, kind == "dw")).astype(np.float32), "q": None}
        entry["b"] = rng.normal(0.0, 0.01, size=cout).astype(np.float32)
        params[name] = entry
    return params


def quantize_params(params):
    """The uint8-stored form of a float parameter dict, the way a tfjs converter stores a trained
    model: per tensor scale = (max - min) / 255, q = round((w - min) / scale), so that
    decodeWeights' w = q * scale + min (io/io_utils.ts:122-146) restores the filter to within half
    a step.  Biases stay float32."""
    out = {}
    for name, p in params.items():
        w = np.asarray(p["w"], np.float64)
        lo, hi = float(w.min()), float(w.max())
        scale = (hi - lo) / 255.0 if hi > lo else 1.0
        q = np.clip(np.rint((w - lo) / scale), 0, 255).astype(np.uint8)
        out[name] = {"w": None, "q": q, "scale": scale, "min": lo, "b": p["b"]}
    return out


def write_manifest(params, directory, shard_bytes=1 << 20):
    """Saves `params` (the dict make_weights returns) as a tfjs weights manifest: one group,
    entries `<layer>/filter` (uint8-quantised with the layer's scale / min when the layer has
    `q`, else float32) and `<layer>/bias`, the concatenated bytes cut into shard files of
    `shard_bytes`.  Returns the manifest (also written to weights_manifest.json)."""
    import json
    import os
    entries, chunks = [], []
    for name, _, _, _ in layer_specs():
        p = params[name]
        if p["q"] is not None:
            entries.append({"name": f"{name}/filter", "dtype": "float32", "shape": list(p["q"].shape),
                            "quantization": {"min": p["min"], "scale": p["scale"], "dtype": "uint8"}})
            chunks.append(p["q"].tobytes())
        else:
            entries.append({"name": f"{name}/filter", "dtype": "float32", "shape": list(p["w"].shape)})
            chunks.append(np.ascontiguousarray(p["w"], "<f4").tobytes())
        entries.append({"name": f"{name}/bias", "dtype": "float32", "shape": list(p["b"].shape)})
        chunks.append(np.ascontiguousarray(p["b"], "<f4").tobytes())
    blob = b"".join(chunks)
    paths = []
    for i in range(0, len(blob), shard_bytes):
        path = f"group1-shard{i // shard_bytes + 1}of{-(-len(blob) // shard_bytes)}"
        with open(os.path.join(directory, path), "wb") as f:
            f.write(blob[i:i + shard_bytes])
        paths.append(path)
    manifest = [{"paths": paths, "weights": entries}]
    with open(os.path.join(directory, "weights_manifest.json"), "w") as f:
        json.dump(manifest, f)
    return manifest


def make_input(seed, batch, offset=0):
    """Images ~U(-1, 1), NHWC float32.  `offset` skips that many images of the stream so that
    shards of one global batch draw disjoint slices of the same sequence."""
    rng = np.random.Generator(np.random.PCG64([seed, 12345]))
    if offset:
        rng.random(size=(offset, 224, 224, 3), dtype=np.float32)
    return (rng.random(size=(batch, 224, 224, 3), dtype=np.float32) * 2.0 - 1.0).astype(np.float32)


class MobileNetV1:
    """Device-resident parameters plus the two forward paths."""

    def __init__(self, params, backend=None):
        self.backend = backend or ENGINE.backend
        self.params = {}
        for name, p in params.items():
            if p["q"] is not None:
                w = self.backend.registerQuantized(list(p["q"].shape), p["q"], p["scale"], p["min"])
            else:
                w = ops.tensor(p["w"])
            self.params[name] = (w, ops.tensor(p["b"]))

    @classmethod
    def from_named_tensors(cls, named, backend=None):
        """The network over tensors that already live on the backend, as tf.io.loadWeights
        returns them: `named["<layer>/filter"]` and `named["<layer>/bias"]` for every layer of
        layer_specs()."""
        net = cls({}, backend)
        for name, _, _, _ in layer_specs():
            net.params[name] = (named[f"{name}/filter"], named[f"{name}/bias"])
        return net

    def dispose(self):
        for w, b in self.params.values():
            w.dispose()
            b.dispose()
        self.params = {}

    def forward_reference_api(self, x):
        """The network as unmodified tf.* code expresses it at this version of the library:
        no relu6 activation and no fused depthwise exist, so every layer is 2-3 backend calls
        and softmax is the 8-kernel op-layer chain."""
        def body():
            w, b = self.params["stem"]
            h = ops.fused_conv2d(x, w, 2, "same", bias=b, activation="linear")
            h = ops.clip_by_value(h, 0, 6)
            for i, s in enumerate(DW_STRIDE, 1):
                w, b = self.params[f"dw{i}"]
                h = ops.depthwise_conv2d(h, w, s, "same")
                h = ops.add(h, b)
                h = ops.clip_by_value(h, 0, 6)
                w, b = self.params[f"pw{i}"]
                h = ops.fused_conv2d(h, w, 1, "same", bias=b)
                h = ops.clip_by_value(h, 0, 6)
            h = ops.avg_pool(h, [7, 7], 1, "valid")
            w, b = self.params["fc"]
            h = ops.fused_conv2d(h, w, 1, "same", bias=b)
            logits = ops.reshape(h, [h.shape[0], NUM_CLASSES])
            return logits, ops.softmax(logits)
        return ENGINE.tidy(body)

    def forward_fused(self, x):
        """The same network through the backend's fused extensions: 1 + 13*2 + 1 + 1 + 1 = 30
        kernel launches."""
        bk = self.backend

        def then(new, old):
            # free each activation as soon as its consumer is enqueued, so that two buffers of
            # every size circulate instead of one per layer
            old.dispose()
            return new

        def body():
            w, b = self.params["stem"]
            ci = conv_util.compute_conv2d_info(x.shape, w.shape, 2, 1, "same")
            h = bk.fusedConv2d(x, w, ci, b, "relu6")
            for i, s in enumerate(DW_STRIDE, 1):
                w, b = self.params[f"dw{i}"]
                ci = conv_util.compute_conv2d_info(h.shape, w.shape, s, 1, "same", None, True)
                h = then(bk.fusedDepthwiseConv2D(h, w, ci, b, "relu6"), h)
                w, b = self.params[f"pw{i}"]
                ci = conv_util.compute_conv2d_info(h.shape, w.shape, 1, 1, "same")
                h = then(bk.fusedConv2d(h, w, ci, b, "relu6"), h)
            ci = conv_util.compute_pool2d_info(h.shape, [7, 7], 1, 1, "valid")
            h = then(bk.avgPool(h, ci), h)
            w, b = self.params["fc"]
            ci = conv_util.compute_conv2d_info(h.shape, w.shape, 1, 1, "same")
            h = then(bk.fusedConv2d(h, w, ci, b, "linear", None, "float32"), h)   # logits stay float32
            logits = then(bk.reshape(h, [h.shape[0], NUM_CLASSES]), h)
            return logits, bk.softmax(logits)
        return ENGINE.tidy(body)


def _forward_separable(self, x):
    """forward_fused with each depthwise + pointwise pair issued as one fusedSeparableConv2d
    call: the blocks the fused kernel takes (3x3 depthwise over at most 256 channels into at
    most 256 output channels: blocks 1-5) keep the depthwise result on chip, the others run
    their two kernels inside the call."""
    bk = self.backend

    def then(new, old):
        old.dispose()
        return new

    def body():
        w, b = self.params["stem"]
        ci = conv_util.compute_conv2d_info(x.shape, w.shape, 2, 1, "same")
        h = bk.fusedConv2d(x, w, ci, b, "relu6")
        for i, s in enumerate(DW_STRIDE, 1):
            wd, bd = self.params[f"dw{i}"]
            wp, bp = self.params[f"pw{i}"]
            ci = conv_util.compute_conv2d_info(h.shape, wd.shape, s, 1, "same", None, True)
            h = then(bk.fusedSeparableConv2d(h, wd, wp, ci, bd, "relu6", bp, "relu6"), h)
        ci = conv_util.compute_pool2d_info(h.shape, [7, 7], 1, 1, "valid")
        h = then(bk.avgPool(h, ci), h)
        w, b = self.params["fc"]
        ci = conv_util.compute_conv2d_info(h.shape, w.shape, 1, 1, "same")
        h = then(bk.fusedConv2d(h, w, ci, b, "linear", None, "float32"), h)   # logits stay float32
        logits = then(bk.reshape(h, [h.shape[0], NUM_CLASSES]), h)
        return logits, bk.softmax(logits)
    return ENGINE.tidy(body)


MobileNetV1.forward_separable = _forward_separable


def layer_algorithmic_bytes(batch, quantized, half=False):
    """Algorithmic bytes of each of the 30 launches of the fused forward, in launch order:
    |x| + |y| at their stored width + filter bytes + 4*|bias| with every tensor counted once.
    `half`: activations are stored as IEEE half (2 bytes) between the stem and the global pool;
    the input image, the pooled features, the logits and the probabilities stay float32."""
    out = []
    h = w = 224
    c = 3
    wb = 1 if quantized else 4
    ab = 2 if half else 4
    for name, kind, shape, s in layer_specs():
        if name == "fc":
            out.append(batch * (ab * 7 * 7 * c + 4 * c))
            out.append(4 * batch * (c + 1000) + wb * c * 1000 + 4 * 1000)
            out.append(4 * batch * 2000)
            break
        ho, wo = -(-h // s), -(-w // s)
        co = c if kind == "dw" else shape[3]
        in_b = 4 if name == "stem" else ab
        out.append(batch * (in_b * h * w * c + ab * ho * wo * co) + wb * int(np.prod(shape)) + 4 * co)
        h, w, c = ho, wo, co
    return out



def launch_algorithmic_bytes(batch, quantized, kernel_names, half=False):
    """Algorithmic bytes of each launch of one forward pass given the names of the kernels it
    launched, in order: a launch whose name starts with 'separableConv2d (fused' covers a
    depthwise + pointwise pair and counts the pair's input, output, filters and biases (the
    intermediate tensor does not exist); every other launch counts its own layer."""
    per_layer = layer_algorithmic_bytes(batch, quantized, half)
    specs = layer_specs()
    out, i = [], 0
    h = w = 224
    c = 3
    ab = 2 if half else 4
    sizes = []  # (in elements, out elements) per image for the 27 conv layers
    for name, kind, shape, s in specs[:-1]:
        ho, wo = -(-h // s), -(-w // s)
        co = c if kind == "dw" else shape[3]
        sizes.append((h * w * c, ho * wo * co))
        h, w, c = ho, wo, co
    for name in kernel_names:
        if name.startswith("separableConv2d (fused"):
            assert specs[i][1] == "dw" and specs[i + 1][1] == "conv", "fused launch out of place"
            mid = sizes[i][1]
            out.append(per_layer[i] + per_layer[i + 1] - 2 * ab * batch * mid)
            i += 2
        else:
            out.append(per_layer[i])
            i += 1
    assert i == len(per_layer), "kernel list does not cover the network"
    return out


def reference_api_launch_bytes(batch, quantized, kernel_names):
    """Algorithmic bytes of each launch of forward_reference_api (the network as unmodified tf.*
    code runs it), in launch order: every contraction / depthwise / pooling launch counts its
    layer once; every element-wise pass (the bias `add`, `clipByValue`, the stages of the softmax
    chain) reads and writes the activation it touches, which is what the unfused form costs."""
    per_layer = layer_algorithmic_bytes(batch, quantized)
    specs = layer_specs()
    sizes = []
    h = w = 224
    c = 3
    for name, kind, shape, s in specs[:-1]:
        ho, wo = -(-h // s), -(-w // s)
        co = c if kind == "dw" else shape[3]
        sizes.append(ho * wo * co)
        h, w, c = ho, wo, co
    sizes += [c, NUM_CLASSES]                      # global average pool, classifier
    out, layer, cur = [], 0, 0
    tail = None
    for name in kernel_names:
        heavy = name.startswith(("conv2d", "gemm_tcgen05", "depthwiseConv2D", "batchMatMul", "avgPool", "pool2d"))
        if heavy and layer < len(sizes):
            out.append(per_layer[layer])
            cur = sizes[layer]
            layer += 1
            if layer == len(sizes):
                n = NUM_CLASSES                     # the 8 stages of tf.softmax (ops/softmax.ts:57-63)
                tail = [n + 1, 2 * n + 1, 2 * n, n + 1, 2, 3, 2 * n + 1, 2 * n]
        elif tail:
            out.append(4 * batch * tail.pop(0))
        else:
            out.append(8 * batch * cur)            # add(bias) or clipByValue: one read, one write
    assert layer == len(sizes) and not tail, "kernel list does not cover the network"
    return out


def algorithmic_bytes_per_image(quantized=False):
    """Bytes one image moves if every tensor is touched once and epilogues are fused:
    4*(|x| + |y|) per layer; weights are counted separately by weight_bytes()."""
    total = 0
    h = w = 224
    c = 3
    for name, kind, shape, s in layer_specs():
        if name == "fc":
            total += 4 * (7 * 7 * c + c)          # global average pool: in + out
            total += 4 * (c + NUM_CLASSES)        # fc
            total += 4 * (NUM_CLASSES * 2)        # softmax
            break
        ho, wo = -(-h // s), -(-w // s)
        co = c if kind == "dw" else shape[3]
        total += 4 * (h * w * c + ho * wo * co)
        h, w, c = ho, wo, co
    return total


def weight_bytes(quantized=False):
    total = 0
    for name, kind, shape, _ in layer_specs():
        n = int(np.prod(shape))
        cout = shape[2] if kind == "dw" else shape[3]
        total += n * (1 if quantized else 4) + 4 * cout
    return total


def flops_per_image():
    total = 0
    h = w = 224
    c = 3
    for name, kind, shape, s in layer_specs():
        if name == "fc":
            total += 7 * 7 * c + 2 * c * NUM_CLASSES
            break
        ho, wo = -(-h // s), -(-w // s)
        if kind == "dw":
            total += 2 * ho * wo * c * 9
            co = c
        else:
            co = shape[3]
            total += 2 * ho * wo * co * shape[0] * shape[1] * shape[2]
        h, w, c = ho, wo, co
    return total
