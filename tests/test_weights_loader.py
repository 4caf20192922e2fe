"""tf.io.loadWeights / decodeWeights restated for this backend, against the reference's own spec
cases (io/weights_loader_test.ts, io/io_utils_test.ts), transcribed as data with their line
numbers.  Runs on the CPU with a recording backend; the GPU variant at the bottom loads a
quantised MobileNet manifest from disk and checks the forward pass against the directly
registered network.
"""
import struct

import numpy as np
import pytest

import tfjs_core_b200 as tfb
from gpu_util import tf  # noqa: F401  (session fixture: the cuda backend)
from tfjs_core_b200 import mobilenet, weights_loader
from tfjs_core_b200.engine import ENGINE


class RecordingBackend:
    """Host-memory KernelBackend stand-in that records what the loader hands to the device."""

    def __init__(self):
        self.data = {}
        self.quantized_calls = []

    def register(self, data_id, shape, dtype):
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
        pass

    def registerQuantized(self, shape, q, scale, min_):
        self.quantized_calls.append((list(shape), np.array(q, copy=True), scale, min_))
        values = (np.asarray(q).astype(np.float64) * scale + min_).astype(np.float32)
        return tfb.ops.tensor(values, shape, "float32")


@pytest.fixture()
def host_backend():
    prev = ENGINE.backendName
    bk = RecordingBackend()
    ENGINE.registerBackend("recording", lambda: bk, 1000)
    assert ENGINE.setBackend("recording")
    yield bk
    ENGINE.removeBackend("recording")
    if prev:
        ENGINE.setBackend(prev)


def f32(*v):
    return np.array(v, "<f4").tobytes()


def i32(*v):
    return np.array(v, "<i4").tobytes()


class Files:
    """setupFakeWeightFiles (weights_loader_test.ts:23-32) with a fetch counter."""

    def __init__(self, files):
        self.files, self.calls = files, 0

    def __call__(self, paths):
        self.calls += len(paths)
        return [self.files[p] for p in paths]


def check(t, values, shape, dtype):
    assert t.shape == shape and t.dtype == dtype
    np.testing.assert_allclose(t.dataSync().reshape(-1), np.array(values, np.float64), atol=1e-3, rtol=0)


TWO_GROUPS = [
    {"paths": ["weightfile0"], "weights": [{"name": "weight0", "dtype": "float32", "shape": [2]},
                                            {"name": "weight1", "dtype": "float32", "shape": [3]}]},
    {"paths": ["weightfile1"], "weights": [{"name": "weight2", "dtype": "float32", "shape": [3, 1]},
                                            {"name": "weight3", "dtype": "float32", "shape": []}]},
]
TWO_GROUP_FILES = {"./weightfile0": f32(1, 2, 3, 4, 5), "./weightfile1": f32(6, 7, 8, 9)}


def test_one_group_one_weight(host_backend):
    # weights_loader_test.ts:34-54
    files = Files({"./weightfile0": f32(1, 2, 3)})
    manifest = [{"paths": ["weightfile0"], "weights": [{"name": "weight0", "dtype": "float32", "shape": [3]}]}]
    w = weights_loader.load_weights(manifest, "./", ["weight0"], fetch=files)
    assert files.calls == 1 and list(w) == ["weight0"]
    check(w["weight0"], [1, 2, 3], [3], "float32")


@pytest.mark.parametrize("names,expect", [
    (["weight0"], {"weight0": ([1, 2], [2])}),                                  # :56-78
    (["weight1"], {"weight1": ([3, 4, 5], [3])}),                               # :80-102
    (["weight0", "weight1"], {"weight0": ([1, 2], [2]), "weight1": ([3, 4, 5], [3])}),  # :104-132
])
def test_one_group_two_weights(host_backend, names, expect):
    files = Files({"./weightfile0": f32(1, 2, 3, 4, 5)})
    manifest = [{"paths": ["weightfile0"], "weights": [{"name": "weight0", "dtype": "float32", "shape": [2]},
                                                       {"name": "weight1", "dtype": "float32", "shape": [3]}]}]
    w = weights_loader.load_weights(manifest, "./", names, fetch=files)
    assert files.calls == 1 and sorted(w) == sorted(expect)
    for k, (vals, shape) in expect.items():
        check(w[k], vals, shape, "float32")


def test_one_group_mixed_dtypes(host_backend):
    # weights_loader_test.ts:134-176: int32 x2, one bool byte, float32 x3 at unaligned offsets
    buf = struct.pack("<iiBfff", 1, 2, 1, 3.0, 4.0, 5.0)
    manifest = [{"paths": ["weightfile0"], "weights": [{"name": "weight0", "dtype": "int32", "shape": [2]},
                                                       {"name": "weight1", "dtype": "bool", "shape": []},
                                                       {"name": "weight2", "dtype": "float32", "shape": [3]}]}]
    w = weights_loader.load_weights(manifest, "./", ["weight0", "weight1", "weight2"],
                                    fetch=Files({"./weightfile0": buf}))
    check(w["weight0"], [1, 2], [2], "int32")
    check(w["weight1"], [1], [], "bool")
    check(w["weight2"], [3, 4, 5], [3], "float32")


def test_one_weight_sharded_over_three_files(host_backend):
    # weights_loader_test.ts:178-205
    files = Files({"./weightfile0": f32(1, 2, 3, 4, 5), "./weightsfile1": f32(1.1, 2.2),
                   "./weightsfile2": f32(10, 20, 30)})
    manifest = [{"paths": ["weightfile0", "weightsfile1", "weightsfile2"],
                 "weights": [{"name": "weight0", "dtype": "float32", "shape": [5, 2]}]}]
    w = weights_loader.load_weights(manifest, "./", ["weight0"], fetch=files)
    assert files.calls == 3
    check(w["weight0"], [1, 2, 3, 4, 5, 1.1, 2.2, 10, 20, 30], [5, 2], "float32")


def test_two_weights_sharded_with_a_shard_spanning_both(host_backend):
    # weights_loader_test.ts:207-249: shard1 holds the end of weight0 and the start of weight1
    files = Files({"./weightfile0": i32(1, 2, 3, 4, 5), "./weightsfile1": i32(10, 20) + f32(3.0, 4.0, 5.0),
                   "./weightsfile2": f32(10, 20, 30)})
    manifest = [{"paths": ["weightfile0", "weightsfile1", "weightsfile2"],
                 "weights": [{"name": "weight0", "dtype": "int32", "shape": [7, 1]},
                             {"name": "weight1", "dtype": "float32", "shape": [3, 2]}]}]
    w = weights_loader.load_weights(manifest, "./", ["weight0", "weight1"], fetch=files)
    assert files.calls == 3
    check(w["weight0"], [1, 2, 3, 4, 5, 10, 20], [7, 1], "int32")
    check(w["weight1"], [3, 4, 5, 10, 20, 30], [3, 2], "float32")


@pytest.mark.parametrize("names,fetches,expect", [
    (["weight0", "weight1"], 1, {"weight0": ([1, 2], [2]), "weight1": ([3, 4, 5], [3])}),       # :251-291
    (["weight0", "weight2"], 2, {"weight0": ([1, 2], [2]), "weight2": ([6, 7, 8], [3, 1])}),    # :293-333
    (None, 2, {"weight0": ([1, 2], [2]), "weight1": ([3, 4, 5], [3]), "weight2": ([6, 7, 8], [3, 1]),
               "weight3": ([9], [])}),                                                          # :335-385
])
def test_two_groups(host_backend, names, fetches, expect):
    files = Files(TWO_GROUP_FILES)
    w = weights_loader.load_weights(TWO_GROUPS, "./", names, fetch=files)
    assert files.calls == fetches and sorted(w) == sorted(expect)
    for k, (vals, shape) in expect.items():
        check(w[k], vals, shape, "float32")


def test_missing_weight_and_unknown_dtype_throw(host_backend):
    manifest = [{"paths": ["weightfile0"], "weights": [{"name": "weight0", "dtype": "float32", "shape": [3]}]}]
    with pytest.raises(ValueError, match="Could not find weights in manifest with names: doesntexist"):
        weights_loader.load_weights(manifest, "./", ["doesntexist"], fetch=Files({"./weightfile0": f32(1, 2, 3)}))  # :387-402
    manifest[0]["weights"][0]["dtype"] = "null"
    with pytest.raises(ValueError):
        weights_loader.load_weights(manifest, "./", ["weight0"], fetch=Files({"./weightfile0": f32(1, 2, 3)}))  # :404-424


@pytest.mark.parametrize("qdtype", ["uint8", "uint16"])
def test_quantized_weights(host_backend, qdtype):
    # weights_loader_test.ts:443-491: min -1, scale 0.1 -> float32 [-1, 3.8, 24.5], int32 [-1, 4, 25]
    raw = np.array([0, 48, 255, 0, 48, 255], "<u1" if qdtype == "uint8" else "<u2").tobytes()
    quant = {"min": -1, "scale": 0.1, "dtype": qdtype}
    manifest = [{"paths": ["weightfile0"],
                 "weights": [{"name": "weight0", "dtype": "float32", "shape": [3], "quantization": quant},
                             {"name": "weight1", "dtype": "int32", "shape": [3], "quantization": quant}]}]
    files = Files({"./weightfile0": raw})
    w = weights_loader.load_weights(manifest, "./", ["weight0", "weight1"], fetch=files)
    assert files.calls == 1
    check(w["weight0"], [-1, 3.8, 24.5], [3], "float32")
    assert np.array_equal(w["weight1"].dataSync(), [-1, 4, 25]) and w["weight1"].dtype == "int32"
    # uint8 float32 entries reach the backend as the raw bytes, everything else is expanded on the host
    if qdtype == "uint8":
        (shape, q, scale, mn), = host_backend.quantized_calls
        assert shape == [3] and q.tolist() == [0, 48, 255] and (scale, mn) == (0.1, -1.0)
    else:
        assert host_backend.quantized_calls == []
    host_backend.quantized_calls.clear()
    w = weights_loader.load_weights(manifest, "./", ["weight0"], fetch=Files({"./weightfile0": raw}),
                                    keep_quantized=False)
    check(w["weight0"], [-1, 3.8, 24.5], [3], "float32")
    assert host_backend.quantized_calls == []


def test_one_quantized_group_and_one_plain_group(host_backend):
    # weights_loader_test.ts:493-543
    quant = {"min": -1, "scale": 0.1, "dtype": "uint8"}
    manifest = [
        {"paths": ["weightfile0"],
         "weights": [{"name": "weight0", "dtype": "float32", "shape": [3], "quantization": quant},
                     {"name": "weight1", "dtype": "int32", "shape": [3], "quantization": quant}]},
        TWO_GROUPS[1],
    ]
    files = Files({"./weightfile0": bytes([0, 48, 255, 0, 48, 255]), "./weightfile1": f32(6, 7, 8, 9)})
    w = weights_loader.load_weights(manifest, "./", ["weight0", "weight2"], fetch=files)
    assert files.calls == 2 and sorted(w) == ["weight0", "weight2"]
    check(w["weight0"], [-1, 3.8, 24.5], [3], "float32")
    check(w["weight2"], [6, 7, 8], [3, 1], "float32")


def test_decode_weights_rejects_other_quantization_dtypes(host_backend):
    # io_utils.ts:125-131
    spec = [{"name": "w", "dtype": "float32", "shape": [2], "quantization": {"min": 0, "scale": 1, "dtype": "int8"}}]
    with pytest.raises(ValueError, match="unknown quantization dtype int8"):
        weights_loader.decode_weights(bytes(2), spec)


def test_string_entries_and_path_prefix(host_backend):
    # io_utils.ts:149-160 wire format: uint32 byte length, then the bytes
    buf = struct.pack("<I", 2) + b"hi" + struct.pack("<I", 0) + f32(7)
    specs = [{"name": "s", "dtype": "string", "shape": [2]}, {"name": "x", "dtype": "float32", "shape": [1]}]
    out = weights_loader.decode_weights(buf, specs)
    assert out["s"] == [b"hi", b""]
    check(out["x"], [7], [1], "float32")
    seen = []
    weights_loader.weights_loader_factory(lambda paths: seen.extend(paths) or [f32(1)])(
        [{"paths": ["a.bin"], "weights": [{"name": "w", "dtype": "float32", "shape": [1]}]}], "http://host/model")
    assert seen == ["http://host/model/a.bin"]  # weights_loader.ts:201-203: one '/' is inserted


def test_manifest_round_trip_of_the_quantised_network(host_backend, tmp_path):
    params = mobilenet.make_weights(4, quantized=True)
    manifest = mobilenet.write_manifest(params, str(tmp_path), shard_bytes=1 << 20)
    assert len(manifest[0]["paths"]) == 5  # 4.33 MB of bytes in 1 MiB shards
    named = weights_loader.model_dir_weights(str(tmp_path))
    assert len(named) == 56 and len(host_backend.quantized_calls) == 28
    for (shape, q, scale, mn), (name, _, _, _) in zip(host_backend.quantized_calls, mobilenet.layer_specs()):
        assert np.array_equal(q.reshape(shape), params[name]["q"]) and scale == params[name]["scale"]
    assert np.array_equal(named["pw13/bias"].dataSync(), params["pw13"]["b"])


@pytest.mark.gpu
def test_network_loaded_from_a_manifest_matches_direct_registration(tf, tmp_path):
    """A quantised MobileNet written as manifest + shard files, loaded back through loadWeights
    (the filter bytes go to the device unexpanded) and run: logits and probabilities equal,
    bit for bit, those of the network whose tensors were registered directly."""
    bk = tf.ENGINE.backend
    params = mobilenet.make_weights(4, quantized=True)
    mobilenet.write_manifest(params, str(tmp_path), shard_bytes=3 << 19)
    named = weights_loader.model_dir_weights(str(tmp_path))
    loaded = mobilenet.MobileNetV1.from_named_tensors(named, bk)
    direct = mobilenet.MobileNetV1(params, bk)
    x = mobilenet.make_input(7, 2)
    try:
        a = [t.dataSync() for t in loaded.forward_fused(tf.ops.tensor(x))]
        b = [t.dataSync() for t in direct.forward_fused(tf.ops.tensor(x))]
        assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
    finally:
        loaded.dispose()
        direct.dispose()
