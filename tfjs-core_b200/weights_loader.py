"""tf.io.loadWeights / decodeWeights for the cuda backend: a tfjs weights manifest (JSON groups
of `paths` + `weights` entries) and its binary shard files become tensors, with uint8-quantised
float32 entries handed to the device as raw bytes (`registerQuantized`) instead of being expanded
on the host.

Follows io/weights_loader.ts:123-247 (group walk, per-entry byte offsets, shard concatenation,
name filter, error text) and io/io_utils.ts:111-177 (wire format of one entry: little-endian
values in manifest order; `quantization: {scale, min, dtype}` entries stored as uint8 / uint16
with value = q*scale + min; string entries as uint32 length + bytes).  Fetching is a caller
supplied function over paths, as in weightsLoaderFactory; `fetch_from_disk` is the Node-style
one.
"""
import math
import os

import numpy as np

from . import ops
from .engine import ENGINE, size_from_shape

# io/types.ts:23-29
DTYPE_VALUE_SIZE_MAP = {"float32": 4, "int32": 4, "uint16": 2, "uint8": 1, "bool": 1}
NUM_BYTES_STRING_LENGTH = 4  # io/io_utils.ts:24


def _js_round(v):
    """Math.round on an array of float64: nearest integer, ties towards +infinity."""
    return np.floor(np.asarray(v, np.float64) + 0.5)


def decode_weights(buffer, specs, keep_quantized=True):
    """decodeWeights (io/io_utils.ts:111-177): {name: Tensor} from one flat buffer holding the
    entries of `specs` back to back.

    keep_quantized: float32 entries quantised as uint8 stay uint8 in device memory when the
    active backend offers `registerQuantized` (the kernels dequantise with the same float64
    arithmetic, io_utils.ts:139); otherwise, and for uint16 or int32-typed quantised entries,
    the values are expanded here exactly as the reference does on the host.
    """
    buffer = memoryview(bytes(buffer))
    out = {}
    offset = 0
    for spec in specs:
        name, dtype, shape = spec["name"], spec["dtype"], list(spec["shape"])
        size = size_from_shape(shape)
        if "quantization" in spec:
            quant = spec["quantization"]
            qdtype = quant["dtype"]
            if qdtype not in ("uint8", "uint16"):
                raise ValueError(f"Weight {name} has unknown quantization dtype {qdtype}. "
                                 "Supported quantization dtypes are: 'uint8' and 'uint16'.")
            nbytes = size * DTYPE_VALUE_SIZE_MAP[qdtype]
            q = np.frombuffer(buffer[offset:offset + nbytes], dtype="<u1" if qdtype == "uint8" else "<u2")
            if q.size != size:
                raise ValueError(f"Weight {name}: the buffer ends before its {nbytes} bytes")
            scale, min_ = float(quant["scale"]), float(quant["min"])
            backend = ENGINE.backend
            if dtype == "float32":
                if keep_quantized and qdtype == "uint8" and hasattr(backend, "registerQuantized"):
                    out[name] = backend.registerQuantized(shape, q, scale, min_)
                else:
                    values = (q.astype(np.float64) * scale + min_).astype(np.float32)
                    out[name] = ops.tensor(values, shape, "float32")
            elif dtype == "int32":
                values = _js_round(q.astype(np.float64) * scale + min_).astype(np.int32)
                out[name] = ops.tensor(values, shape, "int32")
            else:
                raise ValueError(f"Unsupported dtype in weight '{name}': {dtype}")
            offset += nbytes
        elif dtype == "string":
            # host-side data in the reference too (a string tensor never reaches a kernel)
            values = []
            for _ in range(size):
                n = int(np.frombuffer(buffer[offset:offset + NUM_BYTES_STRING_LENGTH], dtype="<u4")[0])
                offset += NUM_BYTES_STRING_LENGTH
                values.append(bytes(buffer[offset:offset + n]))
                offset += n
            out[name] = values
        else:
            if dtype not in ("float32", "int32", "bool"):
                raise ValueError(f"Unsupported dtype in weight '{name}': {dtype}")
            nbytes = size * DTYPE_VALUE_SIZE_MAP[dtype]
            raw = buffer[offset:offset + nbytes]
            if len(raw) != nbytes:
                raise ValueError(f"Weight {name}: the buffer ends before its {nbytes} bytes")
            np_dtype = {"float32": "<f4", "int32": "<i4", "bool": "<u1"}[dtype]
            out[name] = ops.tensor(np.frombuffer(raw, dtype=np_dtype), shape, dtype)
            offset += nbytes
    return out


def weights_loader_factory(fetch_weights_function):
    """weightsLoaderFactory (io/weights_loader.ts:123-247).  `fetch_weights_function(paths)`
    returns one bytes-like object per path, in order."""

    def load(manifest, file_path_prefix="", weight_names=None, keep_quantized=True):
        group_to_fetch = [False] * len(manifest)
        group_weights = {}
        found = [False] * len(weight_names) if weight_names is not None else []
        all_names = []
        for gi, group in enumerate(manifest):
            group_offset = 0
            for entry in group["weights"]:
                raw_dtype = entry["quantization"]["dtype"] if "quantization" in entry else entry["dtype"]
                if raw_dtype not in DTYPE_VALUE_SIZE_MAP:
                    # the reference computes NaN bytes here and fails inside decodeWeights
                    if weight_names is None or entry["name"] in weight_names:
                        raise ValueError(f"Unsupported dtype in weight '{entry['name']}': {raw_dtype}")
                    nbytes = math.nan
                else:
                    nbytes = DTYPE_VALUE_SIZE_MAP[raw_dtype] * size_from_shape(entry["shape"])
                wanted = weight_names is None
                if weight_names is not None:
                    for wi, wn in enumerate(weight_names):
                        if wn == entry["name"]:
                            wanted = True
                            found[wi] = True
                if wanted:
                    group_to_fetch[gi] = True
                    group_weights.setdefault(gi, []).append((entry, group_offset, nbytes))
                all_names.append(entry["name"])
                group_offset += nbytes
        if not all(found):
            missing = [n for n, f in zip(weight_names, found) if not f]
            raise ValueError("Could not find weights in manifest with names: " + ", ".join(missing) +
                             ". \nManifest JSON has weights with names: " + ", ".join(all_names) + ".")
        groups = [gi for gi, f in enumerate(group_to_fetch) if f]
        urls = []
        for gi in groups:
            for path in manifest[gi]["paths"]:
                urls.append(file_path_prefix + ("" if file_path_prefix.endswith("/") else "/") + path)
        buffers = fetch_weights_function(urls)
        result = {}
        index = 0
        for gi in groups:
            n = len(manifest[gi]["paths"])
            group_buffer = b"".join(bytes(b) for b in buffers[index:index + n])
            for entry, group_offset, nbytes in group_weights[gi]:
                result.update(decode_weights(group_buffer[group_offset:group_offset + nbytes], [entry],
                                             keep_quantized))
            index += n
        return result

    return load


def fetch_from_disk(paths):
    out = []
    for p in paths:
        with open(p, "rb") as f:
            out.append(f.read())
    return out


def load_weights(manifest, file_path_prefix="", weight_names=None, fetch=fetch_from_disk, keep_quantized=True):
    """tf.io.loadWeights (io/weights_loader.ts:82-98) with the files read by `fetch`."""
    return weights_loader_factory(fetch)(manifest, file_path_prefix, weight_names, keep_quantized)


def encode_weights(named, quantize=()):
    """Writer used by tests and the benchmark's manifest round trip: the inverse of
    decode_weights for numpy arrays.  `named` is [(name, array)]; arrays whose name is in
    `quantize` are stored uint8 with scale = (max - min) / 255 (the converter's rule).
    Returns (specs, bytes)."""
    specs, chunks = [], []
    for name, arr in named:
        arr = np.asarray(arr)
        if name in quantize:
            lo, hi = float(arr.min()), float(arr.max())
            scale = (hi - lo) / 255.0 if hi > lo else 1.0
            q = np.clip(np.round((arr.astype(np.float64) - lo) / scale), 0, 255).astype(np.uint8)
            specs.append({"name": name, "dtype": "float32", "shape": list(arr.shape),
                          "quantization": {"min": lo, "scale": scale, "dtype": "uint8"}})
            chunks.append(q.tobytes())
        else:
            dtype = {"float32": "float32", "int32": "int32", "bool": "bool", "uint8": "bool"}[str(arr.dtype)]
            specs.append({"name": name, "dtype": dtype, "shape": list(arr.shape)})
            chunks.append(np.ascontiguousarray(arr, {"float32": "<f4", "int32": "<i4", "bool": "<u1"}[dtype]).tobytes())
    return specs, b"".join(chunks)


def model_dir_weights(directory, manifest_name="weights_manifest.json", weight_names=None):
    """Convenience: parse `<directory>/<manifest_name>` and load its shards from the same folder."""
    import json
    with open(os.path.join(directory, manifest_name)) as f:
        manifest = json.load(f)
    if isinstance(manifest, dict):  # model.json of tf.io: {"weightsManifest": [...]}
        manifest = manifest["weightsManifest"]
    return load_weights(manifest, directory, weight_names)
