"""The reference-side binding (js/) cannot be compiled or run on machines without Node, so these
tests keep it honest by other means: the generated N-API addon must be exactly what the header
implies, must export every entry point of the header, must pass a C++ syntax and type check
against a declarations-only stub of node_api.h, and the TypeScript KernelBackend subclass must
define every method the executable Python mirror defines and call only functions the addon
exports."""
import inspect
import os
import re
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
JS = os.path.join(ROOT, "js")
sys.path.insert(0, JS)

import gen_binding  # noqa: E402


def _read(name):
    return open(os.path.join(JS, name)).read()


def test_generated_files_are_current():
    cc, dts = gen_binding.generate()
    assert _read("binding.cc") == cc, "run `python js/gen_binding.py`"
    assert _read("binding.d.ts") == dts, "run `python js/gen_binding.py`"


def test_every_header_export_is_bound():
    from tfjs_core_b200 import _ffi
    names = [name for _, name, _ in gen_binding.parse_header()]
    assert sorted(names) == sorted(_ffi.SIGNATURES), "header and ctypes table disagree"
    cc = _read("binding.cc")
    for name in names:
        assert re.search(r"\b%s\(" % name, cc), f"{name} is not called by binding.cc"
    # every generated function is registered under its camelCase name
    for name in names:
        if name in gen_binding.HAND_WRITTEN:
            continue
        assert f'EXPORT("{gen_binding.js_name(name)}"' in cc


def test_parameter_counts_match_the_ctypes_table():
    from tfjs_core_b200 import _ffi
    for _, name, params in gen_binding.parse_header():
        assert len(params) == len(_ffi.SIGNATURES[name][1]), name


def test_addon_source_passes_a_syntax_check():
    stub = os.path.join(ROOT, "tests", "napi_stub")
    r = subprocess.run(["g++", "-std=c++14", "-fsyntax-only", "-Wall", "-Werror", "-I", stub, "-I",
                        os.path.join(ROOT, "include"), os.path.join(JS, "binding.cc")], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-4000:]


def test_typescript_backend_mirrors_the_python_backend():
    from tfjs_core_b200.backend_cuda import BackendCuda
    ts = _read("backend_cuda.ts")
    ts_methods = set(re.findall(r"^  (?:private |static |async |private static )*(\w+)(?:<[^>]*>)?\(", ts, flags=re.M))
    py_methods = {n for n, f in inspect.getmembers(BackendCuda, inspect.isfunction) if not n.startswith("_")}
    # host-pointer writes are the TypedArray form of write / writeAsync in JavaScript
    py_methods -= {"writeFromHostPointer"}
    missing = sorted(py_methods - ts_methods)
    assert not missing, f"methods of the Python BackendCuda missing from backend_cuda.ts: {missing}"
    # the methods of KernelBackend that the path needs (backend.ts:92-486)
    needed = {"register", "write", "readSync", "read", "disposeData", "memory", "time", "floatPrecision",
              "epsilon", "dispose", "batchMatMul", "fusedBatchMatMul", "add", "subtract", "multiply",
              "realDivide", "sum", "argMax", "max", "notEqual", "exp", "log", "relu", "prelu", "int", "clip",
              "step", "conv2d", "fusedConv2d", "conv2dDerInput", "conv2dDerFilter", "depthwiseConv2D",
              "depthwiseConv2DDerInput", "depthwiseConv2DDerFilter", "maxPool", "maxPoolBackprop", "avgPool",
              "avgPoolBackprop", "reshape", "cast", "transpose"}
    assert not (needed - ts_methods), sorted(needed - ts_methods)


def test_typescript_calls_only_exported_functions():
    dts = _read("binding.d.ts")
    exported = set(re.findall(r"^export function (\w+)", dts, flags=re.M))
    for src in ("backend_cuda.ts", "index.ts", "sharded.ts"):
        for fn in re.findall(r"\bbinding\.(\w+)\(", _read(src)):
            assert fn in exported, f"{src} calls binding.{fn}, which the addon does not export"
        code = re.sub(r"/\*.*?\*/|//[^\n]*", "", _read(src), flags=re.S)
        for fn in re.findall(r"\bbinding\.(\w+)\b(?!\()", code):
            assert fn in exported or fn in ("Handle", "EpilogueLike", "HostBuffer", "Conv2DInfoLike"), (src, fn)


def test_conv_info_fields_are_all_marshalled():
    """tfjs_conv2d_info and the N-API flattening of Conv2DInfo name the same fields."""
    from tfjs_core_b200 import _ffi
    cc = _read("binding.cc")
    for field, _ in _ffi.ConvInfo._fields_:
        if field.startswith("pad"):
            assert f"c.{field} = " in cc
        else:
            assert f"F({field});" in cc, field
