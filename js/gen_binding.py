"""Generates js/binding.cc, the Node N-API addon that exposes the C ABI of include/tfjs_cuda.h
to JavaScript, and js/binding.d.ts, its TypeScript declaration.

The marshalling is mechanical, so it is generated from the header's own prototypes (the single
source of truth) and cannot drift from them: `python js/gen_binding.py` rewrites both files,
`python js/gen_binding.py --check` fails when the committed files differ from what the header
implies (tests/test_js_binding.py runs the check).

Conventions of the generated functions (camelCase of the C name without the `tfjs_cuda_` prefix):
  * handles (context, graph, event) are napi_external values;
  * tensor ids, extents and enums are JS numbers, `const int64_t*` / `const int32_t*` arrays are
    JS number arrays, `const char*` is a string;
  * `const void* host, size_t nbytes` / `void* host, size_t nbytes` / `const uint8_t* q` take a
    TypedArray (the byte length comes from the array);
  * `const tfjs_conv2d_info*` takes the op layer's Conv2DInfo object
    (tfjs-core/src/ops/conv_util.ts:43-64; padInfo is read from `.padInfo`), and
    `const tfjs_epilogue*` takes `{bias, biasLen, activation, prelu, preluLen, clipLo, clipHi}`
    or null;
  * a function without output parameters returns the status number; one with output parameters
    returns `{status, <name>: value, ...}`;
  * raw device pointers (tfjs_cuda_matmul_static_scratch, tensor_device_ptr, ctx_stream) are
    BigInt addresses.
Three entry points are written by hand below because they are not plain marshalling:
tensorReadPromise (KernelBackend.read: the wait for the copy's event runs in a napi_async_work so
the event loop is never blocked), hostAlloc / hostFree (pinned memory surfaced as an external
ArrayBuffer).
"""
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
HEADER = os.path.join(HERE, "..", "include", "tfjs_cuda.h")
OUT_CC = os.path.join(HERE, "binding.cc")
OUT_DTS = os.path.join(HERE, "binding.d.ts")

HAND_WRITTEN = {"tfjs_cuda_host_alloc", "tfjs_cuda_host_free"}
DEVICE_POINTER_FUNCS = {"tfjs_cuda_matmul_static_scratch"}


def parse_header(path=HEADER):
    """[(return type, name, [(type, param name)])] for every prototype in the header."""
    text = open(path).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    protos = []
    for m in re.finditer(r"^\s*((?:const\s+)?[\w]+\s*\**)\s*(tfjs_cuda_\w+)\s*\(([^;{]*)\)\s*;", text, flags=re.M):
        ret, name, params = m.group(1).strip(), m.group(2), m.group(3)
        plist = []
        for p in [q.strip() for q in " ".join(params.split()).split(",") if q.strip()]:
            pm = re.match(r"^(.*?)(\w+)$", p)
            ptype = pm.group(1).replace(" ", "")
            plist.append((ptype, pm.group(2)))
        protos.append((ret.replace(" ", ""), name, plist))
    return protos


def js_name(cname):
    parts = cname[len("tfjs_cuda_"):].split("_")
    return parts[0] + "".join(p.capitalize() for p in parts[1:])


INT_TYPES = {"tfjs_tensor_id", "int64_t", "int32_t", "int", "size_t"}
HANDLE_TYPES = {"tfjs_cuda_ctx", "tfjs_cuda_graph", "tfjs_cuda_event"}


def classify(cname, params):
    """[(kind, ctype, name)] with the `size_t nbytes` that follows a host buffer folded into it."""
    out = []
    i = 0
    while i < len(params):
        t, n = params[i]
        base = t.replace("const", "")
        nxt = params[i + 1] if i + 1 < len(params) else None
        if base.rstrip("*") in HANDLE_TYPES and base.endswith("**"):
            out.append(("handle_out", base[:-2], n))
        elif base.rstrip("*") in HANDLE_TYPES and base.endswith("*"):
            out.append(("handle_in", base[:-1], n))
        elif t in INT_TYPES:
            out.append(("int", t, n))
        elif t in ("float", "double"):
            out.append(("num", t, n))
        elif t == "constchar*":
            out.append(("string", t, n))
        elif t == "constchar**":
            out.append(("out_string", t, n))
        elif cname in DEVICE_POINTER_FUNCS and base in ("float*",):
            out.append(("devptr", t, n))
        elif t in ("constint64_t*", "constint32_t*"):
            out.append(("array_in", base[:-1], n))
        elif t == "consttfjs_conv2d_info*":
            out.append(("conv_info", t, n))
        elif t == "consttfjs_epilogue*":
            out.append(("epilogue", t, n))
        elif t == "tfjs_cuda_mem_stats*":
            out.append(("out_memstats", t, n))
        elif t in ("constvoid*", "void*") and nxt and nxt[0] == "size_t":
            out.append(("buffer_in" if t.startswith("const") else "buffer_out", t, n))
            i += 1  # the byte count is the TypedArray's
        elif t == "constuint8_t*":
            out.append(("bytes_in", t, n))
        elif t == "void**":
            out.append(("out_pointer", t, n))
        elif t in ("tfjs_tensor_id*", "int64_t*"):
            out.append(("out_int64", t, n))
        elif t == "int*":
            out.append(("out_int", t, n))
        elif t == "size_t*":
            out.append(("out_size", t, n))
        elif t == "float*":
            out.append(("out_float", t, n))
        else:
            raise ValueError(f"{cname}: no marshalling rule for parameter `{t} {n}`")
        i += 1
    return out


PROLOGUE = r'''// GENERATED by js/gen_binding.py from include/tfjs_cuda.h -- do not edit by hand.
//
// Node N-API addon for the B200 `cuda` backend of tfjs-core: one function per entry point of
// the C ABI (include/tfjs_cuda.h), pure marshalling.  js/backend_cuda.ts is the only caller.
// Build with node-gyp (js/binding.gyp); links against tfjs-core_b200/libtfjs_cuda.so.
#include <node_api.h>

#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

#include "tfjs_cuda.h"

namespace {

#define NAPI_OK(call)                                                   \
  do {                                                                  \
    if ((call) != napi_ok) {                                            \
      napi_throw_error(env, nullptr, "N-API call failed: " #call);      \
      return nullptr;                                                   \
    }                                                                   \
  } while (0)

constexpr size_t MAX_ARGS = 16;

struct Args {
  napi_env env;
  size_t argc = MAX_ARGS;
  napi_value argv[MAX_ARGS];
  bool ok = true;
  Args(napi_env e, napi_callback_info info) : env(e) {
    if (napi_get_cb_info(env, info, &argc, argv, nullptr, nullptr) != napi_ok) ok = false;
  }
  bool fail(const char* msg) {
    if (ok) napi_throw_type_error(env, nullptr, msg);
    ok = false;
    return false;
  }
  bool is_nullish(size_t i) {
    if (i >= argc) return true;
    napi_valuetype t;
    if (napi_typeof(env, argv[i], &t) != napi_ok) return true;
    return t == napi_undefined || t == napi_null;
  }
  void* handle(size_t i) {  // napi_external -> pointer (null / undefined -> nullptr)
    if (is_nullish(i)) return nullptr;
    void* p = nullptr;
    if (napi_get_value_external(env, argv[i], &p) != napi_ok) fail("expected a native handle");
    return p;
  }
  int64_t integer(size_t i) {
    int64_t v = 0;
    if (i >= argc || napi_get_value_int64(env, argv[i], &v) != napi_ok) fail("expected an integer");
    return v;
  }
  double number(size_t i) {
    double v = 0;
    if (i >= argc || napi_get_value_double(env, argv[i], &v) != napi_ok) fail("expected a number");
    return v;
  }
  std::string string(size_t i) {
    size_t len = 0;
    if (i >= argc || napi_get_value_string_utf8(env, argv[i], nullptr, 0, &len) != napi_ok) {
      fail("expected a string");
      return std::string();
    }
    std::string s(len, '\0');
    napi_get_value_string_utf8(env, argv[i], &s[0], len + 1, &len);
    return s;
  }
  template <typename T>
  std::vector<T> array(size_t i) {
    std::vector<T> out;
    uint32_t n = 0;
    if (i >= argc || napi_get_array_length(env, argv[i], &n) != napi_ok) {
      fail("expected an array of numbers");
      return out;
    }
    out.resize(n);
    for (uint32_t k = 0; k < n; k++) {
      napi_value e;
      int64_t v = 0;
      if (napi_get_element(env, argv[i], k, &e) != napi_ok || napi_get_value_int64(env, e, &v) != napi_ok)
        fail("expected an array of numbers");
      out[k] = (T)v;
    }
    if (out.empty()) out.push_back(0);  // callers pass .data(); keep it non-null for rank 0
    return out;
  }
  // TypedArray / DataView / ArrayBuffer -> (pointer, byte length)
  void* buffer(size_t i, size_t* nbytes) {
    *nbytes = 0;
    if (is_nullish(i)) return nullptr;
    bool is_ta = false, is_ab = false, is_dv = false;
    napi_is_typedarray(env, argv[i], &is_ta);
    void* data = nullptr;
    if (is_ta) {
      napi_typedarray_type type;
      size_t len = 0, off = 0;
      napi_value ab;
      if (napi_get_typedarray_info(env, argv[i], &type, &len, &data, &ab, &off) != napi_ok) fail("bad TypedArray");
      size_t elem = 1;
      switch (type) {
        case napi_int16_array: case napi_uint16_array: elem = 2; break;
        case napi_int32_array: case napi_uint32_array: case napi_float32_array: elem = 4; break;
        case napi_float64_array: case napi_bigint64_array: case napi_biguint64_array: elem = 8; break;
        default: elem = 1;
      }
      *nbytes = len * elem;
      return data;
    }
    napi_is_arraybuffer(env, argv[i], &is_ab);
    if (is_ab) {
      if (napi_get_arraybuffer_info(env, argv[i], &data, nbytes) != napi_ok) fail("bad ArrayBuffer");
      return data;
    }
    napi_is_dataview(env, argv[i], &is_dv);
    if (is_dv) {
      napi_value ab;
      size_t off = 0;
      if (napi_get_dataview_info(env, argv[i], nbytes, &data, &ab, &off) != napi_ok) fail("bad DataView");
      return data;
    }
    fail("expected a TypedArray, DataView or ArrayBuffer");
    return nullptr;
  }
  void* device_pointer(size_t i) {  // BigInt address (null / undefined -> nullptr)
    if (is_nullish(i)) return nullptr;
    uint64_t v = 0;
    bool lossless = true;
    if (napi_get_value_bigint_uint64(env, argv[i], &v, &lossless) != napi_ok) fail("expected a BigInt device address");
    return (void*)(uintptr_t)v;
  }
  int64_t field_i64(napi_value obj, const char* name, bool* present = nullptr) {
    napi_value v;
    int64_t out = 0;
    napi_valuetype t = napi_undefined;
    if (napi_get_named_property(env, obj, name, &v) == napi_ok) napi_typeof(env, v, &t);
    if (present) *present = t == napi_number;
    if (t == napi_number) napi_get_value_int64(env, v, &out);
    return out;
  }
  double field_f64(napi_value obj, const char* name) {
    napi_value v;
    double out = 0;
    napi_valuetype t = napi_undefined;
    if (napi_get_named_property(env, obj, name, &v) == napi_ok) napi_typeof(env, v, &t);
    if (t == napi_number) napi_get_value_double(env, v, &out);
    return out;
  }
  // Conv2DInfo (tfjs-core/src/ops/conv_util.ts:43-64) -> tfjs_conv2d_info.  Only channelsLast is
  // accepted, as the header says; padInfo {top, bottom, left, right} is flattened.
  tfjs_conv2d_info conv_info(size_t i) {
    tfjs_conv2d_info c;
    memset(&c, 0, sizeof(c));
    if (is_nullish(i)) {
      fail("convInfo is required");
      return c;
    }
    napi_value o = argv[i];
    napi_value fmt;
    if (napi_get_named_property(env, o, "dataFormat", &fmt) == napi_ok) {
      napi_valuetype t;
      napi_typeof(env, fmt, &t);
      if (t == napi_string) {
        char buf[32];
        size_t len = 0;
        napi_get_value_string_utf8(env, fmt, buf, sizeof(buf), &len);
        if (strcmp(buf, "channelsLast") != 0) fail("the cuda backend takes channelsLast (NHWC) convolutions only");
      }
    }
#define F(name) c.name = (int32_t)field_i64(o, #name)
    F(batchSize); F(inHeight); F(inWidth); F(inChannels); F(outHeight); F(outWidth); F(outChannels);
    F(strideHeight); F(strideWidth); F(dilationHeight); F(dilationWidth); F(filterHeight); F(filterWidth);
    F(effectiveFilterHeight); F(effectiveFilterWidth);
#undef F
    napi_value pad;
    napi_valuetype pt = napi_undefined;
    if (napi_get_named_property(env, o, "padInfo", &pad) == napi_ok) napi_typeof(env, pad, &pt);
    if (pt == napi_object) {
      c.padTop = (int32_t)field_i64(pad, "top");
      c.padBottom = (int32_t)field_i64(pad, "bottom");
      c.padLeft = (int32_t)field_i64(pad, "left");
      c.padRight = (int32_t)field_i64(pad, "right");
    }
    return c;
  }
  // {bias, biasLen, activation, prelu, preluLen, clipLo, clipHi} | null -> tfjs_epilogue
  bool epilogue(size_t i, tfjs_epilogue* e) {
    memset(e, 0, sizeof(*e));
    if (is_nullish(i)) return false;
    napi_value o = argv[i];
    e->bias = field_i64(o, "bias");
    e->bias_len = field_i64(o, "biasLen");
    e->activation = (int32_t)field_i64(o, "activation");
    e->prelu = field_i64(o, "prelu");
    e->prelu_len = field_i64(o, "preluLen");
    e->clip_lo = (float)field_f64(o, "clipLo");
    e->clip_hi = (float)field_f64(o, "clipHi");
    return true;
  }
};

struct Result {  // {status, ...outs}
  napi_env env;
  napi_value obj;
  Result(napi_env e, int status) : env(e) {
    napi_create_object(env, &obj);
    set_i64("status", status);
  }
  void set(const char* k, napi_value v) { napi_set_named_property(env, obj, k, v); }
  void set_i64(const char* k, int64_t v) { napi_value n; napi_create_int64(env, v, &n); set(k, n); }
  void set_f64(const char* k, double v) { napi_value n; napi_create_double(env, v, &n); set(k, n); }
  void set_str(const char* k, const char* s) { napi_value n; napi_create_string_utf8(env, s ? s : "", NAPI_AUTO_LENGTH, &n); set(k, n); }
  void set_ptr(const char* k, const void* p) { napi_value n; napi_create_bigint_uint64(env, (uint64_t)(uintptr_t)p, &n); set(k, n); }
  void set_handle(const char* k, void* p) {
    napi_value n;
    if (p) napi_create_external(env, p, nullptr, nullptr, &n); else napi_get_null(env, &n);
    set(k, n);
  }
};

napi_value status_value(napi_env env, int64_t status) {
  napi_value n;
  napi_create_int64(env, status, &n);
  return n;
}

// ---- hand-written entry points ---------------------------------------------------------------

// hostAlloc(nbytes) -> {status, buffer}: pinned host memory as an external ArrayBuffer; the
// finalizer returns it with tfjs_cuda_host_free when the ArrayBuffer is collected.
void FreePinned(napi_env, void* data, void*) { tfjs_cuda_host_free(data); }
napi_value HostAlloc(napi_env env, napi_callback_info info) {
  Args a(env, info);
  const int64_t nbytes = a.integer(0);
  if (!a.ok) return nullptr;
  void* p = nullptr;
  const int rc = tfjs_cuda_host_alloc(&p, (size_t)nbytes);
  Result r(env, rc);
  if (rc == TFJS_CUDA_OK) {
    napi_value ab;
    NAPI_OK(napi_create_external_arraybuffer(env, p, (size_t)nbytes, FreePinned, nullptr, &ab));
    r.set("buffer", ab);
  }
  return r.obj;
}
// hostFree(buffer): detaches the ArrayBuffer, which runs the finalizer above.
napi_value HostFree(napi_env env, napi_callback_info info) {
  Args a(env, info);
  if (!a.ok || a.argc < 1) return nullptr;
  NAPI_OK(napi_detach_arraybuffer(env, a.argv[0]));
  return status_value(env, TFJS_CUDA_OK);
}

// tensorReadPromise(ctx, id, typedArray) -> Promise<typedArray>: KernelBackend.read
// (tfjs-core/src/backends/backend.ts:95-97).  The copy is enqueued on the calling thread
// (tfjs_cuda_tensor_read_async); only the wait for its event runs on a worker thread, which
// touches the event and nothing else of the context, so the one-thread-per-context rule holds
// and the event loop is never blocked (precedent: the fence + promise of
// tfjs-core/src/backends/webgl/backend_webgl.ts:425-499).
struct ReadJob {
  napi_async_work work = nullptr;
  napi_deferred deferred = nullptr;
  napi_ref target = nullptr;  // keeps the destination TypedArray alive until the copy has landed
  tfjs_cuda_event* event = nullptr;
  int status = 0;
};
void ReadExecute(napi_env, void* data) {
  ReadJob* job = (ReadJob*)data;
  job->status = tfjs_cuda_event_wait(job->event, -1);
}
void ReadComplete(napi_env env, napi_status, void* data) {
  ReadJob* job = (ReadJob*)data;
  tfjs_cuda_event_destroy(job->event);
  napi_value target;
  napi_get_reference_value(env, job->target, &target);
  if (job->status == TFJS_CUDA_OK) {
    napi_resolve_deferred(env, job->deferred, target);
  } else {
    napi_value msg, err;
    napi_create_string_utf8(env, "cuda backend: asynchronous read failed", NAPI_AUTO_LENGTH, &msg);
    napi_create_error(env, nullptr, msg, &err);
    napi_reject_deferred(env, job->deferred, err);
  }
  napi_delete_reference(env, job->target);
  napi_delete_async_work(env, job->work);
  delete job;
}
napi_value TensorReadPromise(napi_env env, napi_callback_info info) {
  Args a(env, info);
  tfjs_cuda_ctx* ctx = (tfjs_cuda_ctx*)a.handle(0);
  const int64_t id = a.integer(1);
  size_t nbytes = 0;
  void* host = a.buffer(2, &nbytes);
  if (!a.ok) return nullptr;
  ReadJob* job = new ReadJob();
  const int rc = tfjs_cuda_tensor_read_async(ctx, id, host, nbytes, &job->event);
  if (rc != TFJS_CUDA_OK) {
    delete job;
    napi_throw_error(env, nullptr, tfjs_cuda_last_error(ctx));
    return nullptr;
  }
  napi_value promise, name;
  NAPI_OK(napi_create_promise(env, &job->deferred, &promise));
  NAPI_OK(napi_create_reference(env, a.argv[2], 1, &job->target));
  NAPI_OK(napi_create_string_utf8(env, "tfjs_cuda_read", NAPI_AUTO_LENGTH, &name));
  NAPI_OK(napi_create_async_work(env, nullptr, name, ReadExecute, ReadComplete, job, &job->work));
  NAPI_OK(napi_queue_async_work(env, job->work));
  return promise;
}

// ---- generated entry points ------------------------------------------------------------------
'''

EPILOGUE_TMPL = r'''
}  // namespace

#define EXPORT(js, fn)                                                        \
  do {                                                                        \
    napi_value f;                                                             \
    if (napi_create_function(env, js, NAPI_AUTO_LENGTH, fn, nullptr, &f) != napi_ok) return nullptr; \
    if (napi_set_named_property(env, exports, js, f) != napi_ok) return nullptr; \
  } while (0)

static napi_value Init(napi_env env, napi_value exports) {
  EXPORT("hostAlloc", HostAlloc);
  EXPORT("hostFree", HostFree);
  EXPORT("tensorReadPromise", TensorReadPromise);
%s  return exports;
}

NAPI_MODULE(NODE_GYP_MODULE_NAME, Init)
'''


def cpp_func_name(cname):
    n = js_name(cname)
    return n[0].upper() + n[1:]


def gen_function(ret, cname, params):
    kinds = classify(cname, params)
    lines = [f"// {cname}", f"napi_value {cpp_func_name(cname)}(napi_env env, napi_callback_info cbinfo) {{", "  Args argz(env, cbinfo);"]
    call_args, outs = [], []
    js_index = 0
    for kind, ctype, name in kinds:
        if kind == "handle_in":
            lines.append(f"  {ctype}* {name} = ({ctype}*)argz.handle({js_index});")
            call_args.append(name)
            js_index += 1
        elif kind == "handle_out":
            lines.append(f"  {ctype}* {name} = nullptr;")
            call_args.append(f"&{name}")
            outs.append(("handle", name))
        elif kind == "int":
            lines.append(f"  const {ctype} {name} = ({ctype})argz.integer({js_index});")
            call_args.append(name)
            js_index += 1
        elif kind == "num":
            lines.append(f"  const {ctype} {name} = ({ctype})argz.number({js_index});")
            call_args.append(name)
            js_index += 1
        elif kind == "string":
            lines.append(f"  const std::string {name} = argz.string({js_index});")
            call_args.append(f"{name}.c_str()")
            js_index += 1
        elif kind == "array_in":
            lines.append(f"  const std::vector<{ctype}> {name} = argz.array<{ctype}>({js_index});")
            call_args.append(f"{name}.data()")
            js_index += 1
        elif kind == "conv_info":
            lines.append(f"  const tfjs_conv2d_info {name} = argz.conv_info({js_index});")
            call_args.append(f"&{name}")
            js_index += 1
        elif kind == "epilogue":
            lines.append(f"  tfjs_epilogue {name};")
            lines.append(f"  const bool has_{name} = argz.epilogue({js_index}, &{name});")
            call_args.append(f"has_{name} ? &{name} : nullptr")
            js_index += 1
        elif kind in ("buffer_in", "buffer_out"):
            lines.append(f"  size_t {name}_bytes = 0;")
            lines.append(f"  void* {name} = argz.buffer({js_index}, &{name}_bytes);")
            call_args.append(name)
            call_args.append(f"{name}_bytes")
            js_index += 1
        elif kind == "bytes_in":
            lines.append(f"  size_t {name}_bytes = 0;")
            lines.append(f"  const uint8_t* {name} = (const uint8_t*)argz.buffer({js_index}, &{name}_bytes);")
            call_args.append(name)
            js_index += 1
        elif kind == "devptr":
            lines.append(f"  float* {name} = (float*)argz.device_pointer({js_index});")
            call_args.append(name)
            js_index += 1
        elif kind == "out_memstats":
            lines.append(f"  tfjs_cuda_mem_stats {name};")
            lines.append(f"  memset(&{name}, 0, sizeof({name}));")
            call_args.append(f"&{name}")
            outs.append(("memstats", name))
        elif kind == "out_pointer":
            lines.append(f"  void* {name} = nullptr;")
            call_args.append(f"&{name}")
            outs.append(("ptr", name))
        elif kind == "out_int64":
            lines.append(f"  int64_t {name} = 0;")
            call_args.append(f"&{name}")
            outs.append(("i64", name))
        elif kind == "out_int":
            lines.append(f"  int {name} = 0;")
            call_args.append(f"&{name}")
            outs.append(("i64", name))
        elif kind == "out_size":
            lines.append(f"  size_t {name} = 0;")
            call_args.append(f"&{name}")
            outs.append(("i64", name))
        elif kind == "out_float":
            lines.append(f"  float {name} = 0.f;")
            call_args.append(f"&{name}")
            outs.append(("f64", name))
        elif kind == "out_string":
            lines.append(f"  const char* {name} = nullptr;")
            call_args.append(f"&{name}")
            outs.append(("str", name))
    lines.append("  if (!argz.ok) return nullptr;")
    call = f"{cname}({', '.join(call_args)})"
    if ret == "constchar*":
        lines.append(f"  const char* s = {call};")
        lines.append("  napi_value out;")
        lines.append('  NAPI_OK(napi_create_string_utf8(env, s ? s : "", NAPI_AUTO_LENGTH, &out));')
        lines.append("  return out;")
    elif ret == "void*":
        lines.append(f"  void* p = {call};")
        lines.append("  napi_value out;")
        lines.append("  NAPI_OK(napi_create_bigint_uint64(env, (uint64_t)(uintptr_t)p, &out));")
        lines.append("  return out;")
    elif not outs:
        lines.append(f"  return status_value(env, (int64_t){call});")
    else:
        lines.append(f"  Result r(env, (int){call});")
        for kind, name in outs:
            if kind == "handle":
                lines.append(f'  r.set_handle("{name}", {name});')
            elif kind == "memstats":
                for f in ("num_tensors", "bytes_in_use", "bytes_reserved", "num_buffers_cached", "num_device_allocs"):
                    lines.append(f'  r.set_i64("{f}", {name}.{f});')
            elif kind == "ptr":
                lines.append(f'  r.set_ptr("{name}", {name});')
            elif kind == "i64":
                lines.append(f'  r.set_i64("{name}", (int64_t){name});')
            elif kind == "f64":
                lines.append(f'  r.set_f64("{name}", {name});')
            elif kind == "str":
                lines.append(f'  r.set_str("{name}", {name});')
        lines.append("  return r.obj;")
    lines.append("}")
    return "\n".join(lines), kinds, outs


TS_TYPES = {"handle_in": "Handle", "int": "number", "num": "number", "string": "string", "array_in": "number[]",
            "conv_info": "Conv2DInfoLike", "epilogue": "EpilogueLike|null", "buffer_in": "HostBuffer",
            "buffer_out": "HostBuffer", "bytes_in": "Uint8Array", "devptr": "bigint|null"}
TS_OUT = {"handle": "Handle", "ptr": "bigint", "i64": "number", "f64": "number", "str": "string"}


def generate():
    protos = parse_header()
    body, exports, dts = [], [], []
    for ret, cname, params in protos:
        if cname in HAND_WRITTEN:
            continue
        code, kinds, outs = gen_function(ret, cname, params)
        body.append(code)
        exports.append(f'  EXPORT("{js_name(cname)}", {cpp_func_name(cname)});\n')
        args = ", ".join(f"{n}: {TS_TYPES[k]}" for k, _, n in kinds if k in TS_TYPES)
        if ret == "constchar*":
            rtype = "string"
        elif ret == "void*":
            rtype = "bigint"
        elif not outs:
            rtype = "number"
        else:
            fields = ["status: number"]
            for kind, name in outs:
                if kind == "memstats":
                    fields += [f"{f}: number" for f in ("num_tensors", "bytes_in_use", "bytes_reserved",
                                                         "num_buffers_cached", "num_device_allocs")]
                else:
                    fields.append(f"{name}: {TS_OUT[kind]}")
            rtype = "{" + ", ".join(fields) + "}"
        dts.append(f"export function {js_name(cname)}({args}): {rtype};  // {cname}")
    cc = PROLOGUE + "\n\n".join(body) + "\n" + (EPILOGUE_TMPL % "".join(exports))
    d = ("// GENERATED by js/gen_binding.py from include/tfjs_cuda.h -- do not edit by hand.\n"
         "// Type declarations of the N-API addon (js/binding.cc).\n"
         "export type Handle = object;  // napi_external: context, graph or event\n"
         "export type HostBuffer = ArrayBufferView|ArrayBuffer;\n"
         "export interface Conv2DInfoLike {\n"
         "  batchSize: number; inHeight: number; inWidth: number; inChannels: number; outHeight: number;\n"
         "  outWidth: number; outChannels: number; strideHeight: number; strideWidth: number;\n"
         "  dilationHeight: number; dilationWidth: number; filterHeight: number; filterWidth: number;\n"
         "  effectiveFilterHeight: number; effectiveFilterWidth: number; dataFormat?: string;\n"
         "  padInfo: {top: number, bottom: number, left: number, right: number};\n"
         "}\n"
         "export interface EpilogueLike {\n"
         "  bias: number; biasLen: number; activation: number; prelu: number; preluLen: number;\n"
         "  clipLo: number; clipHi: number;\n"
         "}\n"
         "export function hostAlloc(nbytes: number): {status: number, buffer?: ArrayBuffer};  // tfjs_cuda_host_alloc\n"
         "export function hostFree(buffer: ArrayBuffer): number;  // tfjs_cuda_host_free (through the finalizer)\n"
         "export function tensorReadPromise<T extends ArrayBufferView>(ctx: Handle, id: number, into: T): Promise<T>;"
         "  // tfjs_cuda_tensor_read_async + tfjs_cuda_event_wait\n" + "\n".join(dts) + "\n")
    return cc, d


def main():
    cc, d = generate()
    if "--check" in sys.argv:
        stale = [p for p, want in ((OUT_CC, cc), (OUT_DTS, d)) if not os.path.exists(p) or open(p).read() != want]
        if stale:
            print("stale:", ", ".join(stale))
            return 1
        return 0
    open(OUT_CC, "w").write(cc)
    open(OUT_DTS, "w").write(d)
    return 0


if __name__ == "__main__":
    sys.exit(main())
