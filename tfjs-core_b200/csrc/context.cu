// Context, caching allocator, tensor table, events, timing and graph capture.
//
// Plays the role of MathBackendCPU's storage half (tfjs-core/src/backends/cpu/
// backend_cpu.ts:102-254) and of the wasm backend's id-keyed tensor table
// (tfjs-backend-wasm/src/lib.cc:52-132), with device memory instead of typed arrays.
#include <chrono>
#include <thread>

#include "common.cuh"

int set_error(tfjs_cuda_ctx* ctx, int code, const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  if (ctx) ctx->last_error = buf;
  return code;
}

static thread_local std::string g_create_error;

int post_launch(tfjs_cuda_ctx* ctx, const char* what) {
  ctx->launch_count++;
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess)
    return set_error(ctx, TFJS_CUDA_ERR_CUDA, "launch of %s failed: %s", what,
                     cudaGetErrorString(e));
  if (ctx->debug_sync) {
    e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess)
      return set_error(ctx, TFJS_CUDA_ERR_CUDA, "%s failed: %s", what, cudaGetErrorString(e));
  }
  if (ctx->profiling && !ctx->capturing && ctx->profile_used + 1 < ctx->profile_events.size()) {
    cudaEventRecord(ctx->profile_events[ctx->profile_used + 1], ctx->stream);
    ctx->profile_names[ctx->profile_used] = what;
    ctx->profile_used++;
  }
  return TFJS_CUDA_OK;
}

// ---- per-kernel profile --------------------------------------------------------------------
// The stream is in-order, so the time between the events that bracket a launch is that
// kernel's duration (plus any idle gap before it, which vanishes once the host runs ahead).
extern "C" int tfjs_cuda_profile_begin(tfjs_cuda_ctx* ctx, int max_launches) {
  if (!ctx || max_launches < 1) return TFJS_CUDA_ERR_INVALID_ARG;
  TFJS_REQUIRE(ctx, !ctx->capturing, "cannot profile while capturing a graph");
  cudaSetDevice(ctx->device);
  while (ctx->profile_events.size() < (size_t)max_launches + 1) {
    cudaEvent_t ev;
    TFJS_CHECK_CUDA(ctx, cudaEventCreate(&ev));
    ctx->profile_events.push_back(ev);
  }
  ctx->profile_names.assign(ctx->profile_events.size(), nullptr);
  ctx->profile_used = 0;
  TFJS_CHECK_CUDA(ctx, cudaEventRecord(ctx->profile_events[0], ctx->stream));
  ctx->profiling = true;
  return TFJS_CUDA_OK;
}

extern "C" int tfjs_cuda_profile_end(tfjs_cuda_ctx* ctx, int* num_launches) {
  if (!ctx) return TFJS_CUDA_ERR_INVALID_ARG;
  ctx->profiling = false;
  cudaSetDevice(ctx->device);
  if (ctx->profile_used)
    TFJS_CHECK_CUDA(ctx, cudaEventSynchronize(ctx->profile_events[ctx->profile_used]));
  if (num_launches) *num_launches = (int)ctx->profile_used;
  return TFJS_CUDA_OK;
}

extern "C" int tfjs_cuda_profile_get(tfjs_cuda_ctx* ctx, int index, const char** name, float* ms) {
  if (!ctx) return TFJS_CUDA_ERR_INVALID_ARG;
  TFJS_REQUIRE(ctx, index >= 0 && (size_t)index < ctx->profile_used, "profile index out of range");
  float t = 0.f;
  TFJS_CHECK_CUDA(ctx, cudaEventElapsedTime(&t, ctx->profile_events[index], ctx->profile_events[index + 1]));
  if (name) *name = ctx->profile_names[index];
  if (ms) *ms = t;
  return TFJS_CUDA_OK;
}

// ---- allocator ---------------------------------------------------------------------------
// Buffers are recycled through per-size free lists so that the steady state of an inference
// loop never calls cudaMalloc.  Reuse is stream-ordered: everything runs on ctx->stream.
static size_t size_class(size_t n) {
  if (n == 0) return 0;
  if (n <= (1u << 20)) {
    size_t c = 512;
    while (c < n) c <<= 1;
    return c;
  }
  const size_t mb = 1u << 20;
  return (n + mb - 1) / mb * mb;
}

static void release_cached(tfjs_cuda_ctx* ctx) {
  for (auto& kv : ctx->free_lists) {
    for (void* p : kv.second) {
      cudaFree(p);
      ctx->bytes_reserved -= (int64_t)kv.first;
    }
    kv.second.clear();
  }
  ctx->num_cached = 0;
}

// ---- guard pattern behind every buffer (option "debug_canary") ------------------------------
constexpr size_t CANARY_BYTES = 256;
constexpr uint32_t CANARY_WORD = 0xA5C3F00Du;

__global__ void canary_fill_kernel(uint32_t* guard) { guard[threadIdx.x] = CANARY_WORD; }
__global__ void canary_check_kernel(const uint32_t* guard, int* status) {
  if (guard[threadIdx.x] != CANARY_WORD) atomicCAS(status, 0, STATUS_CANARY);
}

int ctx_alloc(tfjs_cuda_ctx* ctx, size_t nbytes, void** ptr, size_t* capacity) {
  *ptr = nullptr;
  *capacity = 0;
  if (nbytes == 0) return TFJS_CUDA_OK;
  const bool canary = ctx->debug_canary && !ctx->capturing;
  const size_t guard_at = (nbytes + 15) / 16 * 16;
  const size_t cls = size_class(canary ? guard_at + CANARY_BYTES : nbytes);
  if (ctx->capturing) {
    // Buffers released earlier in this capture can serve later captured kernels: the graph
    // replays its nodes in the captured order, so the reuse stays stream-ordered.
    auto rit = ctx->capturing->reusable.find(cls);
    if (rit != ctx->capturing->reusable.end() && !rit->second.empty()) {
      *ptr = rit->second.back();
      rit->second.pop_back();
      ctx->capturing->held.erase(*ptr);  // owned by a tensor again; re-held if freed later
      *capacity = cls;
      ctx->bytes_in_use += (int64_t)cls;
      return TFJS_CUDA_OK;
    }
  }
  auto it = ctx->free_lists.find(cls);
  if (it != ctx->free_lists.end() && !it->second.empty()) {
    *ptr = it->second.back();
    it->second.pop_back();
    ctx->num_cached--;
  } else {
    cudaError_t e = cudaMalloc(ptr, cls);
    if (e == cudaErrorMemoryAllocation) {
      cudaGetLastError();
      cudaStreamSynchronize(ctx->stream);
      release_cached(ctx);
      e = cudaMalloc(ptr, cls);
    }
    if (e != cudaSuccess) {
      cudaGetLastError();
      *ptr = nullptr;
      return set_error(ctx, e == cudaErrorMemoryAllocation ? TFJS_CUDA_ERR_OOM : TFJS_CUDA_ERR_CUDA,
                       "cudaMalloc(%zu) failed: %s", cls, cudaGetErrorString(e));
    }
    ctx->num_device_allocs++;
    ctx->bytes_reserved += (int64_t)cls;
  }
  *capacity = cls;
  ctx->bytes_in_use += (int64_t)cls;
  if (canary) {
    canary_fill_kernel<<<1, CANARY_BYTES / 4, 0, ctx->stream>>>((uint32_t*)((char*)*ptr + guard_at));
    ctx->canary_offset[*ptr] = guard_at;
  }
  return TFJS_CUDA_OK;
}

void ctx_free(tfjs_cuda_ctx* ctx, void* ptr, size_t capacity) {
  if (!ptr) return;
  ctx->bytes_in_use -= (int64_t)capacity;
  auto guard = ctx->canary_offset.find(ptr);
  if (guard != ctx->canary_offset.end()) {
    // stream-ordered after every kernel that wrote the buffer; a mismatch lands in the status
    // word and surfaces at the next synchronisation
    if (!ctx->capturing)
      canary_check_kernel<<<1, CANARY_BYTES / 4, 0, ctx->stream>>>(
          (const uint32_t*)((const char*)ptr + guard->second), ctx->d_status);
    ctx->canary_offset.erase(guard);
  }
  if (ctx->capturing) {
    // A captured graph keeps writing to this buffer on every replay.
    ctx->capturing->held[ptr] = capacity;
    ctx->capturing->reusable[capacity].push_back(ptr);
    return;
  }
  ctx->free_lists[capacity].push_back(ptr);
  ctx->num_cached++;
}

// ---- context -----------------------------------------------------------------------------
extern "C" int tfjs_cuda_ctx_create(int device, tfjs_cuda_ctx** out) {
  if (!out) return TFJS_CUDA_ERR_INVALID_ARG;
  *out = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0) {
    cudaGetLastError();
    g_create_error = "no usable CUDA device";
    return TFJS_CUDA_ERR_CUDA;
  }
  if (device < 0 || device >= count) {
    g_create_error = "device ordinal out of range";
    return TFJS_CUDA_ERR_INVALID_ARG;
  }
  if (cudaSetDevice(device) != cudaSuccess) {
    cudaGetLastError();
    g_create_error = "cudaSetDevice failed";
    return TFJS_CUDA_ERR_CUDA;
  }
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) {
    cudaGetLastError();
    g_create_error = "cudaGetDeviceProperties failed";
    return TFJS_CUDA_ERR_CUDA;
  }
  if (prop.major != 10) {
    g_create_error = "this library is built for sm_100a (B200) only";
    return TFJS_CUDA_ERR_UNSUPPORTED;
  }
  tfjs_cuda_ctx* ctx = new tfjs_cuda_ctx();
  ctx->device = device;
  ctx->sm_count = prop.multiProcessorCount;
  bool ok = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) == cudaSuccess &&
            cudaEventCreate(&ctx->time_start) == cudaSuccess &&
            cudaEventCreate(&ctx->time_stop) == cudaSuccess &&
            cudaMalloc(&ctx->d_status, sizeof(int)) == cudaSuccess &&
            cudaMallocHost(&ctx->h_status, sizeof(int)) == cudaSuccess &&
            cudaMemset(ctx->d_status, 0, sizeof(int)) == cudaSuccess;
  if (!ok) {
    g_create_error = std::string("context setup failed: ") + cudaGetErrorString(cudaGetLastError());
    tfjs_cuda_ctx_destroy(ctx);
    return TFJS_CUDA_ERR_CUDA;
  }
  *ctx->h_status = 0;
  *out = ctx;
  return TFJS_CUDA_OK;
}

static void free_entry_buffers(tfjs_cuda_ctx* ctx, TensorEntry& t) {
  ctx_free(ctx, t.ptr, t.capacity);
  t.ptr = nullptr;
  if (t.packed.hi) ctx_free(ctx, t.packed.hi, t.packed.capacity);
  if (t.packed.lo) ctx_free(ctx, t.packed.lo, t.packed.capacity);
  t.packed = PackedWeights();
  if (t.deq) ctx_free(ctx, t.deq, t.deq_capacity);
  t.deq = nullptr;
  if (t.packed_q) ctx_free(ctx, t.packed_q, t.packed_q_capacity);
  t.packed_q = nullptr;
  if (t.w16) ctx_free(ctx, t.w16, t.w16_capacity);
  t.w16 = nullptr;
  if (t.copy_event) {
    // the buffer goes back to the pool: later users are ordered on the compute stream only
    if (t.copy_pending) cudaStreamWaitEvent(ctx->stream, t.copy_event, 0);
    cudaEventDestroy(t.copy_event);
    t.copy_event = nullptr;
    t.copy_pending = false;
  }
}

extern "C" int tfjs_cuda_device_count(int* out) {
  if (!out) return TFJS_CUDA_ERR_INVALID_ARG;
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    n = 0;
  }
  *out = n;
  return TFJS_CUDA_OK;
}

extern "C" int tfjs_cuda_ctx_destroy(tfjs_cuda_ctx* ctx) {
  if (!ctx) return TFJS_CUDA_OK;
  cudaSetDevice(ctx->device);
  if (ctx->stream) cudaStreamSynchronize(ctx->stream);
  ctx->capturing = nullptr;
  for (auto& kv : ctx->tensors) free_entry_buffers(ctx, kv.second);
  ctx->tensors.clear();
  release_cached(ctx);
  if (ctx->d_status) cudaFree(ctx->d_status);
  if (ctx->h_status) cudaFreeHost(ctx->h_status);
  for (cudaEvent_t ev : ctx->profile_events) cudaEventDestroy(ev);
  if (ctx->compute_mark) cudaEventDestroy(ctx->compute_mark);
  if (ctx->copy_stream) {
    cudaStreamSynchronize(ctx->copy_stream);
    cudaStreamDestroy(ctx->copy_stream);
  }
  if (ctx->time_start) cudaEventDestroy(ctx->time_start);
  if (ctx->time_stop) cudaEventDestroy(ctx->time_stop);
  if (ctx->stream) cudaStreamDestroy(ctx->stream);
  cudaGetLastError();
  delete ctx;
  return TFJS_CUDA_OK;
}

extern "C" const char* tfjs_cuda_last_error(const tfjs_cuda_ctx* ctx) {
  return ctx ? ctx->last_error.c_str() : g_create_error.c_str();
}

extern "C" int tfjs_cuda_ctx_set_option(tfjs_cuda_ctx* ctx, const char* key, double value) {
  if (!ctx || !key) return TFJS_CUDA_ERR_INVALID_ARG;
  if (!strcmp(key, "math_mode")) {
    TFJS_REQUIRE(ctx, value == TFJS_MATH_TF32X3 || value == TFJS_MATH_TF32,
                 "math_mode must be 0 (3xTF32) or 1 (TF32)");
    ctx->math_mode = (int)value;
  } else if (!strcmp(key, "use_tensor_cores")) {
    ctx->use_tensor_cores = value != 0;
  } else if (!strcmp(key, "debug_sync")) {
    ctx->debug_sync = value != 0;
  } else if (!strcmp(key, "dequant_in_gemm")) {
    ctx->dequant_in_gemm = value != 0;
  } else if (!strcmp(key, "pdl")) {
    ctx->use_pdl = value != 0;
  } else if (!strcmp(key, "debug_canary")) {
    ctx->debug_canary = value != 0;
  } else if (!strcmp(key, "test_withhold_last_load")) {
    ctx->test_withhold_last_load = value != 0;
  } else if (!strcmp(key, "wait_limit_us")) {
    // bounded device-side waits give up after this long; per device, shared by its contexts
    TFJS_REQUIRE(ctx, value >= 100 && value <= 60e6, "wait_limit_us must lie between 100 and 60 000 000");
    cudaSetDevice(ctx->device);
    int khz = 0;
    TFJS_CHECK_CUDA(ctx, cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, ctx->device));
    const long long cycles = (long long)(value * 1e-3 * (double)khz);
    if (set_wait_limit_gemm(cycles) || set_wait_limit_sepconv(cycles) || set_wait_limit_depthwise_image(cycles) ||
        set_wait_limit_gemm_pair(cycles)) {
      cudaGetLastError();
      return set_error(ctx, TFJS_CUDA_ERR_CUDA, "could not set the wait limit");
    }
  } else if (!strcmp(key, "gemm_block_n")) {
    TFJS_REQUIRE(ctx, value == 0 || value == 32 || value == 64 || value == 128 || value == 256,
                 "gemm_block_n must be 0 (cost model), 32, 64, 128 or 256");
    ctx->gemm_block_n = (int)value;
  } else if (!strcmp(key, "gemm_pair")) {
    TFJS_REQUIRE(ctx, value == 0 || value == 1 || value == 2, "gemm_pair must be 0, 1 or 2");
    ctx->gemm_pair = (int)value;
  } else if (!strcmp(key, "fuse_separable")) {
    TFJS_REQUIRE(ctx, value == 0 || value == 1 || value == 2, "fuse_separable must be 0, 1 or 2");
    ctx->fuse_separable = (int)value;
  } else {
    return set_error(ctx, TFJS_CUDA_ERR_INVALID_ARG, "unknown option '%s'", key);
  }
  return TFJS_CUDA_OK;
}

// Copies the device status word back and turns a non-zero value into an error.
static int check_device_status(tfjs_cuda_ctx* ctx) {
  if (*ctx->h_status != 0) {
    int code = *ctx->h_status;
    *ctx->h_status = 0;
    cudaMemsetAsync(ctx->d_status, 0, sizeof(int), ctx->stream);
    if (code == STATUS_CANARY)
      return set_error(ctx, TFJS_CUDA_ERR_CUDA,
                       "a kernel wrote past the end of a buffer (guard pattern overwritten; device status %d)", code);
    if (code == STATUS_SMEM_LAYOUT)
      return set_error(ctx, TFJS_CUDA_ERR_CUDA,
                       "a kernel found its shared-memory window misaligned and did not run (device status %d)", code);
    return set_error(ctx, TFJS_CUDA_ERR_TIMEOUT,
                     "a kernel gave up on a bounded wait (device status %d)", code);
  }
  return TFJS_CUDA_OK;
}

static int sync_stream(tfjs_cuda_ctx* ctx, int timeout_ms) {
  TFJS_REQUIRE(ctx, !ctx->capturing, "cannot synchronise while capturing a graph");
  TFJS_CHECK_CUDA(ctx, cudaMemcpyAsync(ctx->h_status, ctx->d_status, sizeof(int),
                                       cudaMemcpyDeviceToHost, ctx->stream));
  if (timeout_ms < 0) {
    TFJS_CHECK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  } else {
    auto t0 = std::chrono::steady_clock::now();
    for (;;) {
      cudaError_t e = cudaStreamQuery(ctx->stream);
      if (e == cudaSuccess) break;
      if (e != cudaErrorNotReady) {
        cudaGetLastError();
        return set_error(ctx, TFJS_CUDA_ERR_CUDA, "stream error: %s", cudaGetErrorString(e));
      }
      auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(
                    std::chrono::steady_clock::now() - t0).count();
      if (ms > timeout_ms)
        return set_error(ctx, TFJS_CUDA_ERR_TIMEOUT, "sync timed out after %d ms", timeout_ms);
      std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
  }
  return check_device_status(ctx);
}

extern "C" int tfjs_cuda_ctx_sync(tfjs_cuda_ctx* ctx, int timeout_ms) {
  if (!ctx) return TFJS_CUDA_ERR_INVALID_ARG;
  cudaSetDevice(ctx->device);
  return sync_stream(ctx, timeout_ms);
}

extern "C" int tfjs_cuda_ctx_memory(tfjs_cuda_ctx* ctx, tfjs_cuda_mem_stats* out) {
  if (!ctx || !out) return TFJS_CUDA_ERR_INVALID_ARG;
  out->num_tensors = (int64_t)ctx->tensors.size();
  out->bytes_in_use = ctx->bytes_in_use;
  out->bytes_reserved = ctx->bytes_reserved;
  out->num_buffers_cached = ctx->num_cached;
  out->num_device_allocs = ctx->num_device_allocs;
  return TFJS_CUDA_OK;
}

extern "C" int tfjs_cuda_ctx_time_begin(tfjs_cuda_ctx* ctx) {
  if (!ctx) return TFJS_CUDA_ERR_INVALID_ARG;
  cudaSetDevice(ctx->device);
  ctx->time_start_launches = ctx->launch_count;
  TFJS_CHECK_CUDA(ctx, cudaEventRecord(ctx->time_start, ctx->stream));
  return TFJS_CUDA_OK;
}

extern "C" int tfjs_cuda_ctx_time_end(tfjs_cuda_ctx* ctx, float* ms, int64_t* launches) {
  if (!ctx) return TFJS_CUDA_ERR_INVALID_ARG;
  cudaSetDevice(ctx->device);
  TFJS_CHECK_CUDA(ctx, cudaEventRecord(ctx->time_stop, ctx->stream));
  TFJS_CHECK_CUDA(ctx, cudaEventSynchronize(ctx->time_stop));
  float t = 0.f;
  TFJS_CHECK_CUDA(ctx, cudaEventElapsedTime(&t, ctx->time_start, ctx->time_stop));
  if (ms) *ms = t;
  if (launches) *launches = ctx->launch_count - ctx->time_start_launches;
  return TFJS_CUDA_OK;
}

extern "C" int64_t tfjs_cuda_ctx_launch_count(const tfjs_cuda_ctx* ctx) {
  return ctx ? ctx->launch_count : 0;
}

extern "C" void* tfjs_cuda_ctx_stream(tfjs_cuda_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }

// ---- tensors -----------------------------------------------------------------------------
TensorEntry* find_tensor(tfjs_cuda_ctx* ctx, tfjs_tensor_id id) {
  auto it = ctx->tensors.find(id);
  return it == ctx->tensors.end() ? nullptr : &it->second;
}

static size_t dtype_size(int dtype) { return dtype == TFJS_BOOL ? 1 : (dtype == TFJS_F16 ? 2 : 4); }

// Records whether the values the host just handed over are all finite (small float tensors only:
// filters and biases; an image batch is not scanned).
static void note_host_values(TensorEntry* t, const void* host) {
  if (t->quant.quantized) {  // raw bytes: every decoded value q * scale + min stays as finite as before
    if (t->finite_version + 1 == t->version) t->finite_version = t->version;
    return;
  }
  t->finite_version = ~0ull;
  if (t->dtype != TFJS_F32 || t->size > 65536 || (t->size > 0 && !host)) return;
  const uint32_t* bits = (const uint32_t*)host;
  for (int64_t i = 0; i < t->size; i++)
    if ((bits[i] & 0x7f800000u) == 0x7f800000u) return;  // inf or NaN
  t->finite_version = t->version;
}

static int register_impl(tfjs_cuda_ctx* ctx, tfjs_tensor_id* out_id, int rank, const int64_t* shape,
                         int dtype, size_t elem_size) {
  TFJS_REQUIRE(ctx, out_id != nullptr, "out_id is null");
  TFJS_REQUIRE(ctx, rank >= 0 && rank <= 8, "rank %d out of range", rank);
  TFJS_REQUIRE(ctx, dtype == TFJS_F32 || dtype == TFJS_I32 || dtype == TFJS_BOOL || dtype == TFJS_F16,
               "unsupported dtype %d", dtype);
  TensorEntry t;
  t.dtype = dtype;
  t.rank = rank;
  t.size = 1;
  for (int i = 0; i < rank; i++) {
    TFJS_REQUIRE(ctx, shape[i] >= 0, "negative dimension");
    t.shape[i] = shape[i];
    t.size *= shape[i];
  }
  t.nbytes = (size_t)t.size * elem_size;
  cudaSetDevice(ctx->device);
  int rc = ctx_alloc(ctx, t.nbytes, &t.ptr, &t.capacity);
  if (rc) return rc;
  tfjs_tensor_id id = ctx->next_id++;
  ctx->tensors.emplace(id, t);
  *out_id = id;
  return TFJS_CUDA_OK;
}

extern "C" int tfjs_cuda_tensor_register(tfjs_cuda_ctx* ctx, tfjs_tensor_id* out_id, int rank,
                                         const int64_t* shape, int dtype) {
  if (!ctx) return TFJS_CUDA_ERR_INVALID_ARG;
  return register_impl(ctx, out_id, rank, shape, dtype, dtype_size(dtype));
}

extern "C" int tfjs_cuda_tensor_register_quantized(tfjs_cuda_ctx* ctx, tfjs_tensor_id* out_id,
                                                   int rank, const int64_t* shape,
                                                   const uint8_t* q, double scale, double min) {
  if (!ctx) return TFJS_CUDA_ERR_INVALID_ARG;
  TFJS_REQUIRE(ctx, q != nullptr, "quantised bytes are null");
  int rc = register_impl(ctx, out_id, rank, shape, TFJS_F32, 1);
  if (rc) return rc;
  TensorEntry* t = find_tensor(ctx, *out_id);
  t->quant.quantized = true;
  t->quant.scale = scale;
  t->quant.min = min;
  if (t->nbytes)
    TFJS_CHECK_CUDA(ctx, cudaMemcpyAsync(t->ptr, q, t->nbytes, cudaMemcpyHostToDevice, ctx->stream));
  t->version++;
  // q * scale + min over the 256 byte values is finite when both ends are
  const double w0 = min, w255 = 255.0 * scale + min;
  if (w0 == w0 && w255 == w255 && w0 - w0 == 0.0 && w255 - w255 == 0.0 && (float)w0 - (float)w0 == 0.f &&
      (float)w255 - (float)w255 == 0.f)
    t->finite_version = t->version;
  return TFJS_CUDA_OK;
}

extern "C" int tfjs_cuda_tensor_write(tfjs_cuda_ctx* ctx, tfjs_tensor_id id, const void* host,
                                      size_t nbytes) {
  if (!ctx) return TFJS_CUDA_ERR_INVALID_ARG;
  TensorEntry* t = find_tensor(ctx, id);
  if (!t) return set_error(ctx, TFJS_CUDA_ERR_NOT_FOUND, "write: unknown tensor id %lld", (long long)id);
  // backend_cpu.ts:125-127: writing null throws
  TFJS_REQUIRE(ctx, host != nullptr || nbytes == 0, "MathBackendCUDA.write(): values cannot be null");
  // a quantised tensor is refilled with raw bytes (one per element), e.g. the next batch of pixels
  TFJS_REQUIRE(ctx, !t->quant.quantized || nbytes == t->nbytes,
               "a quantised tensor takes its %zu raw bytes, not float values", t->nbytes);
  cudaSetDevice(ctx->device);
  if (t->copy_pending) {  // an earlier asynchronous upload must not land after this one
    TFJS_CHECK_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, t->copy_event, 0));
    t->copy_pending = false;
  }
  if (t->dtype == TFJS_F16) {
    // half-precision storage: the host hands over float32 values, converted on the device
    TFJS_REQUIRE(ctx, nbytes == (size_t)t->size * 4, "write: %zu bytes given, tensor holds %zu float32 values",
                 nbytes, (size_t)t->size);
    if (nbytes) {
      void* tmp;
      size_t cap;
      int rc = ctx_alloc(ctx, nbytes, &tmp, &cap);
      if (rc) return rc;
      cudaError_t e = cudaMemcpyAsync(tmp, host, nbytes, cudaMemcpyHostToDevice, ctx->stream);
      rc = e == cudaSuccess ? launch_convert(ctx, tmp, TFJS_F32, t->ptr, TFJS_F16, t->size)
                            : set_error(ctx, TFJS_CUDA_ERR_CUDA, "write failed: %s", cudaGetErrorString(e));
      ctx_free(ctx, tmp, cap);
      if (rc) return rc;
    }
    t->version++;
    return TFJS_CUDA_OK;
  }
  TFJS_REQUIRE(ctx, nbytes == t->nbytes, "write: %zu bytes given, tensor holds %zu", nbytes, t->nbytes);
  if (nbytes)
    TFJS_CHECK_CUDA(ctx, cudaMemcpyAsync(t->ptr, host, nbytes, cudaMemcpyHostToDevice, ctx->stream));
  t->version++;
  note_host_values(t, host);
  return TFJS_CUDA_OK;
}

// Makes work enqueued on the context's stream from now on wait for an asynchronous upload of
// this tensor that may still be in flight on the copy stream.
static int wait_for_upload(tfjs_cuda_ctx* ctx, TensorEntry* t) {
  if (t->copy_pending) {
    TFJS_CHECK_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, t->copy_event, 0));
    t->copy_pending = false;
  }
  return TFJS_CUDA_OK;
}

extern "C" int tfjs_cuda_tensor_write_async(tfjs_cuda_ctx* ctx, tfjs_tensor_id id, const void* host,
                                            size_t nbytes) {
  if (!ctx) return TFJS_CUDA_ERR_INVALID_ARG;
  TensorEntry* t = find_tensor(ctx, id);
  if (!t) return set_error(ctx, TFJS_CUDA_ERR_NOT_FOUND, "write: unknown tensor id %lld", (long long)id);
  TFJS_REQUIRE(ctx, host != nullptr || nbytes == 0, "MathBackendCUDA.write(): values cannot be null");
  TFJS_REQUIRE(ctx, !t->quant.quantized || nbytes == t->nbytes,
               "a quantised tensor takes its %zu raw bytes, not float values", t->nbytes);
  TFJS_REQUIRE(ctx, t->dtype != TFJS_F16, "asynchronous writes need float32 storage (use tensor_write)");
  TFJS_REQUIRE(ctx, nbytes == t->nbytes, "write: %zu bytes given, tensor holds %zu", nbytes, t->nbytes);
  TFJS_REQUIRE(ctx, !ctx->capturing, "asynchronous writes cannot be captured into a graph");
  cudaSetDevice(ctx->device);
  if (!ctx->copy_stream) {
    TFJS_CHECK_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->copy_stream, cudaStreamNonBlocking));
    TFJS_CHECK_CUDA(ctx, cudaEventCreateWithFlags(&ctx->compute_mark, cudaEventDisableTiming));
  }
  if (!t->copy_event)
    TFJS_CHECK_CUDA(ctx, cudaEventCreateWithFlags(&t->copy_event, cudaEventDisableTiming));
  t->version++;
  note_host_values(t, host);
  if (!nbytes) return TFJS_CUDA_OK;
  // write-after-read: kernels already enqueued may still read the old contents
  TFJS_CHECK_CUDA(ctx, cudaEventRecord(ctx->compute_mark, ctx->stream));
  TFJS_CHECK_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_stream, ctx->compute_mark, 0));
  TFJS_CHECK_CUDA(ctx, cudaMemcpyAsync(t->ptr, host, nbytes, cudaMemcpyHostToDevice, ctx->copy_stream));
  TFJS_CHECK_CUDA(ctx, cudaEventRecord(t->copy_event, ctx->copy_stream));
  t->copy_pending = true;
  return TFJS_CUDA_OK;
}

extern "C" int tfjs_cuda_tensor_wait(tfjs_cuda_ctx* ctx, tfjs_tensor_id id) {
  if (!ctx) return TFJS_CUDA_ERR_INVALID_ARG;
  TensorEntry* t = find_tensor(ctx, id);
  if (!t) return set_error(ctx, TFJS_CUDA_ERR_NOT_FOUND, "wait: unknown tensor id %lld", (long long)id);
  cudaSetDevice(ctx->device);
  return wait_for_upload(ctx, t);
}

static int enqueue_read(tfjs_cuda_ctx* ctx, TensorEntry* t, void* host, size_t nbytes) {
  int wrc = wait_for_upload(ctx, t);
  if (wrc) return wrc;
  if (t->quant.quantized || t->dtype == TFJS_F16) {
    // stored narrower than float32: the host gets float32 values, expanded on the device
    TFJS_REQUIRE(ctx, nbytes == (size_t)t->size * 4, "read: %zu bytes asked, tensor holds %zu",
                 nbytes, (size_t)t->size * 4);
    if (!nbytes) return TFJS_CUDA_OK;
    void* tmp;
    size_t cap;
    int rc = ctx_alloc(ctx, nbytes, &tmp, &cap);
    if (rc) return rc;
    rc = t->quant.quantized
             ? launch_dequant(ctx, (const uint8_t*)t->ptr, (float*)tmp, t->size, t->quant.scale, t->quant.min)
             : launch_convert(ctx, t->ptr, TFJS_F16, tmp, TFJS_F32, t->size);
    if (!rc) {
      cudaError_t e = cudaMemcpyAsync(host, tmp, nbytes, cudaMemcpyDeviceToHost, ctx->stream);
      if (e != cudaSuccess) rc = set_error(ctx, TFJS_CUDA_ERR_CUDA, "read failed: %s", cudaGetErrorString(e));
    }
    ctx_free(ctx, tmp, cap);
    return rc;
  }
  TFJS_REQUIRE(ctx, nbytes == t->nbytes, "read: %zu bytes asked, tensor holds %zu", nbytes, t->nbytes);
  if (nbytes)
    TFJS_CHECK_CUDA(ctx, cudaMemcpyAsync(host, t->ptr, nbytes, cudaMemcpyDeviceToHost, ctx->stream));
  return TFJS_CUDA_OK;
}

extern "C" int tfjs_cuda_tensor_read(tfjs_cuda_ctx* ctx, tfjs_tensor_id id, void* host, size_t nbytes) {
  if (!ctx) return TFJS_CUDA_ERR_INVALID_ARG;
  TensorEntry* t = find_tensor(ctx, id);
  if (!t) return set_error(ctx, TFJS_CUDA_ERR_NOT_FOUND, "read: unknown tensor id %lld", (long long)id);
  TFJS_REQUIRE(ctx, host != nullptr || nbytes == 0, "read: host buffer is null");
  TFJS_REQUIRE(ctx, !ctx->capturing, "cannot read while capturing a graph");
  cudaSetDevice(ctx->device);
  int rc = enqueue_read(ctx, t, host, nbytes);
  if (rc) return rc;
  return sync_stream(ctx, -1);
}

extern "C" int tfjs_cuda_tensor_read_async(tfjs_cuda_ctx* ctx, tfjs_tensor_id id, void* host,
                                           size_t nbytes, tfjs_cuda_event** out_event) {
  if (!ctx || !out_event) return TFJS_CUDA_ERR_INVALID_ARG;
  TensorEntry* t = find_tensor(ctx, id);
  if (!t) return set_error(ctx, TFJS_CUDA_ERR_NOT_FOUND, "read: unknown tensor id %lld", (long long)id);
  TFJS_REQUIRE(ctx, host != nullptr || nbytes == 0, "read: host buffer is null");
  TFJS_REQUIRE(ctx, !ctx->capturing, "cannot read while capturing a graph");
  cudaSetDevice(ctx->device);
  int rc = enqueue_read(ctx, t, host, nbytes);
  if (rc) return rc;
  tfjs_cuda_event* ev = new tfjs_cuda_event();
  ev->device = ctx->device;
  cudaError_t e = cudaEventCreateWithFlags(&ev->ev, cudaEventDisableTiming);
  if (e == cudaSuccess) e = cudaEventRecord(ev->ev, ctx->stream);
  if (e != cudaSuccess) {
    if (ev->ev) cudaEventDestroy(ev->ev);
    delete ev;
    return set_error(ctx, TFJS_CUDA_ERR_CUDA, "event setup failed: %s", cudaGetErrorString(e));
  }
  *out_event = ev;
  return TFJS_CUDA_OK;
}

extern "C" int tfjs_cuda_event_query(tfjs_cuda_event* ev) {
  if (!ev) return TFJS_CUDA_ERR_INVALID_ARG;
  cudaError_t e = cudaEventQuery(ev->ev);
  if (e == cudaSuccess) return 1;
  if (e == cudaErrorNotReady) return 0;
  cudaGetLastError();
  return TFJS_CUDA_ERR_CUDA;
}

extern "C" int tfjs_cuda_event_wait(tfjs_cuda_event* ev, int timeout_ms) {
  if (!ev) return TFJS_CUDA_ERR_INVALID_ARG;
  if (timeout_ms < 0) return cudaEventSynchronize(ev->ev) == cudaSuccess ? TFJS_CUDA_OK : TFJS_CUDA_ERR_CUDA;
  auto t0 = std::chrono::steady_clock::now();
  for (;;) {
    int q = tfjs_cuda_event_query(ev);
    if (q == 1) return TFJS_CUDA_OK;
    if (q < 0) return q;
    auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(
                  std::chrono::steady_clock::now() - t0).count();
    if (ms > timeout_ms) return TFJS_CUDA_ERR_TIMEOUT;
    std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
}

extern "C" int tfjs_cuda_event_destroy(tfjs_cuda_event* ev) {
  if (!ev) return TFJS_CUDA_OK;
  if (ev->ev) cudaEventDestroy(ev->ev);
  delete ev;
  return TFJS_CUDA_OK;
}

extern "C" int tfjs_cuda_tensor_dispose(tfjs_cuda_ctx* ctx, tfjs_tensor_id id) {
  if (!ctx) return TFJS_CUDA_ERR_INVALID_ARG;
  auto it = ctx->tensors.find(id);
  if (it == ctx->tensors.end()) return TFJS_CUDA_OK;  // idempotent
  free_entry_buffers(ctx, it->second);
  ctx->tensors.erase(it);
  return TFJS_CUDA_OK;
}

extern "C" int tfjs_cuda_tensor_device_ptr(tfjs_cuda_ctx* ctx, tfjs_tensor_id id, void** ptr,
                                           size_t* nbytes) {
  if (!ctx) return TFJS_CUDA_ERR_INVALID_ARG;
  TensorEntry* t = find_tensor(ctx, id);
  if (!t) return set_error(ctx, TFJS_CUDA_ERR_NOT_FOUND, "unknown tensor id %lld", (long long)id);
  if (ptr) *ptr = t->ptr;
  if (nbytes) *nbytes = t->nbytes;
  return TFJS_CUDA_OK;
}

extern "C" int tfjs_cuda_host_alloc(void** ptr, size_t nbytes) {
  if (!ptr) return TFJS_CUDA_ERR_INVALID_ARG;
  cudaError_t e = cudaMallocHost(ptr, nbytes ? nbytes : 1);
  if (e != cudaSuccess) {
    cudaGetLastError();
    *ptr = nullptr;
    return TFJS_CUDA_ERR_OOM;
  }
  return TFJS_CUDA_OK;
}

extern "C" int tfjs_cuda_host_free(void* ptr) {
  if (ptr) cudaFreeHost(ptr);
  return TFJS_CUDA_OK;
}

int get_f32(tfjs_cuda_ctx* ctx, tfjs_tensor_id id, int64_t min_elems, const char* what,
            TensorEntry** out) {
  TensorEntry* t = find_tensor(ctx, id);
  if (!t) return set_error(ctx, TFJS_CUDA_ERR_NOT_FOUND, "%s: unknown tensor id %lld", what, (long long)id);
  TFJS_REQUIRE(ctx, t->dtype == TFJS_F32, "%s must be stored as float32 (cast it first)", what);
  TFJS_REQUIRE(ctx, t->size >= min_elems, "%s holds %lld elements, %lld needed", what,
               (long long)t->size, (long long)min_elems);
  *out = t;
  return wait_for_upload(ctx, t);  // kernels that take this operand run after its upload
}

// Same for an activation operand, which may be stored as float32 or as half precision.
int get_activation(tfjs_cuda_ctx* ctx, tfjs_tensor_id id, int64_t min_elems, const char* what,
                   TensorEntry** out) {
  TensorEntry* t = find_tensor(ctx, id);
  if (!t) return set_error(ctx, TFJS_CUDA_ERR_NOT_FOUND, "%s: unknown tensor id %lld", what, (long long)id);
  TFJS_REQUIRE(ctx, t->dtype == TFJS_F32 || t->dtype == TFJS_F16,
               "%s must be stored as float32 or float16 (cast it first)", what);
  TFJS_REQUIRE(ctx, !t->quant.quantized, "%s cannot be a quantised tensor", what);
  TFJS_REQUIRE(ctx, t->size >= min_elems, "%s holds %lld elements, %lld needed", what,
               (long long)t->size, (long long)min_elems);
  *out = t;
  return wait_for_upload(ctx, t);
}

int resolve_epilogue(tfjs_cuda_ctx* ctx, const tfjs_epilogue* epi, int64_t channels,
                     EpilogueArgs* out) {
  *out = EpilogueArgs();
  if (!epi) return TFJS_CUDA_OK;
  if (epi->bias) {
    TFJS_REQUIRE(ctx, epi->bias_len == 1 || epi->bias_len == channels,
                 "fused bias must be a scalar or one value per output channel");
    TensorEntry* b;
    int rc = get_f32(ctx, epi->bias, epi->bias_len, "bias", &b);
    if (rc) return rc;
    TFJS_REQUIRE(ctx, !b->quant.quantized, "bias cannot be quantised");
    out->bias = (const float*)b->ptr;
    out->bias_scalar = epi->bias_len == 1 && channels != 1;
  }
  out->activation = epi->activation;
  TFJS_REQUIRE(ctx, epi->activation >= TFJS_ACT_LINEAR && epi->activation <= TFJS_ACT_CLIP,
               "unknown activation %d", epi->activation);
  if (epi->activation == TFJS_ACT_PRELU) {
    TFJS_REQUIRE(ctx, epi->prelu != 0, "prelu activation needs preluActivationWeights");
    TFJS_REQUIRE(ctx, epi->prelu_len == 1 || epi->prelu_len == channels,
                 "fused prelu weights must be a scalar or one value per output channel");
    TensorEntry* p;
    int rc = get_f32(ctx, epi->prelu, epi->prelu_len, "preluActivationWeights", &p);
    if (rc) return rc;
    out->prelu = (const float*)p->ptr;
    out->prelu_scalar = epi->prelu_len == 1 && channels != 1;
  }
  out->clip_lo = epi->clip_lo;
  out->clip_hi = epi->clip_hi;
  return TFJS_CUDA_OK;
}

// ---- graph capture -----------------------------------------------------------------------
extern "C" int tfjs_cuda_graph_begin(tfjs_cuda_ctx* ctx) {
  if (!ctx) return TFJS_CUDA_ERR_INVALID_ARG;
  TFJS_REQUIRE(ctx, !ctx->capturing, "a graph capture is already in progress");
  cudaSetDevice(ctx->device);
  TFJS_CHECK_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeRelaxed));
  ctx->capturing = new tfjs_cuda_graph();
  ctx->capture_start_launches = ctx->launch_count;
  return TFJS_CUDA_OK;
}

extern "C" int tfjs_cuda_graph_end(tfjs_cuda_ctx* ctx, tfjs_cuda_graph** out) {
  if (!ctx || !out) return TFJS_CUDA_ERR_INVALID_ARG;
  TFJS_REQUIRE(ctx, ctx->capturing, "no graph capture in progress");
  tfjs_cuda_graph* g = ctx->capturing;
  ctx->capturing = nullptr;
  g->launches_per_replay = ctx->launch_count - ctx->capture_start_launches;
  g->reusable.clear();
  cudaError_t e = cudaStreamEndCapture(ctx->stream, &g->graph);
  if (e == cudaSuccess) e = cudaGraphInstantiate(&g->exec, g->graph, 0);
  if (e != cudaSuccess) {
    cudaGetLastError();
    tfjs_cuda_graph_destroy(ctx, g);
    return set_error(ctx, TFJS_CUDA_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
  }
  *out = g;
  return TFJS_CUDA_OK;
}

extern "C" int tfjs_cuda_graph_launch(tfjs_cuda_ctx* ctx, tfjs_cuda_graph* g) {
  if (!ctx || !g || !g->exec) return TFJS_CUDA_ERR_INVALID_ARG;
  cudaSetDevice(ctx->device);
  TFJS_CHECK_CUDA(ctx, cudaGraphLaunch(g->exec, ctx->stream));
  ctx->launch_count += g->launches_per_replay;
  return TFJS_CUDA_OK;
}

extern "C" int tfjs_cuda_graph_destroy(tfjs_cuda_ctx* ctx, tfjs_cuda_graph* g) {
  if (!g) return TFJS_CUDA_OK;
  if (g->exec) cudaGraphExecDestroy(g->exec);
  if (g->graph) cudaGraphDestroy(g->graph);
  if (ctx) {
    cudaStreamSynchronize(ctx->stream);
    for (auto& p : g->held) {
      ctx->bytes_in_use += (int64_t)p.second;  // ctx_free subtracts it again
      ctx_free(ctx, p.first, p.second);
    }
  }
  delete g;
  return TFJS_CUDA_OK;
}
