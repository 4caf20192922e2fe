// Internal definitions shared by the translation units of libtfjs_cuda.so.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/tfjs_cuda.h"

struct QuantInfo {
  bool quantized = false;
  double scale = 0.0, min = 0.0;
};

// Operand of a contraction repacked for the tensor-core kernel: K-major [N, Kp] float32,
// tf32-rounded "hi" plane and (for 3xTF32) the "lo" residual plane.  Cached per weight
// tensor and invalidated when the tensor is written.
struct PackedWeights {
  float* hi = nullptr;
  float* lo = nullptr;
  size_t capacity = 0;  // allocator size class of each plane
  int64_t n = 0, k = 0, kp = 0;
  uint64_t version = 0;
  bool transposed_source = false;
  int row_pad = 0;  // > 0: filter rows padded to this many floats (Cin == 3 conv gather)
};

struct TensorEntry {
  void* ptr = nullptr;   // device storage (nullptr for zero-sized tensors)
  size_t nbytes = 0;     // logical byte size (f32/i32: 4 per element, bool/quantised: 1)
  size_t capacity = 0;   // size class of the buffer behind ptr
  int dtype = TFJS_F32;
  int rank = 0;
  int64_t shape[8] = {0};
  int64_t size = 0;      // element count
  uint64_t version = 0;  // bumped on every write / kernel output
  QuantInfo quant;
  PackedWeights packed;
  // float32 copy of a quantised tensor for the kernels that read plain floats
  float* deq = nullptr;
  size_t deq_capacity = 0;
  uint64_t deq_version = 0;
  // K-major uint8 copy [N, kq] of a quantised contraction operand: the tensor-core GEMM loads
  // these bytes with TMA and dequantises them in shared memory inside its main loop
  uint8_t* packed_q = nullptr;
  size_t packed_q_capacity = 0;
  int64_t packed_q_n = 0, packed_q_k = 0, packed_q_kq = 0;
  uint64_t packed_q_version = 0;
  bool packed_q_transposed = false;
  // asynchronous upload in flight on the copy stream (tensor_write_async)
  cudaEvent_t copy_event = nullptr;
  bool copy_pending = false;
};

struct tfjs_cuda_graph {
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  // Buffers disposed while capturing stay owned by the graph: replays write to them.
  std::map<void*, size_t> held;
  // held buffers that are free again inside the capture: later captured kernels may reuse them
  std::map<size_t, std::vector<void*>> reusable;
  int64_t launches_per_replay = 0;
};

struct tfjs_cuda_event {
  cudaEvent_t ev = nullptr;
  int device = 0;
};

struct tfjs_cuda_ctx {
  int device = 0;
  int sm_count = 0;
  cudaStream_t stream = nullptr;
  cudaStream_t copy_stream = nullptr;   // created on the first tensor_write_async
  cudaEvent_t compute_mark = nullptr;   // orders an upload after the kernels already enqueued
  std::string last_error;
  std::unordered_map<tfjs_tensor_id, TensorEntry> tensors;
  tfjs_tensor_id next_id = 1;
  // caching allocator: size class -> free buffers
  std::map<size_t, std::vector<void*>> free_lists;
  int64_t bytes_in_use = 0, bytes_reserved = 0, num_device_allocs = 0, num_cached = 0;
  // options
  int math_mode = TFJS_MATH_TF32X3;
  bool use_tensor_cores = true;
  bool debug_sync = false;
  // Quantised matmul / 1x1-conv weights: false expands them once into cached tf32 planes, true
  // keeps them uint8 and dequantises every tile in shared memory inside the GEMM main loop.
  bool dequant_in_gemm = false;
  // separable_conv2d: 0 = always two kernels, 1 = one fused kernel where that is faster,
  // 2 = fused wherever the kernel takes the shape
  int fuse_separable = 1;
  // launch the kernels that support it with programmatic stream serialization (off by default:
  // with one persistent block per SM the next kernel's blocks cannot become resident before this
  // kernel's blocks retire, and the measured step time is 0.5-3 % worse with it on)
  bool use_pdl = false;
  // bookkeeping
  int64_t launch_count = 0;
  cudaEvent_t time_start = nullptr, time_stop = nullptr;
  int64_t time_start_launches = 0;
  // per-kernel profile: while enabled, an event is recorded after every launch
  bool profiling = false;
  std::vector<cudaEvent_t> profile_events;   // [0] is the start marker
  std::vector<const char*> profile_names;    // name of the launch that precedes event i+1
  size_t profile_used = 0;
  // graph capture
  tfjs_cuda_graph* capturing = nullptr;
  int64_t capture_start_launches = 0;
  // device-side status word written by kernels whose bounded waits gave up
  int* d_status = nullptr;
  int* h_status = nullptr;  // pinned mirror
};

int set_error(tfjs_cuda_ctx* ctx, int code, const char* fmt, ...);

#define TFJS_CHECK_CUDA(ctx, expr)                                                        \
  do {                                                                                    \
    cudaError_t _e = (expr);                                                              \
    if (_e != cudaSuccess)                                                                \
      return set_error(ctx, _e == cudaErrorMemoryAllocation ? TFJS_CUDA_ERR_OOM           \
                                                            : TFJS_CUDA_ERR_CUDA,         \
                       "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__,  \
                       __LINE__);                                                         \
  } while (0)

#define TFJS_REQUIRE(ctx, cond, ...)                                        \
  do {                                                                      \
    if (!(cond)) return set_error(ctx, TFJS_CUDA_ERR_INVALID_ARG, __VA_ARGS__); \
  } while (0)

// Called after every kernel launch: counts it and surfaces launch errors.
int post_launch(tfjs_cuda_ctx* ctx, const char* what);

// kernel<<<grid, block, smem, ctx->stream>>>(args...) with the programmatic-serialization launch
// attribute when the context allows it (the kernel must call pdl_wait() before touching global
// memory).  Errors surface through post_launch.
template <typename... Params, typename... Args>
inline void launch_ex(tfjs_cuda_ctx* ctx, void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem,
                      Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->use_pdl ? 1 : 0;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);
}

// Allocator (context.cu).
int ctx_alloc(tfjs_cuda_ctx* ctx, size_t nbytes, void** ptr, size_t* capacity);
void ctx_free(tfjs_cuda_ctx* ctx, void* ptr, size_t capacity);

TensorEntry* find_tensor(tfjs_cuda_ctx* ctx, tfjs_tensor_id id);
// Looks the id up and checks dtype float32 with at least `min_elems` elements.
int get_f32(tfjs_cuda_ctx* ctx, tfjs_tensor_id id, int64_t min_elems, const char* what,
            TensorEntry** out);

static inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Epilogue resolved to device pointers, passed by value to kernels.
struct EpilogueArgs {
  const float* bias = nullptr;
  int bias_scalar = 0;  // 1: bias[0] for every channel
  int activation = TFJS_ACT_LINEAR;
  const float* prelu = nullptr;
  int prelu_scalar = 0;
  float clip_lo = 0.f, clip_hi = 0.f;
};
int resolve_epilogue(tfjs_cuda_ctx* ctx, const tfjs_epilogue* epi, int64_t channels,
                     EpilogueArgs* out);

// NaN-propagating max / min (PTX max.NaN / min.NaN): max_nan(v, 0) is Math.max(0, v) and
// min_nan(max_nan(v, lo), hi) is `v > hi ? hi : (v < lo ? lo : v)` for lo <= hi, NaN included.
__device__ __forceinline__ float max_nan(float a, float b) {
  float d;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
  return d;
}
__device__ __forceinline__ float min_nan(float a, float b) {
  float d;
  asm("min.NaN.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
  return d;
}

// Programmatic dependent launch.  A kernel launched through launch_ex may start while the
// kernel before it on the stream is still running; pdl_wait() blocks until that kernel (and
// therefore everything before it) has completed and its writes are visible, and must precede
// every access to global memory.  pdl_launch_dependents() then lets the next kernel's blocks be
// scheduled as this kernel's blocks retire, so that its launch latency and prologue overlap
// this kernel's tail.  It is called after pdl_wait(), which keeps the chain transitive: when a
// kernel starts, all kernels before its predecessor have finished.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// act(v + bias) with the NaN behaviour of MathBackendCPU: relu is Math.max(0, v) (keeps NaN),
// clip is `v > hi ? hi : (v < lo ? lo : v)` (keeps NaN), prelu is `v < 0 ? a * v : v`.
__device__ __forceinline__ float apply_epilogue(float v, int c, const EpilogueArgs& e) {
  if (e.bias) v = v + (e.bias_scalar ? e.bias[0] : e.bias[c]);
  switch (e.activation) {
    case TFJS_ACT_RELU: v = (v < 0.f) ? 0.f : v; break;
    case TFJS_ACT_PRELU: {
      float a = e.prelu_scalar ? e.prelu[0] : e.prelu[c];
      v = (v < 0.f) ? a * v : v;
      break;
    }
    case TFJS_ACT_CLIP: v = (v > e.clip_hi) ? e.clip_hi : ((v < e.clip_lo) ? e.clip_lo : v); break;
    default: break;
  }
  return v;
}

// ---- kernel launchers implemented in the other translation units -------------------------
// gemm_simt.cu
int launch_gemm_simt(tfjs_cuda_ctx* ctx, const float* a, const float* b, float* out, int batch,
                     int M, int N, int K, int64_t a_batch, int64_t a_row, int64_t a_col,
                     int64_t b_batch, int64_t b_row, int64_t b_col, const EpilogueArgs& epi);
int launch_pack_weights(tfjs_cuda_ctx* ctx, const void* src, bool src_is_u8, double scale,
                        double min, int64_t K, int64_t N, int64_t src_k_stride,
                        int64_t src_n_stride, int64_t kp, float* hi, float* lo);
int launch_pack_weights_rows(tfjs_cuda_ctx* ctx, const void* src, bool src_is_u8, double scale,
                             double min, int64_t K, int64_t N, int row_len, int row_pad, int64_t kp,
                             float* hi, float* lo);
int launch_transpose_batched(tfjs_cuda_ctx* ctx, const float* src, float* dst, int batch,
                             int rows, int cols);
int launch_pack_u8(tfjs_cuda_ctx* ctx, const uint8_t* src, int64_t K, int64_t N, int64_t k_stride,
                   int64_t n_stride, int64_t kq, uint8_t* dst);
int launch_dequant(tfjs_cuda_ctx* ctx, const uint8_t* q, float* out, int64_t n, double scale,
                   double min);
// gemm_tcgen05.cu
bool tcgen05_gemm_supported(int64_t M, int64_t N, int64_t K);
int launch_gemm_tcgen05(tfjs_cuda_ctx* ctx, const float* a, int64_t M, int64_t K,
                        const float* w_hi, const float* w_lo, int64_t kp, float* out, int64_t N,
                        const EpilogueArgs& epi, int math_mode);
// Same contraction with the weights as K-major uint8 [N, kq] (kq a multiple of 16, zero
// padded): w = q*scale + min is evaluated in shared memory inside the main loop.
int launch_gemm_tcgen05_u8(tfjs_cuda_ctx* ctx, const float* a, int64_t M, int64_t K,
                           const uint8_t* w_q, int64_t kq, double scale, double min, float* out,
                           int64_t N, const EpilogueArgs& epi, int math_mode);
// Implicit-GEMM convolution on the tensor cores: mode 0 = not eligible, otherwise the gather
// flavour; tcgen05_conv_k is the contraction length the packed weights must have.
int tcgen05_conv_mode(const tfjs_conv2d_info& ci);
int64_t tcgen05_conv_k(const tfjs_conv2d_info& ci, int mode);
int launch_conv_tcgen05(tfjs_cuda_ctx* ctx, int mode, const float* x, const tfjs_conv2d_info& ci,
                        const float* w_hi, const float* w_lo, int64_t kp, float* out,
                        const EpilogueArgs& epi, int math_mode);
// sepconv_tcgen05.cu: depthwise 3x3 (+bias, activation) fused into the pointwise GEMM that
// consumes it; `supported` says whether the fused kernel takes the shapes (else the caller runs
// the two kernels back to back).
bool sepconv_tcgen05_supported(const tfjs_conv2d_info& dw, int64_t N, int dw_activation, int pw_activation,
                               int math_mode);
int launch_sepconv_tcgen05(tfjs_cuda_ctx* ctx, const float* x, const tfjs_conv2d_info& dw, const float* dw_filter,
                           const EpilogueArgs& dw_epi, const float* w_hi, int64_t kp, float* y, int64_t N,
                           const EpilogueArgs& pw_epi);
bool conv_rgb_tcgen05_supported(const tfjs_conv2d_info& ci, int activation, int math_mode);
int launch_conv_rgb_tcgen05(tfjs_cuda_ctx* ctx, const float* x, const tfjs_conv2d_info& ci, const float* w_hi,
                            int64_t kp, float* y, const EpilogueArgs& epi);
bool conv_tma_tcgen05_supported(const tfjs_conv2d_info& ci, int activation, int math_mode);
int launch_conv_tma_tcgen05(tfjs_cuda_ctx* ctx, const float* x, const tfjs_conv2d_info& ci, const float* w_hi,
                            int64_t kp, float* y, const EpilogueArgs& epi);
// conv.cu
int launch_conv2d_direct(tfjs_cuda_ctx* ctx, const float* x, const float* w, float* y,
                         const tfjs_conv2d_info& ci, const EpilogueArgs& epi);
// 3x3 depthwise on 14x14 / 7x7 images through whole-image TMA windows (depthwise_tma.cu)
bool depthwise_image_supported(const tfjs_conv2d_info& ci, int activation);
int launch_depthwise_image(tfjs_cuda_ctx* ctx, const float* x, const float* w, float* y, const tfjs_conv2d_info& ci,
                           const EpilogueArgs& epi);
int launch_depthwise(tfjs_cuda_ctx* ctx, const float* x, const float* w, float* y,
                     const tfjs_conv2d_info& ci, const EpilogueArgs& epi);
int launch_pool2d(tfjs_cuda_ctx* ctx, const float* x, float* y, const tfjs_conv2d_info& ci,
                  int is_avg);
