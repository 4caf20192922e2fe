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
  // == version when the host wrote the current contents and every value was finite (checked on
  // small float tensors only): kernels whose padding relies on 0 * tap == 0 need finite taps
  uint64_t finite_version = ~0ull;
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
  // K-major IEEE half plane [N, kp] of a contraction operand, for the kind::f16 kernel that
  // serves 16-bit activation storage
  void* w16 = nullptr;
  size_t w16_capacity = 0;
  int64_t w16_n = 0, w16_k = 0, w16_kp = 0;
  uint64_t w16_version = ~0ull;
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
  int gemm_block_n = 0;  // diagnostic: tile width of the single-CTA GEMM (32 .. 256) instead of the cost model's choice
  int gemm_pair = 1;  // 0: never use the CTA-pair GEMM, 1: where it pays, 2: wherever its shape rules allow
  // launch the kernels that support it with programmatic stream serialization (off by default:
  // with one persistent block per SM the next kernel's blocks cannot become resident before this
  // kernel's blocks retire, and the measured step time is 0.5-3 % worse with it on)
  bool use_pdl = false;
  // debug_canary: every buffer handed out by the allocator is followed by a 256-byte guard
  // pattern that is verified when the buffer is released; a kernel that wrote past the end of its
  // output is then reported through the status word at the next synchronisation (the substitute
  // for a memory checker on machines where none can run)
  bool debug_canary = false;
  std::unordered_map<void*, size_t> canary_offset;  // buffer -> byte offset of its guard
  // Diagnostic: the tensor-core GEMM withholds the last load of every CTA, so that the bounded
  // wait of its consumers runs out and the error path (status word, TFJS_CUDA_ERR_TIMEOUT,
  // context still usable) can be exercised without a fault
  bool test_withhold_last_load = false;
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
inline bool known_finite(const TensorEntry* t) { return t->finite_version == t->version; }
// Looks the id up and checks dtype float32 with at least `min_elems` elements.
int get_f32(tfjs_cuda_ctx* ctx, tfjs_tensor_id id, int64_t min_elems, const char* what,
            TensorEntry** out);

// An activation operand: float32 or half-precision storage.
int get_activation(tfjs_cuda_ctx* ctx, tfjs_tensor_id id, int64_t min_elems, const char* what,
                   TensorEntry** out);
// elementwise.cu: dst[i] = convert(src[i]) between the storage dtypes (float32, int32, bool, float16)
int launch_convert(tfjs_cuda_ctx* ctx, const void* src, int src_dtype, void* dst, int dst_dtype, int64_t n);

static inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Epilogue resolved to device pointers, passed by value to kernels.
struct EpilogueArgs {
  const float* bias = nullptr;
  int bias_scalar = 0;  // 1: bias[0] for every channel
  int activation = TFJS_ACT_LINEAR;
  const float* prelu = nullptr;
  int prelu_scalar = 0;
  float clip_lo = 0.f, clip_hi = 0.f;
  // Internal (never set through the C ABI): round the result to the nearest tf32 value before
  // storing it (as far as the tensor core can tell: the low 13 bits may be left as they fall).
  // Set for a private intermediate whose only reader is a TF32 tensor-core contraction, which
  // would otherwise truncate it.
  int round_tf32 = 0;
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

// Round to the nearest tf32 value (10 mantissa bits, ties away from zero); the low 13 bits of the
// result are zero, so the tensor core, which reads only the upper 19 bits, takes it exactly.
__device__ __forceinline__ float round_tf32(float v) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
  return __uint_as_float(r);
}

// The same rounding for a value that goes straight to the tensor core, as one integer add: the
// tensor core reads bits [13, 32) only, so adding half a tf32 unit to the bit pattern and letting
// it drop the rest is round-to-nearest (ties away from zero).  inf and NaN are left alone (the add
// would turn inf into NaN).  The low 13 bits of the result are NOT cleared.  cvt.rna.tf32 goes
// through the conversion unit, whose throughput is a fraction of the integer ALU's; on the stem,
// which rounds 27 values per output pixel, that difference was 10 % of the kernel.
__device__ __forceinline__ float round_tf32_for_mma(float v) {
  uint32_t b = __float_as_uint(v);
  b += ((b & 0x7f800000u) != 0x7f800000u) ? 0x1000u : 0u;
  return __uint_as_float(b);
}

// The same for a value that float32 arithmetic on this device has just produced (an fma chain, a
// max.NaN / min.NaN clamp): two instructions instead of three.  Such a value is finite, +-inf or
// the canonical NaN 0x7fffffff.  inf + 0x1000 still reads as inf in the 19 bits the tensor core
// takes; for the NaN the add wraps to a negative integer and the signed max keeps the NaN.  (A
// NaN with the sign bit and all of the top 11 mantissa bits set, which no arithmetic instruction
// returns, would come out as a tiny positive number: operands that arrive from the caller go
// through round_tf32_for_mma instead.)
__device__ __forceinline__ float round_tf32_after_arith(float v) {
  const int b = __float_as_int(v);
  const int t = (int)((uint32_t)b + 0x1000u);
  return __int_as_float(max(t, b));
}

// Codes a kernel may leave in the context's device status word besides the number of the bounded
// wait that gave up (1 .. 89): the host turns them into errors at the next synchronisation.
constexpr int STATUS_CANARY = 90;       // a guard pattern behind a buffer was overwritten
constexpr int STATUS_SMEM_LAYOUT = 91;  // a kernel's dynamic shared-memory window did not start 1024-aligned

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
  if (e.round_tf32) v = round_tf32(v);
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
// Limit, in SM clock cycles, of every bounded device-side wait in the three translation units
// that have such waits (each keeps its own copy of the constant); the device must be current.
int set_wait_limit_gemm(long long cycles);
int set_wait_limit_sepconv(long long cycles);
int set_wait_limit_depthwise_image(long long cycles);
int set_wait_limit_gemm_pair(long long cycles);
// gemm_tcgen05_pair.cu: the 256 x 256 tile on a pair of CTAs (tcgen05 cta_group::2); TF32 (w_lo null;
// A rounded on chip unless a_tf32_exact), 3xTF32 (w_lo = the residual weight plane), or TF32 with the
// weights as uint8 bytes dequantised in the main loop (w_q; A tf32-exact)
bool gemm_pair_supported(const tfjs_cuda_ctx* ctx, int64_t M, int64_t K, int64_t N);
int launch_gemm_tcgen05_pair(tfjs_cuda_ctx* ctx, const float* a, int64_t M, int64_t K, const float* w_hi,
                             const float* w_lo, int64_t kp, float* out, int64_t N, const EpilogueArgs& epi,
                             bool a_tf32_exact, const uint8_t* w_q = nullptr, double q_scale = 0.0,
                             double q_min = 0.0);
// gemm_tcgen05.cu
bool tcgen05_gemm_supported(int64_t M, int64_t N, int64_t K);
// a_tf32_exact (TF32 mode only): every element of `a` already has its low 13 mantissa bits zero
// (its producer rounded it), so the kernel may hand the tiles to the tensor core as they are;
// otherwise it rounds them to nearest in shared memory, because the tensor core truncates.
int launch_gemm_tcgen05(tfjs_cuda_ctx* ctx, const float* a, int64_t M, int64_t K,
                        const float* w_hi, const float* w_lo, int64_t kp, float* out, int64_t N,
                        const EpilogueArgs& epi, int math_mode, bool a_tf32_exact = false);
// The contraction on IEEE half operands (16-bit activation storage): a is [M, K] half, w16 the
// K-major half plane [N, kp] (kp a multiple of 8, zero padded), out is float32 or half.
bool tcgen05_gemm_f16_supported(int64_t M, int64_t N, int64_t K, bool out16);
int launch_gemm_tcgen05_f16(tfjs_cuda_ctx* ctx, const void* a, int64_t M, int64_t K, const void* w16, int64_t kp,
                            void* out, bool out16, int64_t N, const EpilogueArgs& epi);
// K-major half plane [N, kp] of a [K, N] operand addressed through strides (float32 or uint8 source)
int launch_pack_weights_f16(tfjs_cuda_ctx* ctx, const void* src, bool src_is_u8, double scale, double min,
                            int64_t K, int64_t N, int64_t src_k_stride, int64_t src_n_stride, int64_t kp,
                            void* dst);
// Same contraction with the weights as K-major uint8 [N, kq] (kq a multiple of 16, zero
// padded): w = q*scale + min is evaluated in shared memory inside the main loop.
int launch_gemm_tcgen05_u8(tfjs_cuda_ctx* ctx, const float* a, int64_t M, int64_t K,
                           const uint8_t* w_q, int64_t kq, double scale, double min, float* out,
                           int64_t N, const EpilogueArgs& epi, int math_mode, bool a_tf32_exact = false);
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
// half: x and y are stored as IEEE half (16-bit activation storage); weights and biases are float32
int launch_sepconv_tcgen05(tfjs_cuda_ctx* ctx, const void* x, const tfjs_conv2d_info& dw, const float* dw_filter,
                           const EpilogueArgs& dw_epi, const float* w_hi, int64_t kp, void* y, int64_t N,
                           const EpilogueArgs& pw_epi, bool half = false);
bool conv_rgb_tcgen05_supported(const tfjs_conv2d_info& ci, int activation, int math_mode);
// in_u8: x holds one unsigned byte per value (image pixels), decoded on chip as q * q_scale + q_min
bool conv_rgb_u8_tcgen05_supported(const tfjs_conv2d_info& ci, int activation, int math_mode);
int launch_conv_rgb_tcgen05(tfjs_cuda_ctx* ctx, const void* x, const tfjs_conv2d_info& ci, const float* w_hi,
                            int64_t kp, void* y, const EpilogueArgs& epi, bool out_half = false, bool in_u8 = false,
                            double q_scale = 0.0, double q_min = 0.0, const float* w_lo = nullptr);
bool conv_tma_tcgen05_supported(const tfjs_conv2d_info& ci, int activation, int math_mode);
int launch_conv_tma_tcgen05(tfjs_cuda_ctx* ctx, const float* x, const tfjs_conv2d_info& ci, const float* w_hi,
                            int64_t kp, float* y, const EpilogueArgs& epi, const float* w_lo = nullptr);
// conv.cu
int launch_conv2d_direct(tfjs_cuda_ctx* ctx, const float* x, const float* w, float* y,
                         const tfjs_conv2d_info& ci, const EpilogueArgs& epi);
// 3x3 depthwise on 14x14 / 7x7 images through whole-image TMA windows (depthwise_tma.cu)
// half: x and y are stored as IEEE half (16-bit activation storage); the filter and bias stay float32
bool depthwise_image_supported(const tfjs_conv2d_info& ci, int activation, bool half = false);
int launch_depthwise_image(tfjs_cuda_ctx* ctx, const void* x, const float* w, void* y, const tfjs_conv2d_info& ci,
                           const EpilogueArgs& epi, bool half = false);
int launch_depthwise(tfjs_cuda_ctx* ctx, const float* x, const float* w, float* y,
                     const tfjs_conv2d_info& ci, const EpilogueArgs& epi);
int launch_pool2d(tfjs_cuda_ctx* ctx, const float* x, float* y, const tfjs_conv2d_info& ci,
                  int is_avg);
// global average pool (window = whole image) of a half-stored image into float32
bool global_avgpool_half_supported(const tfjs_conv2d_info& ci, int is_avg, const void* x, const void* y);
int launch_global_avgpool_half(tfjs_cuda_ctx* ctx, const void* x, float* y, const tfjs_conv2d_info& ci);
