// Memory-bound element-wise, reduction and softmax kernels.
//
// Arithmetic follows MathBackendCPU (tfjs-core/src/backends/cpu/backend_cpu.ts): binary ops
// are single float32 operations (a float64 op on two float32 values, rounded once, is the
// float32 op); exp/log are evaluated in float64 and rounded once, like Math.exp/Math.log
// stored into a Float32Array; sum accumulates in float64.
#include <cuda_fp16.h>

#include "common.cuh"

namespace {

constexpr int kThreads = 256;

inline int grid_for(int64_t work_items, int sm_count, int per_sm = 8) {
  int64_t blocks = ceil_div64(work_items, kThreads);
  int64_t cap = (int64_t)sm_count * per_sm;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

__device__ __forceinline__ float binary_apply(int op, float a, float b) {
  switch (op) {
    case TFJS_BIN_ADD: return a + b;
    case TFJS_BIN_SUB: return a - b;
    case TFJS_BIN_MUL: return a * b;
    case TFJS_BIN_DIV: return __fdiv_rn(a, b);
    case TFJS_BIN_PRELU: return a < 0.f ? b * a : a;
    default: return 0.f;
  }
}

// out[i] = op(a[i], b[i]) for two operands of the same length, 128-bit accesses.
template <int OP>
__global__ void binary_same_kernel(const float4* __restrict__ a, const float4* __restrict__ b,
                                   float4* __restrict__ out, int64_t n4) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4;
       i += (int64_t)gridDim.x * blockDim.x) {
    float4 x = a[i], y = b[i], r;
    r.x = binary_apply(OP, x.x, y.x);
    r.y = binary_apply(OP, x.y, y.y);
    r.z = binary_apply(OP, x.z, y.z);
    r.w = binary_apply(OP, x.w, y.w);
    out[i] = r;
  }
}

// The reference's modulo fast path (backend_cpu.ts:3527-3530) for an operand that repeats
// along the inner-most axis: out[i] = op(a[i], b[i % nb]) with nb a multiple of 4, so that a
// float4 of `a` lines up with a float4 of `b` (bias add over NHWC channels).
template <int OP, bool SWAP>
__global__ void binary_rowvec_kernel(const float4* __restrict__ a, const float4* __restrict__ b,
                                     float4* __restrict__ out, int64_t n4, int nb4) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4;
       i += (int64_t)gridDim.x * blockDim.x) {
    float4 x = a[i], y = __ldg(&b[i % nb4]), r;
    if (SWAP) {
      r.x = binary_apply(OP, y.x, x.x);
      r.y = binary_apply(OP, y.y, x.y);
      r.z = binary_apply(OP, y.z, x.z);
      r.w = binary_apply(OP, y.w, x.w);
    } else {
      r.x = binary_apply(OP, x.x, y.x);
      r.y = binary_apply(OP, x.y, y.y);
      r.z = binary_apply(OP, x.z, y.z);
      r.w = binary_apply(OP, x.w, y.w);
    }
    out[i] = r;
  }
}

struct BroadcastDesc {
  int rank;
  int64_t out_dims[8];
  int64_t a_strides[8];  // 0 where the operand is broadcast
  int64_t b_strides[8];
};

// General path: indexToLoc / locToIndex of backend_cpu.ts:3532-3546 as stride arithmetic.
__global__ void binary_general_kernel(int op, const float* __restrict__ a,
                                      const float* __restrict__ b, void* __restrict__ out,
                                      int64_t n, BroadcastDesc d, int out_is_bool) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    int64_t rem = i, ai = 0, bi = 0;
    for (int k = d.rank - 1; k >= 0; --k) {
      int64_t c = rem % d.out_dims[k];
      rem /= d.out_dims[k];
      ai += c * d.a_strides[k];
      bi += c * d.b_strides[k];
    }
    float x = a[ai], y = b[bi];
    if (out_is_bool)
      ((uint8_t*)out)[i] = (x != y) ? 1 : 0;
    else
      ((float*)out)[i] = binary_apply(op, x, y);
  }
}

__device__ __forceinline__ float unary_apply(int op, float v, float p0, float p1) {
  switch (op) {
    case TFJS_UN_RELU: return (v < 0.f) ? 0.f : v;  // Math.max(0, v): NaN stays NaN
    case TFJS_UN_CLIP: return v > p1 ? p1 : (v < p0 ? p0 : v);
    case TFJS_UN_EXP: return (float)exp((double)v);
    case TFJS_UN_LOG: return (float)log((double)v);
    case TFJS_UN_STEP: return (v != v) ? v : (v > 0.f ? 1.f : p0);  // backend_cpu.ts:1520-1534
    default: return v;
  }
}

template <int OP>
__global__ void unary_kernel(const float* __restrict__ x, float* __restrict__ out, int64_t n,
                             float p0, float p1) {
  const int64_t n4 = n / 4;
  const float4* x4 = reinterpret_cast<const float4*>(x);
  float4* o4 = reinterpret_cast<float4*>(out);
  const int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = tid; i < n4; i += stride) {
    float4 v = x4[i], r;
    r.x = unary_apply(OP, v.x, p0, p1);
    r.y = unary_apply(OP, v.y, p0, p1);
    r.z = unary_apply(OP, v.z, p0, p1);
    r.w = unary_apply(OP, v.w, p0, p1);
    o4[i] = r;
  }
  for (int64_t i = n4 * 4 + tid; i < n; i += stride) out[i] = unary_apply(OP, x[i], p0, p1);
}

// dtype conversions: KernelBackend.int (truncation toward zero, backend_cpu.ts `int`),
// castTensor (backend_util.ts:36-71).
__global__ void cast_kernel(const void* __restrict__ src, int src_dtype, void* __restrict__ dst,
                            int dst_dtype, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    float v;
    if (src_dtype == TFJS_F32) v = ((const float*)src)[i];
    else if (src_dtype == TFJS_F16) v = __half2float(((const __half*)src)[i]);
    else if (src_dtype == TFJS_I32) v = (float)((const int32_t*)src)[i];
    else v = ((const uint8_t*)src)[i] ? 1.f : 0.f;
    if (dst_dtype == TFJS_F32) ((float*)dst)[i] = v;
    else if (dst_dtype == TFJS_F16) ((__half*)dst)[i] = __float2half_rn(v);
    else if (dst_dtype == TFJS_I32) ((int32_t*)dst)[i] = (src_dtype == TFJS_F32) ? (int32_t)v : (int32_t)v;
    else ((uint8_t*)dst)[i] = (v != 0.f) ? 1 : 0;
  }
}

// float32 <-> float16, 8 elements (16 / 32 bytes) per thread step
__global__ void convert_half_kernel(const void* __restrict__ src, void* __restrict__ dst, int to_half, int64_t n8) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n8; i += (int64_t)gridDim.x * blockDim.x) {
    if (to_half) {
      const float4 a = ((const float4*)src)[2 * i], b = ((const float4*)src)[2 * i + 1];
      __half2 h[4] = {__floats2half2_rn(a.x, a.y), __floats2half2_rn(a.z, a.w), __floats2half2_rn(b.x, b.y),
                      __floats2half2_rn(b.z, b.w)};
      ((uint4*)dst)[i] = *reinterpret_cast<uint4*>(h);
    } else {
      uint4 raw = ((const uint4*)src)[i];
      const __half2* h = reinterpret_cast<const __half2*>(&raw);
      const float2 p0 = __half22float2(h[0]), p1 = __half22float2(h[1]), p2 = __half22float2(h[2]),
                   p3 = __half22float2(h[3]);
      ((float4*)dst)[2 * i] = make_float4(p0.x, p0.y, p1.x, p1.y);
      ((float4*)dst)[2 * i + 1] = make_float4(p2.x, p2.y, p3.x, p3.y);
    }
  }
}

__global__ void dequant_kernel(const uint8_t* __restrict__ q, float* __restrict__ out, int64_t n,
                               double scale, double mn) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    out[i] = (float)((double)q[i] * scale + mn);  // io_utils.ts:139, evaluated in float64
}

__device__ __forceinline__ double warp_sum(double v) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

constexpr int kNoIndex = 0x7fffffff;

// Merge step of the max/argMax reduction.  The reference scans left to right and replaces
// the running maximum only when `value > max` (backend_cpu.ts:697-705, 914-921): NaNs never
// win and ties keep the smaller index.  idx == kNoIndex marks a lane that saw no number.
__device__ __forceinline__ void warp_argmax(float& m, int& idx) {
  for (int o = 16; o > 0; o >>= 1) {
    float om = __shfl_xor_sync(0xffffffffu, m, o);
    int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (oi != kNoIndex && (idx == kNoIndex || om > m || (om == m && oi < idx))) {
      m = om;
      idx = oi;
    }
  }
}

// One warp per row.  sum: float64 accumulation, one rounding (backend_cpu.ts:601-607).
__global__ void reduce_last_kernel(int op, const float* __restrict__ x, void* __restrict__ out,
                                   int64_t outer, int64_t inner) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t row = warp; row < outer; row += nwarps) {
    const float* r = x + row * inner;
    if (op == TFJS_RED_SUM) {
      double s = 0.0;
      for (int64_t j = lane; j < inner; j += 32) s += (double)r[j];
      s = warp_sum(s);
      if (lane == 0) ((float*)out)[row] = (float)s;
    } else {
      // The reference seeds max with element 0, so a NaN there is never replaced.
      const float first = r[0];
      float m = 0.f;
      int idx = kNoIndex;
      for (int64_t j = lane; j < inner; j += 32) {
        float v = r[j];
        if (v == v && (idx == kNoIndex || v > m)) { m = v; idx = (int)j; }
      }
      warp_argmax(m, idx);
      if (lane == 0) {
        if (first != first || idx == kNoIndex) { m = first; idx = 0; }
        if (op == TFJS_RED_MAX) ((float*)out)[row] = m;
        else ((int32_t*)out)[row] = idx;
      }
    }
  }
}

// tf.softmax over the last axis in one pass per row, one warp per row, reproducing the
// rounding points of the op-layer chain (softmax.ts:57-63, reduction_ops.ts:56-73):
//   m = max(x); a = f32(x - m); b = f32(exp(a)); c = f32(sum_f64(b)); d = f32(log(c));
//   lse = f32(m + d); out = f32(exp(f32(x - lse))).
__global__ void softmax_last_kernel(const float* __restrict__ x, float* __restrict__ out,
                                    int64_t outer, int64_t inner) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t row = warp; row < outer; row += nwarps) {
    const float* r = x + row * inner;
    float first = r[0];
    float m = -INFINITY;
    bool any = false;
    for (int64_t j = lane; j < inner; j += 32) {
      float v = r[j];
      if (v == v && (!any || v > m)) { m = v; any = true; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      float om = __shfl_xor_sync(0xffffffffu, m, o);
      int oa = __shfl_xor_sync(0xffffffffu, (int)any, o);
      if (oa && (!any || om > m)) { m = om; any = true; }
    }
    if (first != first || !any) m = first;  // NaN seed sticks (backend_cpu.ts:914)
    double c = 0.0;
    for (int64_t j = lane; j < inner; j += 32) {
      float a = r[j] - m;
      float b = (float)exp((double)a);
      c += (double)b;
    }
    c = warp_sum(c);
    float cf = (float)c;
    float d = (float)log((double)cf);
    float lse = m + d;
    for (int64_t j = lane; j < inner; j += 32) {
      float lr = r[j] - lse;
      out[row * inner + j] = (float)exp((double)lr);
    }
  }
}

// The same softmax with one 256-thread block per row and the row held in registers (up to
// PER * 256 elements): the float64 exp / log chains of a row run on 8 warps instead of one.
template <int PER>
__global__ void __launch_bounds__(256) softmax_last_block_kernel(const float* __restrict__ x,
                                                                  float* __restrict__ out, int64_t outer,
                                                                  int inner) {
  __shared__ float s_m[8];
  __shared__ int s_any[8];
  __shared__ double s_c[8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  pdl_wait();
  pdl_launch_dependents();
  for (int64_t row = blockIdx.x; row < outer; row += gridDim.x) {
    const float* r = x + row * inner;
    float v[PER];
    float m = -INFINITY;
    bool any = false;
#pragma unroll
    for (int i = 0; i < PER; i++) {
      const int j = threadIdx.x + i * 256;
      v[i] = j < inner ? r[j] : 0.f;
      if (j < inner && v[i] == v[i] && (!any || v[i] > m)) { m = v[i]; any = true; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o);
      const int oa = __shfl_xor_sync(0xffffffffu, (int)any, o);
      if (oa && (!any || om > m)) { m = om; any = true; }
    }
    __syncthreads();  // the previous row's readers of the shared arrays are done
    if (lane == 0) { s_m[warp] = m; s_any[warp] = any; }
    __syncthreads();
    m = -INFINITY;
    any = false;
#pragma unroll
    for (int w = 0; w < 8; w++)
      if (s_any[w] && (!any || s_m[w] > m)) { m = s_m[w]; any = true; }
    const float first = r[0];
    if (first != first || !any) m = first;  // NaN seed sticks (backend_cpu.ts:914)
    double c = 0.0;
#pragma unroll
    for (int i = 0; i < PER; i++) {
      if (threadIdx.x + i * 256 < inner) {
        const float a = v[i] - m;
        c += (double)(float)exp((double)a);
      }
    }
    c = warp_sum(c);
    if (lane == 0) s_c[warp] = c;
    __syncthreads();
    c = 0.0;
#pragma unroll
    for (int w = 0; w < 8; w++) c += s_c[w];
    const float cf = (float)c;
    const float d = (float)log((double)cf);
    const float lse = m + d;
#pragma unroll
    for (int i = 0; i < PER; i++) {
      const int j = threadIdx.x + i * 256;
      if (j < inner) out[row * inner + j] = (float)exp((double)(v[i] - lse));
    }
  }
}

}  // namespace

int launch_dequant(tfjs_cuda_ctx* ctx, const uint8_t* q, float* out, int64_t n, double scale,
                   double mn) {
  if (n == 0) return TFJS_CUDA_OK;
  dequant_kernel<<<grid_for(n, ctx->sm_count), kThreads, 0, ctx->stream>>>(q, out, n, scale, mn);
  return post_launch(ctx, "dequant");
}

template <int OP>
static void launch_binary_fast(tfjs_cuda_ctx* ctx, const float* a, const float* b, float* out,
                               int64_t n, int64_t na, int64_t nb) {
  const int64_t n4 = n / 4;
  const int grid = grid_for(n4, ctx->sm_count);
  if (na == nb) {
    binary_same_kernel<OP><<<grid, kThreads, 0, ctx->stream>>>(
        (const float4*)a, (const float4*)b, (float4*)out, n4);
  } else if (na == n) {
    binary_rowvec_kernel<OP, false><<<grid, kThreads, 0, ctx->stream>>>(
        (const float4*)a, (const float4*)b, (float4*)out, n4, (int)(nb / 4));
  } else {
    binary_rowvec_kernel<OP, true><<<grid, kThreads, 0, ctx->stream>>>(
        (const float4*)b, (const float4*)a, (float4*)out, n4, (int)(na / 4));
  }
}

static bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

extern "C" int tfjs_cuda_binary(tfjs_cuda_ctx* ctx, int op, tfjs_tensor_id a_id, int a_rank,
                                const int64_t* a_shape, tfjs_tensor_id b_id, int b_rank,
                                const int64_t* b_shape, tfjs_tensor_id out_id) {
  if (!ctx) return TFJS_CUDA_ERR_INVALID_ARG;
  TFJS_REQUIRE(ctx, op >= TFJS_BIN_ADD && op <= TFJS_BIN_NOT_EQUAL, "unknown binary op %d", op);
  TFJS_REQUIRE(ctx, a_rank >= 0 && a_rank <= 8 && b_rank >= 0 && b_rank <= 8, "rank out of range");
  // broadcast_util.ts:58-87 assertAndGetBroadcastShape
  BroadcastDesc d;
  d.rank = a_rank > b_rank ? a_rank : b_rank;
  int64_t n = 1, na = 1, nb = 1;
  bool stretched = false;  // getBroadcastDims non-empty: a size-1 dim stretched to >1
  {
    int64_t sa = 1, sb = 1;
    for (int i = 0; i < d.rank; i++) {
      int64_t da = i < a_rank ? a_shape[a_rank - 1 - i] : 1;
      int64_t db = i < b_rank ? b_shape[b_rank - 1 - i] : 1;
      int64_t r;
      if (da == 1) r = db;
      else if (db == 1) r = da;
      else if (da != db)
        return set_error(ctx, TFJS_CUDA_ERR_INVALID_ARG,
                         "Operands could not be broadcast together");
      else r = da;
      int k = d.rank - 1 - i;
      d.out_dims[k] = r;
      d.a_strides[k] = (i < a_rank && da != 1) ? sa : 0;
      d.b_strides[k] = (i < b_rank && db != 1) ? sb : 0;
      if (i < a_rank && da == 1 && r > 1) stretched = true;
      if (i < b_rank && db == 1 && r > 1) stretched = true;
      sa *= da;
      sb *= db;
      n *= r;
    }
    na = sa;
    nb = sb;
  }
  TensorEntry *a, *b;
  int rc = get_f32(ctx, a_id, na, "a", &a);
  if (rc) return rc;
  rc = get_f32(ctx, b_id, nb, "b", &b);
  if (rc) return rc;
  TFJS_REQUIRE(ctx, !a->quant.quantized && !b->quant.quantized, "binary ops take float tensors");
  TensorEntry* o = find_tensor(ctx, out_id);
  if (!o) return set_error(ctx, TFJS_CUDA_ERR_NOT_FOUND, "binary: unknown output id");
  const bool out_bool = op == TFJS_BIN_NOT_EQUAL;
  TFJS_REQUIRE(ctx, o->dtype == (out_bool ? TFJS_BOOL : TFJS_F32) && o->size == n,
               "binary: output has the wrong dtype or size (%lld elements expected)", (long long)n);
  o->version++;
  if (n == 0) return TFJS_CUDA_OK;
  cudaSetDevice(ctx->device);
  const float* ap = (const float*)a->ptr;
  const float* bp = (const float*)b->ptr;
  // Fast paths: no stretched dims, so out[i] = op(a[i % na], b[i % nb]); taken when one
  // operand spans the whole output and the other divides it in float4 units.
  const bool fast = !out_bool && !stretched && n % 4 == 0 && (na == n || nb == n) &&
                    na % 4 == 0 && nb % 4 == 0 && aligned16(ap) && aligned16(bp) &&
                    aligned16(o->ptr);
  if (fast) {
    float* op_out = (float*)o->ptr;
    switch (op) {
      case TFJS_BIN_ADD: launch_binary_fast<TFJS_BIN_ADD>(ctx, ap, bp, op_out, n, na, nb); break;
      case TFJS_BIN_SUB: launch_binary_fast<TFJS_BIN_SUB>(ctx, ap, bp, op_out, n, na, nb); break;
      case TFJS_BIN_MUL: launch_binary_fast<TFJS_BIN_MUL>(ctx, ap, bp, op_out, n, na, nb); break;
      case TFJS_BIN_DIV: launch_binary_fast<TFJS_BIN_DIV>(ctx, ap, bp, op_out, n, na, nb); break;
      default: launch_binary_fast<TFJS_BIN_PRELU>(ctx, ap, bp, op_out, n, na, nb); break;
    }
    return post_launch(ctx, "binary (vectorised)");
  }
  binary_general_kernel<<<grid_for(n, ctx->sm_count), kThreads, 0, ctx->stream>>>(
      op, ap, bp, o->ptr, n, d, out_bool ? 1 : 0);
  return post_launch(ctx, "binary (general)");
}

extern "C" int tfjs_cuda_unary(tfjs_cuda_ctx* ctx, int op, tfjs_tensor_id x_id,
                               tfjs_tensor_id out_id, float p0, float p1) {
  if (!ctx) return TFJS_CUDA_ERR_INVALID_ARG;
  TFJS_REQUIRE(ctx, op >= TFJS_UN_RELU && op <= TFJS_UN_STEP, "unknown unary op %d", op);
  TensorEntry* x;
  int rc = get_f32(ctx, x_id, 0, "x", &x);
  if (rc) return rc;
  TFJS_REQUIRE(ctx, !x->quant.quantized, "unary ops take float tensors");
  TensorEntry* o = find_tensor(ctx, out_id);
  if (!o) return set_error(ctx, TFJS_CUDA_ERR_NOT_FOUND, "unary: unknown output id");
  TFJS_REQUIRE(ctx, o->size == x->size, "unary: output size differs from input size");
  o->version++;
  const int64_t n = x->size;
  if (n == 0) return TFJS_CUDA_OK;
  cudaSetDevice(ctx->device);
  if (op == TFJS_UN_INT) {
    TFJS_REQUIRE(ctx, o->dtype == TFJS_I32, "int: output must be int32");
    cast_kernel<<<grid_for(n, ctx->sm_count), kThreads, 0, ctx->stream>>>(x->ptr, TFJS_F32, o->ptr,
                                                                           TFJS_I32, n);
    return post_launch(ctx, "int");
  }
  TFJS_REQUIRE(ctx, o->dtype == TFJS_F32, "unary: output must be float32");
  // clip_test 'min greater than max' is rejected by the op layer (unary_ops.ts:448-451).
  const float* xp = (const float*)x->ptr;
  float* outp = (float*)o->ptr;
  const int grid = grid_for(ceil_div64(n, 4), ctx->sm_count);
  switch (op) {
    case TFJS_UN_RELU: unary_kernel<TFJS_UN_RELU><<<grid, kThreads, 0, ctx->stream>>>(xp, outp, n, p0, p1); break;
    case TFJS_UN_CLIP: unary_kernel<TFJS_UN_CLIP><<<grid, kThreads, 0, ctx->stream>>>(xp, outp, n, p0, p1); break;
    case TFJS_UN_EXP: unary_kernel<TFJS_UN_EXP><<<grid, kThreads, 0, ctx->stream>>>(xp, outp, n, p0, p1); break;
    case TFJS_UN_STEP: unary_kernel<TFJS_UN_STEP><<<grid, kThreads, 0, ctx->stream>>>(xp, outp, n, p0, p1); break;
    default: unary_kernel<TFJS_UN_LOG><<<grid, kThreads, 0, ctx->stream>>>(xp, outp, n, p0, p1); break;
  }
  return post_launch(ctx, "unary");
}

int launch_convert(tfjs_cuda_ctx* ctx, const void* src, int src_dtype, void* dst, int dst_dtype, int64_t n) {
  if (n == 0) return TFJS_CUDA_OK;
  const bool halves = (src_dtype == TFJS_F32 && dst_dtype == TFJS_F16) || (src_dtype == TFJS_F16 && dst_dtype == TFJS_F32);
  if (halves && n % 8 == 0 && (((uintptr_t)src | (uintptr_t)dst) & 15) == 0) {
    convert_half_kernel<<<grid_for(n / 8, ctx->sm_count), kThreads, 0, ctx->stream>>>(src, dst, dst_dtype == TFJS_F16,
                                                                                    n / 8);
    return post_launch(ctx, "cast (float16)");
  }
  cast_kernel<<<grid_for(n, ctx->sm_count), kThreads, 0, ctx->stream>>>(src, src_dtype, dst, dst_dtype, n);
  return post_launch(ctx, "cast");
}

extern "C" int tfjs_cuda_cast(tfjs_cuda_ctx* ctx, tfjs_tensor_id x_id, tfjs_tensor_id out_id) {
  if (!ctx) return TFJS_CUDA_ERR_INVALID_ARG;
  TensorEntry* x = find_tensor(ctx, x_id);
  TensorEntry* o = find_tensor(ctx, out_id);
  if (!x || !o) return set_error(ctx, TFJS_CUDA_ERR_NOT_FOUND, "cast: unknown tensor id");
  TFJS_REQUIRE(ctx, x->size == o->size, "cast: sizes differ");
  TFJS_REQUIRE(ctx, !o->quant.quantized, "cast: output cannot be quantised");
  o->version++;
  if (x->size == 0) return TFJS_CUDA_OK;
  cudaSetDevice(ctx->device);
  if (x->quant.quantized) {
    TFJS_REQUIRE(ctx, o->dtype == TFJS_F32, "cast: a quantised tensor converts to float32 only");
    return launch_dequant(ctx, (const uint8_t*)x->ptr, (float*)o->ptr, x->size, x->quant.scale,
                          x->quant.min);
  }
  return launch_convert(ctx, x->ptr, x->dtype, o->ptr, o->dtype, x->size);
}

extern "C" int tfjs_cuda_reduce_last(tfjs_cuda_ctx* ctx, int op, tfjs_tensor_id x_id,
                                     tfjs_tensor_id out_id, int64_t outer, int64_t inner) {
  if (!ctx) return TFJS_CUDA_ERR_INVALID_ARG;
  TFJS_REQUIRE(ctx, op >= TFJS_RED_SUM && op <= TFJS_RED_ARGMAX, "unknown reduce op %d", op);
  TFJS_REQUIRE(ctx, outer >= 0 && inner >= 0, "negative extent");
  TensorEntry* x;
  int rc = get_f32(ctx, x_id, outer * inner, "x", &x);
  if (rc) return rc;
  TensorEntry* o = find_tensor(ctx, out_id);
  if (!o) return set_error(ctx, TFJS_CUDA_ERR_NOT_FOUND, "reduce: unknown output id");
  TFJS_REQUIRE(ctx, o->size == outer, "reduce: output must hold %lld elements", (long long)outer);
  TFJS_REQUIRE(ctx, o->dtype == (op == TFJS_RED_ARGMAX ? TFJS_I32 : TFJS_F32),
               "reduce: output dtype mismatch");
  o->version++;
  if (outer == 0) return TFJS_CUDA_OK;
  cudaSetDevice(ctx->device);
  if (inner == 0) {
    // sum over an empty axis is 0; max/argMax of nothing read element 0 of nothing -> 0 here.
    TFJS_CHECK_CUDA(ctx, cudaMemsetAsync(o->ptr, 0, o->nbytes, ctx->stream));
    return TFJS_CUDA_OK;
  }
  reduce_last_kernel<<<grid_for(outer * 32, ctx->sm_count), kThreads, 0, ctx->stream>>>(
      op, (const float*)x->ptr, o->ptr, outer, inner);
  return post_launch(ctx, "reduce_last");
}

extern "C" int tfjs_cuda_softmax_last(tfjs_cuda_ctx* ctx, tfjs_tensor_id x_id,
                                      tfjs_tensor_id out_id, int64_t outer, int64_t inner) {
  if (!ctx) return TFJS_CUDA_ERR_INVALID_ARG;
  TFJS_REQUIRE(ctx, outer >= 0 && inner >= 0, "negative extent");
  TensorEntry *x, *o;
  int rc = get_f32(ctx, x_id, outer * inner, "logits", &x);
  if (rc) return rc;
  rc = get_f32(ctx, out_id, outer * inner, "softmax output", &o);
  if (rc) return rc;
  o->version++;
  if (outer * inner == 0) return TFJS_CUDA_OK;
  cudaSetDevice(ctx->device);
  const int row_blocks = (int)(outer < (int64_t)ctx->sm_count * 8 ? outer : (int64_t)ctx->sm_count * 8);
  if (inner >= 256 && inner <= 1024)
    launch_ex(ctx, softmax_last_block_kernel<4>, dim3(row_blocks), dim3(256), 0, (const float*)x->ptr,
              (float*)o->ptr, outer, (int)inner);
  else if (inner > 1024 && inner <= 2048)
    launch_ex(ctx, softmax_last_block_kernel<8>, dim3(row_blocks), dim3(256), 0, (const float*)x->ptr,
              (float*)o->ptr, outer, (int)inner);
  else
    softmax_last_kernel<<<grid_for(outer * 32, ctx->sm_count), kThreads, 0, ctx->stream>>>(
        (const float*)x->ptr, (float*)o->ptr, outer, inner);
  return post_launch(ctx, "softmax_last");
}
