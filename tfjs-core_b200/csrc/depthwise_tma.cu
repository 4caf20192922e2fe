// depthwiseConv2D 3x3 for small images (MobileNet's 14x14 and 7x7 layers): the whole padded image
// of one channel group arrives in shared memory by ONE tiled TMA load, several images ahead.
//
// Reference semantics: MathBackendCPU.depthwiseConv2D (tfjs-core/src/backends/cpu/backend_cpu.ts:1979-2035):
// taps in the order (wR, wC) ascending, one float32 rounding per tap (fmaf), taps outside the image
// skipped.  The load zero-fills outside the image; rows outside are skipped (the branch is uniform
// over a warp) and columns outside get a zero filter tap, so that 0 * 0 is added and the
// accumulator is unchanged even for a non-finite filter value.
//
// Why a second depthwise kernel: the strip kernel walks down strips of rows with a per-thread
// cp.async ring; on a 14x14 image a strip's start-up (ring fill, halo rows) is a fifth of its
// work, and at small batches there are too few strips to hide it.  Here a CTA takes (image,
// channel group) items: the producer thread keeps NUM_STAGES - 1 whole windows in flight
// (64 KB each at 14x14 x 64 channels), which covers the DRAM latency with two or three requests,
// and the consumers never wait on anything but the stage barrier.
#include <cuda.h>

#include "common.cuh"
#include "tcgen05_ptx.cuh"

namespace {

constexpr int CONSUMERS = 256;
constexpr int THREADS = CONSUMERS + 32;  // + the producer warp
constexpr int MAX_STAGES = 8;  // half-precision windows are half as large: twice as many in flight
constexpr int HEADER_BYTES = 256;  // barriers + abort flag in front of the stages
constexpr int SMEM_BUDGET = 200 * 1024;

struct ImageParams {
  int B, C, CG;            // channels per item (multiple of 4)
  int inH, inW, outW;
  int pad;                 // first input row / column of output (0, 0) is -pad
  int boxH, boxW;          // window rows / columns in shared memory
  int stage_floats, num_stages, num_items, groups;  // groups = C / CG
  int stage_stride;        // bytes between stages: the window's bytes rounded up to 128 (TMA destination alignment)
  const float* filter;     // [3, 3, C, 1]
  const float* bias;
  int bias_scalar;
  float lo, hi;
  int round_tf32;          // round the results to tf32 (their only reader is a TF32 contraction)
  float* y;                // [B, outH, outW, C]
  int* status;
};

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1,
                                            int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ float4 lds128(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}
template <int ACT>
__device__ __forceinline__ float act(float v, float lo, float hi) {
  if (ACT == TFJS_ACT_RELU) return max_nan(v, 0.f);
  if (ACT == TFJS_ACT_CLIP) return min_nan(max_nan(v, lo), hi);
  return v;
}
__device__ __forceinline__ void fma4(float4& a, const float4& v, const float4& f) {
  a.x = fmaf(v.x, f.x, a.x);
  a.y = fmaf(v.y, f.y, a.y);
  a.z = fmaf(v.z, f.z, a.z);
  a.w = fmaf(v.w, f.w, a.w);
}

// Thread t of the consumers owns channel quad t % (CG / 4) of output column t / (CG / 4) and walks
// down the OUT_H output rows with the 3 x 3 window in registers: at stride 1 one new window row is
// read per output row, at stride 2 two (the loop is unrolled, so the rotation costs no moves).
// 16 bytes (float32) or 8 bytes (IEEE half) of a pixel: four channels as float32
template <bool HALF>
__device__ __forceinline__ float4 lds_quad(uint32_t addr) {
  if (!HALF) return lds128(addr);
  uint32_t a, b;
  asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(a), "=r"(b) : "r"(addr));
  float4 v;
  unpack_half2(a, v.x, v.y);
  unpack_half2(b, v.z, v.w);
  return v;
}

// HALF: input and output are stored as IEEE half (16-bit activation storage); the arithmetic is
// the same float32 fmaf chain on the exactly converted inputs, the result is rounded to half once.
template <int S, int OUT_H, int ACT, bool HALF>
__global__ void __launch_bounds__(THREADS, 1)
depthwise3x3_image_kernel(const __grid_constant__ CUtensorMap map_x, ImageParams p) {
  constexpr uint32_t ELEM = HALF ? 2 : 4;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);  // [MAX_STAGES] TMA -> consumers
  uint64_t* empty = full + MAX_STAGES;                 // [MAX_STAGES] consumers -> TMA
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + MAX_STAGES);
  const uint32_t stages = smem_u32(smem) + HEADER_BYTES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == CONSUMERS) prefetch_tensormap(&map_x);  // the producer's first lane

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.num_stages; s++) {
      mbar_init(smem_u32(&full[s]), 1);
      mbar_init(smem_u32(&empty[s]), CONSUMERS / 32);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  pdl_wait();
  pdl_launch_dependents();

  if (warp == CONSUMERS / 32) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int item = blockIdx.x; item < p.num_items; item += gridDim.x) {
        if (!mbar_wait(smem_u32(&empty[stage]), phase ^ 1, abort_flag, p.status, 21)) break;
        const int b = item / p.groups, g = item - b * p.groups;
        mbar_arrive_expect_tx(smem_u32(&full[stage]), (uint32_t)p.stage_floats * ELEM);
        tma_load_4d(stages + (uint32_t)stage * p.stage_stride, &map_x, smem_u32(&full[stage]), g * p.CG, -p.pad,
                    -p.pad, b);
        if (++stage == p.num_stages) { stage = 0; phase ^= 1; }
      }
    }
    return;
  }

  // ---------------- consumers ----------------
  const int nq = p.CG >> 2;
  const int q = threadIdx.x % nq;
  const int col = threadIdx.x / nq;
  const bool active = col < p.outW;
  const uint32_t pixel_bytes = (uint32_t)p.CG * ELEM;
  const uint32_t row_bytes = (uint32_t)p.boxW * pixel_bytes;
  // which filter columns fall inside the image for this thread's output column
  bool ck[3];
#pragma unroll
  for (int wc = 0; wc < 3; wc++) {
    const int xi = col * S - p.pad + wc;
    ck[wc] = xi >= 0 && xi < p.inW;
  }
  int stage = 0;
  uint32_t phase = 0;
  bool ok = true;
  for (int item = blockIdx.x; item < p.num_items && ok; item += gridDim.x) {
    const int b = item / p.groups, g = item - b * p.groups;
    const int ch = g * p.CG + q * 4;
    // (fetching the next item's taps during this item's arithmetic measured no faster)
    float4 f[3][3];
    float4 bias4 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (active) {
#pragma unroll
      for (int k = 0; k < 9; k++) {
        const float4 w = __ldg(reinterpret_cast<const float4*>(p.filter + (size_t)k * p.C + ch));
        f[k / 3][k % 3] = ck[k % 3] ? w : make_float4(0.f, 0.f, 0.f, 0.f);
      }
      if (p.bias)
        bias4 = p.bias_scalar ? make_float4(__ldg(p.bias), __ldg(p.bias), __ldg(p.bias), __ldg(p.bias))
                              : __ldg(reinterpret_cast<const float4*>(p.bias + ch));
    }
    ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&full[stage]), phase, abort_flag, p.status, 22));
    if (!ok) break;
    if (active) {
      const uint32_t base = stages + (uint32_t)stage * p.stage_stride + (uint32_t)(col * S) * pixel_bytes + q * 4 * ELEM;
      const size_t y_first = ((size_t)b * OUT_H * p.outW + col) * p.C + ch;
      float4* yp = reinterpret_cast<float4*>(p.y + (HALF ? 0 : y_first));
      uint2* yp16 = reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(p.y) + (HALF ? y_first : 0));
      const size_t y_row = (size_t)p.outW * p.C / 4;
      float4 R[3][3];  // window rows; the unrolled loop renames them instead of moving
#pragma unroll
      for (int r = 0; r < 3 - S; r++)
#pragma unroll
        for (int wc = 0; wc < 3; wc++) R[r + S][wc] = lds_quad<HALF>(base + r * row_bytes + wc * pixel_bytes);
#pragma unroll
      for (int yo = 0; yo < OUT_H; yo++) {
        // rows move up by S; the S new rows come from shared memory
#pragma unroll
        for (int r = 0; r < 3 - S; r++)
#pragma unroll
          for (int wc = 0; wc < 3; wc++) R[r][wc] = R[r + S][wc];
#pragma unroll
        for (int r = 3 - S; r < 3; r++)
#pragma unroll
          for (int wc = 0; wc < 3; wc++) R[r][wc] = lds_quad<HALF>(base + (yo * S + r) * row_bytes + wc * pixel_bytes);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int dr = 0; dr < 3; dr++) {
          const int yi = yo * S - p.pad + dr;
          if (yi < 0 || yi >= p.inH) continue;  // the reference skips taps outside the image
#pragma unroll
          for (int wc = 0; wc < 3; wc++) fma4(acc, R[dr][wc], f[dr][wc]);
        }
        if (p.bias) { acc.x += bias4.x; acc.y += bias4.y; acc.z += bias4.z; acc.w += bias4.w; }
        acc.x = act<ACT>(acc.x, p.lo, p.hi);
        acc.y = act<ACT>(acc.y, p.lo, p.hi);
        acc.z = act<ACT>(acc.z, p.lo, p.hi);
        acc.w = act<ACT>(acc.w, p.lo, p.hi);
        if (p.round_tf32) {
          // (the integer form: cvt.rna.tf32 runs at a fraction of the ALU rate and cost 10 % of this kernel)
          acc.x = round_tf32_after_arith(acc.x); acc.y = round_tf32_after_arith(acc.y);
          acc.z = round_tf32_after_arith(acc.z); acc.w = round_tf32_after_arith(acc.w);
        }
        if (HALF)
          yp16[yo * y_row] = make_uint2(pack_half2(acc.x, acc.y), pack_half2(acc.z, acc.w));
        else
          yp[yo * y_row] = acc;
      }
    }
    __syncwarp();  // every lane has read all it needs of the window
    if (lane == 0) mbar_arrive(smem_u32(&empty[stage]));
    if (++stage == p.num_stages) { stage = 0; phase ^= 1; }
  }
}

template <int S, int OUT_H, bool HALF>
int launch_act(tfjs_cuda_ctx* ctx, const CUtensorMap& mx, const ImageParams& p, int activation, int grid,
               size_t smem) {
#define TFJS_LAUNCH_IMG(ACT)                                                                  \
  do {                                                                                        \
    auto k = depthwise3x3_image_kernel<S, OUT_H, ACT, HALF>;                                  \
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);          \
    launch_ex(ctx, k, dim3((unsigned)grid), dim3(THREADS), smem, mx, p);                      \
  } while (0)
  switch (activation) {
    case TFJS_ACT_RELU: TFJS_LAUNCH_IMG(TFJS_ACT_RELU); break;
    case TFJS_ACT_CLIP: TFJS_LAUNCH_IMG(TFJS_ACT_CLIP); break;
    default: TFJS_LAUNCH_IMG(TFJS_ACT_LINEAR); break;
  }
#undef TFJS_LAUNCH_IMG
  return post_launch(ctx, HALF ? "depthwiseConv2D (3x3 image window, TMA, float16)"
                               : "depthwiseConv2D (3x3 image window, TMA)");
}

// channels per item: the widest group that fills the consumer threads without exceeding them and
// leaves room for two windows in shared memory
int pick_group(const tfjs_conv2d_info& ci, bool half) {
  const int box = (ci.outHeight - 1) * ci.strideHeight + 3;
  for (int cg = 128; cg >= 32; cg /= 2)
    if (ci.inChannels % cg == 0 && ci.outWidth * (cg / 4) <= CONSUMERS &&
        (size_t)2 * box * box * cg * (half ? 2 : 4) <= SMEM_BUDGET)
      return cg;
  return 0;
}

}  // namespace

int set_wait_limit_depthwise_image(long long cycles) { return set_wait_limit_here(cycles); }

bool depthwise_image_supported(const tfjs_conv2d_info& ci, int activation, bool half) {
  const int S = ci.strideHeight;
  if (!(ci.filterHeight == 3 && ci.filterWidth == 3 && ci.dilationHeight == 1 && ci.dilationWidth == 1 &&
        ci.outChannels == ci.inChannels && ci.strideHeight == ci.strideWidth && (S == 1 || S == 2) &&
        activation != TFJS_ACT_PRELU && ci.padTop == ci.padLeft && ci.outHeight == ci.outWidth &&
        ci.batchSize >= 1 && ci.batchSize < 65536))
    return false;
  // half storage halves the window bytes, which lets the 28x28 -> 14x14 stride-2 layer in as well
  if (!((S == 1 && (ci.outHeight == 14 || ci.outHeight == 7)) || (S == 2 && ci.outHeight == 7) ||
        (half && S == 2 && ci.outHeight == 14)))
    return false;
  return pick_group(ci, half) != 0 && tcgen05_gemm_supported(128, 32, 32);  // (the driver's tensor-map encoder is there)
}

int launch_depthwise_image(tfjs_cuda_ctx* ctx, const void* x, const float* w, void* y, const tfjs_conv2d_info& ci,
                           const EpilogueArgs& epi, bool half) {
  const int S = ci.strideHeight;
  const size_t elem = half ? 2 : 4;
  ImageParams p;
  p.B = ci.batchSize;
  p.C = ci.inChannels;
  p.CG = pick_group(ci, half);
  p.inH = ci.inHeight;
  p.inW = ci.inWidth;
  p.outW = ci.outWidth;
  p.pad = ci.padTop;
  p.boxH = p.boxW = (ci.outHeight - 1) * S + 3;
  p.stage_floats = p.boxH * p.boxW * p.CG;
  p.stage_stride = (int)(((size_t)p.stage_floats * elem + 127) / 128 * 128);
  const int fit = (int)(SMEM_BUDGET / (size_t)p.stage_stride);
  p.num_stages = fit > MAX_STAGES ? MAX_STAGES : fit;
  p.groups = p.C / p.CG;
  p.num_items = p.B * p.groups;
  p.filter = w;
  p.bias = epi.bias;
  p.bias_scalar = epi.bias_scalar;
  p.lo = epi.clip_lo;
  p.hi = epi.clip_hi;
  p.round_tf32 = epi.round_tf32;
  p.y = (float*)y;
  p.status = ctx->d_status;
  CUtensorMap mx;
  const uint64_t xd[4] = {(uint64_t)p.C, (uint64_t)ci.inWidth, (uint64_t)ci.inHeight, (uint64_t)ci.batchSize};
  const uint64_t xs[3] = {(uint64_t)p.C * elem, (uint64_t)ci.inWidth * p.C * elem,
                          (uint64_t)ci.inHeight * ci.inWidth * p.C * elem};
  const uint32_t xb[4] = {(uint32_t)p.CG, (uint32_t)p.boxW, (uint32_t)p.boxH, 1};
  if (!tma_encode_tiled(&mx, half ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, x, xd, xs, xb,
                        CU_TENSOR_MAP_SWIZZLE_NONE))
    return set_error(ctx, TFJS_CUDA_ERR_CUDA, "cuTensorMapEncodeTiled failed");
  const int grid = p.num_items < ctx->sm_count ? p.num_items : ctx->sm_count;
  const size_t smem = 128 + HEADER_BYTES + (size_t)p.num_stages * p.stage_stride;
  if (half) {
    if (S == 1 && ci.outHeight == 14) return launch_act<1, 14, true>(ctx, mx, p, epi.activation, grid, smem);
    if (S == 1) return launch_act<1, 7, true>(ctx, mx, p, epi.activation, grid, smem);
    if (ci.outHeight == 14) return launch_act<2, 14, true>(ctx, mx, p, epi.activation, grid, smem);
    return launch_act<2, 7, true>(ctx, mx, p, epi.activation, grid, smem);
  }
  if (S == 1 && ci.outHeight == 14) return launch_act<1, 14, false>(ctx, mx, p, epi.activation, grid, smem);
  if (S == 1) return launch_act<1, 7, false>(ctx, mx, p, epi.activation, grid, smem);
  return launch_act<2, 7, false>(ctx, mx, p, epi.activation, grid, smem);
}

