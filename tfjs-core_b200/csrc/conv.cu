// CUDA-core convolution, depthwise convolution and pooling kernels (NHWC float32).
//
// These are the HBM-bound members of the path.  They follow the loop order of
// MathBackendCPU (tfjs-core/src/backends/cpu/backend_cpu.ts): taps are visited wR, wC, d1
// ascending, out-of-bounds taps are skipped, and every multiply-accumulate rounds once to
// float32 (fmaf), which reproduces `y[i] += x * w` on a Float32Array except for rare
// double-rounding cases.  The results are therefore (almost always) bit-identical to the
// reference's.
#include "common.cuh"

namespace {

// ---- generic direct conv2d (backend_cpu.ts:1552-1616) --------------------------------------
// One thread per (output pixel, block of CO_PER_THREAD output channels).  Used for every
// conv2d the tensor-core GEMM does not take: strided/dilated/odd shapes and Cin = 3.
template <int CO>
__global__ void conv2d_direct_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                     float* __restrict__ y, tfjs_conv2d_info ci, EpilogueArgs epi) {
  const int co_blocks = (ci.outChannels + CO - 1) / CO;
  const int64_t total = (int64_t)ci.batchSize * ci.outHeight * ci.outWidth * co_blocks;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int cb = (int)(t % co_blocks);
    int64_t pix = t / co_blocks;
    const int yc = (int)(pix % ci.outWidth);
    pix /= ci.outWidth;
    const int yr = (int)(pix % ci.outHeight);
    const int b = (int)(pix / ci.outHeight);
    const int co0 = cb * CO;
    float acc[CO];
#pragma unroll
    for (int j = 0; j < CO; j++) acc[j] = 0.f;
    const int xr_corner = yr * ci.strideHeight - ci.padTop;
    const int xc_corner = yc * ci.strideWidth - ci.padLeft;
    for (int wr = 0; wr < ci.filterHeight; ++wr) {
      const int xr = xr_corner + wr * ci.dilationHeight;
      if (xr < 0 || xr >= ci.inHeight) continue;
      for (int wc = 0; wc < ci.filterWidth; ++wc) {
        const int xc = xc_corner + wc * ci.dilationWidth;
        if (xc < 0 || xc >= ci.inWidth) continue;
        const float* xp = x + (((int64_t)b * ci.inHeight + xr) * ci.inWidth + xc) * ci.inChannels;
        const float* wp = w + ((int64_t)(wr * ci.filterWidth + wc) * ci.inChannels) * ci.outChannels + co0;
        for (int d1 = 0; d1 < ci.inChannels; ++d1) {
          const float xv = xp[d1];
#pragma unroll
          for (int j = 0; j < CO; j++)
            if (co0 + j < ci.outChannels) acc[j] = fmaf(xv, __ldg(wp + j), acc[j]);
          wp += ci.outChannels;
        }
      }
    }
    float* yp = y + (((int64_t)b * ci.outHeight + yr) * ci.outWidth + yc) * ci.outChannels + co0;
#pragma unroll
    for (int j = 0; j < CO; j++)
      if (co0 + j < ci.outChannels) yp[j] = apply_epilogue(acc[j], co0 + j, epi);
  }
}

// ---- stem conv: small Cin (<= 4), Cout = 32, any 3x3 geometry --------------------------------
// MobileNet's first layer (224x224x3 -> 112x112x32, stride 2) moves 141 MB per 64 images and
// has 27 MACs per output value: HBM-bound.  One thread produces all 32 channels of one output
// pixel, so a warp writes 4 KB contiguously; the 3x3xCinx32 filter sits in shared memory.
template <int CIN>
__global__ void __launch_bounds__(128)
conv2d_stem_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ y,
                   tfjs_conv2d_info ci, EpilogueArgs epi) {
  constexpr int CO = 32;
  __shared__ float ws[9 * CIN * CO];
  __shared__ float bs[CO];
  for (int i = threadIdx.x; i < 9 * CIN * CO; i += blockDim.x) ws[i] = w[i];
  if (threadIdx.x < CO)
    bs[threadIdx.x] = epi.bias ? (epi.bias_scalar ? epi.bias[0] : epi.bias[threadIdx.x]) : 0.f;
  __syncthreads();
  EpilogueArgs e2 = epi;
  e2.bias = nullptr;
  const int64_t total = (int64_t)ci.batchSize * ci.outHeight * ci.outWidth;
  for (int64_t pix = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; pix < total;
       pix += (int64_t)gridDim.x * blockDim.x) {
    const int yc = (int)(pix % ci.outWidth);
    const int yr = (int)((pix / ci.outWidth) % ci.outHeight);
    const int b = (int)(pix / ((int64_t)ci.outWidth * ci.outHeight));
    float acc[CO];
#pragma unroll
    for (int j = 0; j < CO; j++) acc[j] = 0.f;
    const int xr_corner = yr * ci.strideHeight - ci.padTop;
    const int xc_corner = yc * ci.strideWidth - ci.padLeft;
#pragma unroll
    for (int wr = 0; wr < 3; ++wr) {
      const int xr = xr_corner + wr * ci.dilationHeight;
      if (xr < 0 || xr >= ci.inHeight) continue;
#pragma unroll
      for (int wc = 0; wc < 3; ++wc) {
        const int xc = xc_corner + wc * ci.dilationWidth;
        if (xc < 0 || xc >= ci.inWidth) continue;
        const float* xp = x + (((int64_t)b * ci.inHeight + xr) * ci.inWidth + xc) * CIN;
#pragma unroll
        for (int d1 = 0; d1 < CIN; ++d1) {
          const float xv = __ldg(xp + d1);
          const float* wp = ws + ((wr * 3 + wc) * CIN + d1) * CO;
#pragma unroll
          for (int j = 0; j < CO; j++) acc[j] = fmaf(xv, wp[j], acc[j]);
        }
      }
    }
    float4* yp = reinterpret_cast<float4*>(y + pix * CO);
#pragma unroll
    for (int j = 0; j < CO; j += 4) {
      float4 o;
      o.x = apply_epilogue(epi.bias ? acc[j + 0] + bs[j + 0] : acc[j + 0], j + 0, e2);
      o.y = apply_epilogue(epi.bias ? acc[j + 1] + bs[j + 1] : acc[j + 1], j + 1, e2);
      o.z = apply_epilogue(epi.bias ? acc[j + 2] + bs[j + 2] : acc[j + 2], j + 2, e2);
      o.w = apply_epilogue(epi.bias ? acc[j + 3] + bs[j + 3] : acc[j + 3], j + 3, e2);
      yp[j / 4] = o;
    }
  }
}

// ---- depthwise conv2d (backend_cpu.ts:1979-2035) --------------------------------------------
// Generic kernel: any filter size, stride, dilation and channel multiplier; one thread per
// output value.  Note the reference's corner arithmetic: rows use padLeft and columns use
// padTop (backend_cpu.ts:2000, 2010); the two are equal for every SAME/VALID case with square
// geometry, and we reproduce the swap rather than "fix" it.
__global__ void depthwise_generic_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                         float* __restrict__ y, tfjs_conv2d_info ci,
                                         EpilogueArgs epi) {
  const int ch_mul = ci.outChannels / ci.inChannels;
  const int64_t total = (int64_t)ci.batchSize * ci.outHeight * ci.outWidth * ci.outChannels;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int oc = (int)(t % ci.outChannels);
    int64_t pix = t / ci.outChannels;
    const int yc = (int)(pix % ci.outWidth);
    pix /= ci.outWidth;
    const int yr = (int)(pix % ci.outHeight);
    const int b = (int)(pix / ci.outHeight);
    const int d1 = oc / ch_mul, q = oc % ch_mul;
    const int xr_corner = yr * ci.strideHeight - ci.padLeft;
    const int xc_corner = yc * ci.strideWidth - ci.padTop;
    float acc = 0.f;
    for (int wr = 0; wr < ci.filterHeight; ++wr) {
      const int xr = xr_corner + wr * ci.dilationHeight;
      if (xr < 0 || xr >= ci.inHeight) continue;
      for (int wc = 0; wc < ci.filterWidth; ++wc) {
        const int xc = xc_corner + wc * ci.dilationWidth;
        if (xc < 0 || xc >= ci.inWidth) continue;
        const float xv = x[(((int64_t)b * ci.inHeight + xr) * ci.inWidth + xc) * ci.inChannels + d1];
        const float wv = __ldg(w + ((int64_t)(wr * ci.filterWidth + wc) * ci.inChannels + d1) * ch_mul + q);
        acc = fmaf(xv, wv, acc);
      }
    }
    y[t] = apply_epilogue(acc, oc, epi);
  }
}

// Fast path: 3x3, dilation 1, channel multiplier 1, C % 4 == 0 (every MobileNet depthwise
// layer).  A thread owns 4 consecutive channels of TILE_W consecutive output columns of one
// output row: the 3 x (TILE_W*S + 2) input window is loaded once as float4 (128-bit NHWC
// loads, consecutive threads on consecutive channel quads => fully coalesced rows) and every
// loaded value feeds up to 3 outputs from registers, so each input row is fetched once per
// output row it contributes to (L2 absorbs the 3x / 1.5x vertical reuse).
template <int S, int TILE_W>
__global__ void __launch_bounds__(256)
depthwise3x3_kernel(const float* __restrict__ x, const float* __restrict__ w,
                    float* __restrict__ y, tfjs_conv2d_info ci, EpilogueArgs epi) {
  constexpr int IN_W = (TILE_W - 1) * S + 3;
  const int C4 = ci.inChannels >> 2;
  const int w_tiles = (ci.outWidth + TILE_W - 1) / TILE_W;
  const int64_t total = (int64_t)ci.batchSize * ci.outHeight * w_tiles * C4;
  const float4* x4 = reinterpret_cast<const float4*>(x);
  const float4* w4 = reinterpret_cast<const float4*>(w);
  float4* y4 = reinterpret_cast<float4*>(y);
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int c4 = (int)(t % C4);
    int64_t r = t / C4;
    const int wt = (int)(r % w_tiles);
    r /= w_tiles;
    const int yr = (int)(r % ci.outHeight);
    const int b = (int)(r / ci.outHeight);
    const int yc0 = wt * TILE_W;
    // (sic) rows use padLeft, columns use padTop, as the reference does.
    const int xr0 = yr * S - ci.padLeft;
    const int xc0 = yc0 * S - ci.padTop;
    float4 wv[9];
#pragma unroll
    for (int k = 0; k < 9; k++) wv[k] = __ldg(w4 + k * C4 + c4);
    float4 acc[TILE_W];
#pragma unroll
    for (int j = 0; j < TILE_W; j++) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int wr = 0; wr < 3; ++wr) {
      const int xr = xr0 + wr;
      if (xr < 0 || xr >= ci.inHeight) continue;
      const float4* row = x4 + ((int64_t)b * ci.inHeight + xr) * ci.inWidth * C4 + c4;
      float4 in[IN_W];
#pragma unroll
      for (int i = 0; i < IN_W; i++) {
        const int xc = xc0 + i;
        // NaN marks an out-of-bounds tap: it is skipped below, never multiplied.
        in[i] = (xc >= 0 && xc < ci.inWidth) ? row[(int64_t)xc * C4] : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int j = 0; j < TILE_W; j++) {
#pragma unroll
        for (int wc = 0; wc < 3; ++wc) {
          const int xc = xc0 + j * S + wc;
          if (xc < 0 || xc >= ci.inWidth) continue;  // skipped tap: no MAC, like the reference
          const float4 v = in[j * S + wc];
          const float4 f = wv[wr * 3 + wc];
          acc[j].x = fmaf(v.x, f.x, acc[j].x);
          acc[j].y = fmaf(v.y, f.y, acc[j].y);
          acc[j].z = fmaf(v.z, f.z, acc[j].z);
          acc[j].w = fmaf(v.w, f.w, acc[j].w);
        }
      }
    }
    float4* yrow = y4 + (((int64_t)b * ci.outHeight + yr) * ci.outWidth + yc0) * C4 + c4;
#pragma unroll
    for (int j = 0; j < TILE_W; j++) {
      if (yc0 + j >= ci.outWidth) break;
      float4 o;
      o.x = apply_epilogue(acc[j].x, c4 * 4 + 0, epi);
      o.y = apply_epilogue(acc[j].y, c4 * 4 + 1, epi);
      o.z = apply_epilogue(acc[j].z, c4 * 4 + 2, epi);
      o.w = apply_epilogue(acc[j].w, c4 * 4 + 3, epi);
      yrow[(int64_t)j * C4] = o;
    }
  }
}

// ---- pooling (backend_cpu.ts:2273-2341) ------------------------------------------------------
// One thread per output value, channel fastest (coalesced over C).  avg accumulates in
// float64 over the in-bounds taps and divides by their count; max starts at -inf and uses
// `pixel > cur`, so NaNs are ignored by max and propagated by avg, as in the reference.
__global__ void pool2d_kernel(const float* __restrict__ x, float* __restrict__ y,
                              tfjs_conv2d_info ci, int is_avg) {
  const int C = ci.inChannels;
  const int64_t total = (int64_t)ci.batchSize * ci.outHeight * ci.outWidth * C;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int d = (int)(t % C);
    int64_t pix = t / C;
    const int yc = (int)(pix % ci.outWidth);
    pix /= ci.outWidth;
    const int yr = (int)(pix % ci.outHeight);
    const int b = (int)(pix / ci.outHeight);
    const int xr_corner = yr * ci.strideHeight - ci.padTop;
    const int xc_corner = yc * ci.strideWidth - ci.padLeft;
    const int xr_min = max(0, xr_corner), xr_max = min(ci.inHeight, ci.effectiveFilterHeight + xr_corner);
    const int xc_min = max(0, xc_corner), xc_max = min(ci.inWidth, ci.effectiveFilterWidth + xc_corner);
    float mm = -INFINITY;
    double avg = 0.0;
    int count = 0;
    for (int xr = xr_min; xr < xr_max; xr += ci.dilationHeight)
      for (int xc = xc_min; xc < xc_max; xc += ci.dilationWidth) {
        const float p = x[(((int64_t)b * ci.inHeight + xr) * ci.inWidth + xc) * C + d];
        if (is_avg) {
          avg += (double)p;
          count++;
        } else if (p > mm) {
          mm = p;
        }
      }
    y[t] = is_avg ? (float)(avg / (double)count) : mm;
  }
}

// Global average pool (window = whole image, VALID, stride 1): MobileNet's 7x7x1024 -> 1024.
// One thread per (image, channel); taps are summed in the reference's order (row-major) in
// float64, so the result is bit-identical.  Reads are coalesced over channels.
__global__ void global_avgpool_kernel(const float* __restrict__ x, float* __restrict__ y, int batch,
                                      int hw, int C) {
  const int64_t total = (int64_t)batch * C;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int d = (int)(t % C);
    const int b = (int)(t / C);
    const float* p = x + (int64_t)b * hw * C + d;
    double s = 0.0;
    for (int i = 0; i < hw; i++) s += (double)p[(int64_t)i * C];
    y[t] = (float)(s / (double)hw);
  }
}

inline int grid_1d(int64_t work, int threads, int sm_count, int per_sm) {
  int64_t blocks = ceil_div64(work, threads);
  int64_t cap = (int64_t)sm_count * per_sm;
  if (blocks > cap) blocks = cap;
  return (int)(blocks < 1 ? 1 : blocks);
}

}  // namespace

int launch_conv2d_direct(tfjs_cuda_ctx* ctx, const float* x, const float* w, float* y,
                         const tfjs_conv2d_info& ci, const EpilogueArgs& epi) {
  const int64_t pixels = (int64_t)ci.batchSize * ci.outHeight * ci.outWidth;
  if (pixels * ci.outChannels == 0) return TFJS_CUDA_OK;
  const bool stem = ci.filterHeight == 3 && ci.filterWidth == 3 && ci.outChannels == 32 &&
                    (ci.inChannels == 3 || ci.inChannels == 4) && ((uintptr_t)y & 15) == 0;
  if (stem) {
    const int grid = grid_1d(pixels, 128, ctx->sm_count, 16);
    if (ci.inChannels == 3)
      conv2d_stem_kernel<3><<<grid, 128, 0, ctx->stream>>>(x, w, y, ci, epi);
    else
      conv2d_stem_kernel<4><<<grid, 128, 0, ctx->stream>>>(x, w, y, ci, epi);
    return post_launch(ctx, "conv2d (stem)");
  }
  if (ci.outChannels >= 8) {
    const int64_t work = pixels * ((ci.outChannels + 7) / 8);
    conv2d_direct_kernel<8><<<grid_1d(work, 128, ctx->sm_count, 16), 128, 0, ctx->stream>>>(x, w, y, ci, epi);
  } else {
    const int64_t work = pixels * ci.outChannels;
    conv2d_direct_kernel<1><<<grid_1d(work, 128, ctx->sm_count, 16), 128, 0, ctx->stream>>>(x, w, y, ci, epi);
  }
  return post_launch(ctx, "conv2d (direct)");
}

int launch_depthwise(tfjs_cuda_ctx* ctx, const float* x, const float* w, float* y,
                     const tfjs_conv2d_info& ci, const EpilogueArgs& epi) {
  const int64_t total = (int64_t)ci.batchSize * ci.outHeight * ci.outWidth * ci.outChannels;
  if (total == 0) return TFJS_CUDA_OK;
  const bool fast = ci.filterHeight == 3 && ci.filterWidth == 3 && ci.dilationHeight == 1 &&
                    ci.dilationWidth == 1 && ci.outChannels == ci.inChannels &&
                    ci.inChannels % 4 == 0 && ci.strideHeight == ci.strideWidth &&
                    (ci.strideHeight == 1 || ci.strideHeight == 2) &&
                    (((uintptr_t)x | (uintptr_t)w | (uintptr_t)y) & 15) == 0;
  if (fast) {
    constexpr int TILE_W = 4;
    const int64_t work = (int64_t)ci.batchSize * ci.outHeight * ((ci.outWidth + TILE_W - 1) / TILE_W) *
                         (ci.inChannels / 4);
    const int grid = grid_1d(work, 256, ctx->sm_count, 8);
    if (ci.strideHeight == 1)
      depthwise3x3_kernel<1, TILE_W><<<grid, 256, 0, ctx->stream>>>(x, w, y, ci, epi);
    else
      depthwise3x3_kernel<2, TILE_W><<<grid, 256, 0, ctx->stream>>>(x, w, y, ci, epi);
    return post_launch(ctx, "depthwiseConv2D (3x3)");
  }
  depthwise_generic_kernel<<<grid_1d(total, 256, ctx->sm_count, 8), 256, 0, ctx->stream>>>(x, w, y, ci, epi);
  return post_launch(ctx, "depthwiseConv2D (generic)");
}

int launch_pool2d(tfjs_cuda_ctx* ctx, const float* x, float* y, const tfjs_conv2d_info& ci,
                  int is_avg) {
  const int64_t total = (int64_t)ci.batchSize * ci.outHeight * ci.outWidth * ci.inChannels;
  if (total == 0) return TFJS_CUDA_OK;
  const bool global = is_avg && ci.outHeight == 1 && ci.outWidth == 1 && ci.padTop == 0 &&
                      ci.padLeft == 0 && ci.dilationHeight == 1 && ci.dilationWidth == 1 &&
                      ci.filterHeight == ci.inHeight && ci.filterWidth == ci.inWidth;
  if (global) {
    global_avgpool_kernel<<<grid_1d(total, 128, ctx->sm_count, 16), 128, 0, ctx->stream>>>(
        x, y, ci.batchSize, ci.inHeight * ci.inWidth, ci.inChannels);
    return post_launch(ctx, "avgPool (global)");
  }
  pool2d_kernel<<<grid_1d(total, 256, ctx->sm_count, 8), 256, 0, ctx->stream>>>(x, y, ci, is_avg);
  return post_launch(ctx, "pool2d");
}
