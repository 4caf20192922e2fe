// CUDA-core convolution, depthwise convolution and pooling kernels (NHWC float32).
//
// These are the HBM-bound members of the path.  They follow the loop order of
// MathBackendCPU (tfjs-core/src/backends/cpu/backend_cpu.ts): taps are visited wR, wC, d1
// ascending, out-of-bounds taps are skipped, and every multiply-accumulate rounds once to
// float32 (fmaf), which reproduces `y[i] += x * w` on a Float32Array except for rare
// double-rounding cases.  The results are therefore (almost always) bit-identical to the
// reference's.
#include <cuda_fp16.h>

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

// Shared-memory float4 load the compiler may not hoist: the filter taps are re-read every
// step on purpose, keeping them out of the register file (36 registers) for occupancy.
__device__ __forceinline__ float4 lds128_volatile(const float4* p) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"((uint32_t)__cvta_generic_to_shared(p)));
  return v;
}

template <int ACT>
__device__ __forceinline__ float activate(float v, float lo, float hi) {
  if (ACT == TFJS_ACT_RELU) return max_nan(v, 0.f);              // Math.max(0, v): keeps NaN
  if (ACT == TFJS_ACT_CLIP) return min_nan(max_nan(v, lo), hi);  // v > hi ? hi : (v < lo ? lo : v)
  return v;
}

// Fast path: 3x3, dilation 1, channel multiplier 1, C % 4 == 0, stride 1 or 2 (every MobileNet
// depthwise layer).  A thread owns 4 channels of TW adjacent output columns and walks down a
// strip of output rows with the 3 x IN_W input window in registers.
//  - Input rows stream through a per-thread ring in shared memory filled with cp.async
//    (16-byte LDGSTS straight from L2, consecutive threads on consecutive channel quads), DEPTH-1
//    rows ahead of their use, so that the HBM latency is covered by several steps of arithmetic
//    without holding registers for data in flight.  Each thread reads back only what it copied
//    itself, so cp.async.wait_group is the only synchronisation.
//  - The three window rows live in three register banks whose roles (top / middle / bottom)
//    rotate from step to step, so nothing is shifted: the bank of the top row is refilled from
//    the ring as soon as its taps are issued.
//  - A block covers a slice of at most 128 channel quads (blockIdx.y) and stages only that
//    slice of the filter in shared memory; blocks are persistent (one wave).
// Taps outside the image are skipped, not multiplied by zero, as the reference skips them
// (backend_cpu.ts:2002-2014); accumulation order is wR, wC ascending with one float32 rounding
// per tap (fmaf), so results match the reference bit for bit up to double rounding.
template <int S, int TW, int ACT, int DEPTH>
struct DepthwiseStrip {
  static constexpr int IN_W = (TW - 1) * S + 3;
  float4 R[3][IN_W];   // window rows; which is top/middle/bottom rotates
  bool rk[3];          // row inside the image (border items only)
  bool ck[IN_W];       // column inside the image (border items only)
  float4 acc[TW];
  // ring state
  uint32_t ring;       // shared-memory address of this thread's slot 0, column 0
  int slot_in, slot_out;   // next ring slot to fill / to drain
  int rows_issued, rows_total, yi_issue;
  const float4* p_issue;   // global address of the next row to request (column xi0)

  static __device__ __forceinline__ uint32_t slot_addr(uint32_t ring, int slot, int i) {
    return ring + (uint32_t)((slot * IN_W + i) * 128 * 16);
  }

  // Requests the next input row (if any is left) and closes one cp.async group either way, so
  // that "DEPTH - 1 groups may be pending" always means "the row about to be drained is here".
  template <bool INTERIOR>
  __device__ __forceinline__ void issue(int64_t row_stride, int C4, int in_height) {
    if (rows_issued < rows_total) {
      const bool row_ok = INTERIOR || (yi_issue >= 0 && yi_issue < in_height);
      if (row_ok) {
#pragma unroll
        for (int i = 0; i < IN_W; i++)
          if (INTERIOR || ck[i])
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(slot_addr(ring, slot_in, i)),
                         "l"(p_issue + i * C4)
                         : "memory");
      }
      p_issue += row_stride;
      yi_issue++;
      rows_issued++;
      slot_in = (slot_in + 1 == DEPTH) ? 0 : slot_in + 1;
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  }

  // Moves the oldest ring row into register bank `bank`.
  template <bool INTERIOR>
  __device__ __forceinline__ void drain(int bank, int yi, int64_t row_stride, int C4, int in_height) {
    issue<INTERIOR>(row_stride, C4, in_height);
    asm volatile("cp.async.wait_group %0;" ::"n"(DEPTH - 1) : "memory");
    if (!INTERIOR) rk[bank] = (yi >= 0) && (yi < in_height);
#pragma unroll
    for (int i = 0; i < IN_W; i++) {
      float4 v;
      asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                   : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                   : "r"(slot_addr(ring, slot_out, i)));
      R[bank][i] = v;  // unspecified where the tap is outside the image; never used there
    }
    slot_out = (slot_out + 1 == DEPTH) ? 0 : slot_out + 1;
  }

  template <bool INTERIOR>
  __device__ __forceinline__ void taps(int slot, int wr, const float4* w_s, int cbn, int c_local) {
    if (!INTERIOR && !rk[slot]) return;  // the whole filter row lies outside: skipped
#pragma unroll
    for (int wc = 0; wc < 3; ++wc) {
      const float4 f = lds128_volatile(&w_s[(wr * 3 + wc) * cbn + c_local]);
#pragma unroll
      for (int j = 0; j < TW; j++) {
        if (INTERIOR || ck[j * S + wc]) {
          const float4 v = R[slot][j * S + wc];
          acc[j].x = fmaf(v.x, f.x, acc[j].x);
          acc[j].y = fmaf(v.y, f.y, acc[j].y);
          acc[j].z = fmaf(v.z, f.z, acc[j].z);
          acc[j].w = fmaf(v.w, f.w, acc[j].w);
        }
      }
    }
  }

  // One output row.  A = register bank holding the top row; yi = input row of the top row.
  template <int A, bool INTERIOR>
  __device__ __forceinline__ void step(int yi, bool more, int64_t row_stride, int in_height, int C4,
                                       const float4* w_s, int cbn, int c_local, float4* yrow,
                                       int cols_left, bool has_bias, const float4& bias4, float lo,
                                       float hi, bool round) {
    constexpr int B = (A + 1) % 3, C = (A + 2) % 3;
#pragma unroll
    for (int j = 0; j < TW; j++) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    taps<INTERIOR>(A, 0, w_s, cbn, c_local);
    // bank A is free: it receives the row that enters the window next (input row yi + 3)
    if (more) drain<INTERIOR>(A, yi + 3, row_stride, C4, in_height);
    taps<INTERIOR>(B, 1, w_s, cbn, c_local);
    if (S == 2 && more) drain<INTERIOR>(B, yi + 4, row_stride, C4, in_height);
    taps<INTERIOR>(C, 2, w_s, cbn, c_local);
#pragma unroll
    for (int j = 0; j < TW; j++) {
      if (j < cols_left) {
        float4 o = acc[j];
        if (has_bias) { o.x += bias4.x; o.y += bias4.y; o.z += bias4.z; o.w += bias4.w; }
        o.x = activate<ACT>(o.x, lo, hi);
        o.y = activate<ACT>(o.y, lo, hi);
        o.z = activate<ACT>(o.z, lo, hi);
        o.w = activate<ACT>(o.w, lo, hi);
        if (round) {  // the only reader is a TF32 contraction: round instead of letting it truncate
          o.x = round_tf32_after_arith(o.x); o.y = round_tf32_after_arith(o.y);
          o.z = round_tf32_after_arith(o.z); o.w = round_tf32_after_arith(o.w);
        }
        yrow[j * C4] = o;
      }
    }
  }

  template <bool INTERIOR>
  __device__ __forceinline__ void run(const float4* xb, float4* yb, int yo0, int yo1, int xo0, int xi0,
                                      const tfjs_conv2d_info& ci, int C4, const float4* w_s, int cbn,
                                      int c_local, bool has_bias, const float4& bias4, float lo,
                                      float hi, bool round) {
    const int64_t row_stride = (int64_t)ci.inWidth * C4;
    const int64_t out_stride = (int64_t)ci.outWidth * C4;
    const int in_height = ci.inHeight;
    if (!INTERIOR) {
#pragma unroll
      for (int i = 0; i < IN_W; i++) ck[i] = (xi0 + i >= 0) && (xi0 + i < ci.inWidth);
    }
    // (sic) rows use padLeft, as backend_cpu.ts:2000 does
    int yi = yo0 * S - ci.padLeft;
    float4* yrow = yb + (int64_t)yo0 * out_stride + (int64_t)xo0 * C4;
    const int cols_left = ci.outWidth - xo0;
    rows_total = (yo1 - yo0 - 1) * S + 3;
    rows_issued = 0;
    yi_issue = yi;
    p_issue = xb + (int64_t)yi * row_stride + (int64_t)xi0 * C4;
    slot_in = slot_out = 0;
#pragma unroll
    for (int d = 0; d < DEPTH - 1; d++) issue<INTERIOR>(row_stride, C4, in_height);
#pragma unroll
    for (int k = 0; k < 3; k++) drain<INTERIOR>(k, yi + k, row_stride, C4, in_height);
    int yo = yo0;
    // bank of the top row: 0, 1, 2, 0, ... for stride 1 and 0, 2, 1, 0, ... for stride 2
    while (true) {
      step<0, INTERIOR>(yi, yo + 1 < yo1, row_stride, in_height, C4, w_s, cbn, c_local, yrow, cols_left,
                        has_bias, bias4, lo, hi, round);
      if (++yo >= yo1) break;
      yi += S; yrow += out_stride;
      step<(S == 1 ? 1 : 2), INTERIOR>(yi, yo + 1 < yo1, row_stride, in_height, C4, w_s, cbn, c_local, yrow,
                                       cols_left, has_bias, bias4, lo, hi, round);
      if (++yo >= yo1) break;
      yi += S; yrow += out_stride;
      step<(S == 1 ? 2 : 1), INTERIOR>(yi, yo + 1 < yo1, row_stride, in_height, C4, w_s, cbn, c_local, yrow,
                                       cols_left, has_bias, bias4, lo, hi, round);
      if (++yo >= yo1) break;
      yi += S; yrow += out_stride;
    }
    // every requested row was drained; close the bookkeeping groups before the ring is reused
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  }
};

template <int S, int TW, int ACT, int MINB, int DEPTH>
__global__ void __launch_bounds__(128, MINB)
depthwise3x3_strip_kernel(const float* __restrict__ x, const float* __restrict__ w,
                          float* __restrict__ y, tfjs_conv2d_info ci, EpilogueArgs epi,
                          int rows_per_strip, int cb /* channel quads per block */) {
  constexpr int IN_W = (TW - 1) * S + 3;
  pdl_wait();
  pdl_launch_dependents();
  extern __shared__ float4 smem_dw[];
  float4* ring_s = smem_dw;                         // [DEPTH][IN_W][128 threads]
  float4* w_s = smem_dw + DEPTH * IN_W * 128;       // [9][quads of this slice]
  const int C4 = ci.inChannels >> 2;
  const int c4_base = blockIdx.y * cb;
  const int cbn = min(cb, C4 - c4_base);
  for (int i = threadIdx.x; i < 9 * cbn; i += blockDim.x)
    w_s[i] = reinterpret_cast<const float4*>(w)[(i / cbn) * C4 + c4_base + (i % cbn)];
  __syncthreads();
  const int groups = blockDim.x / cb;  // pixel groups per block
  const int c_local = threadIdx.x % cb;
  const int group = threadIdx.x / cb;
  if (group >= groups || c_local >= cbn) return;
  const int c4 = c4_base + c_local;
  const int strips = (ci.outHeight + rows_per_strip - 1) / rows_per_strip;
  const int w_tiles = (ci.outWidth + TW - 1) / TW;
  const int64_t items = (int64_t)ci.batchSize * strips * w_tiles;
  const bool has_bias = epi.bias != nullptr;
  float4 bias4 = make_float4(0.f, 0.f, 0.f, 0.f);
  if (has_bias) {
    if (epi.bias_scalar) {
      const float bv = __ldg(epi.bias);
      bias4 = make_float4(bv, bv, bv, bv);
    } else {
      bias4 = __ldg(reinterpret_cast<const float4*>(epi.bias) + c4);
    }
  }
  DepthwiseStrip<S, TW, ACT, DEPTH> ds;
  ds.ring = (uint32_t)__cvta_generic_to_shared(ring_s + threadIdx.x);
  for (int64_t item = (int64_t)blockIdx.x * groups + group; item < items;
       item += (int64_t)gridDim.x * groups) {
    const int wt = (int)(item % w_tiles);
    const int64_t rest = item / w_tiles;
    const int strip = (int)(rest % strips);
    const int b = (int)(rest / strips);
    const int yo0 = strip * rows_per_strip;
    const int yo1 = min(yo0 + rows_per_strip, ci.outHeight);
    const int xo0 = wt * TW;
    const int xi0 = xo0 * S - ci.padTop;  // (sic) columns use padTop, backend_cpu.ts:2010
    const float4* xb = reinterpret_cast<const float4*>(x) + (int64_t)b * ci.inHeight * ci.inWidth * C4 + c4;
    float4* yb = reinterpret_cast<float4*>(y) + (int64_t)b * ci.outHeight * ci.outWidth * C4 + c4;
    const int yi_first = yo0 * S - ci.padLeft;
    const int yi_last = (yo1 - 1) * S - ci.padLeft + 2;
    const bool interior = xi0 >= 0 && xi0 + IN_W <= ci.inWidth && yi_first >= 0 &&
                          yi_last < ci.inHeight && xo0 + TW <= ci.outWidth;
    if (interior)
      ds.template run<true>(xb, yb, yo0, yo1, xo0, xi0, ci, C4, w_s, cbn, c_local, has_bias, bias4,
                            epi.clip_lo, epi.clip_hi, epi.round_tf32 != 0);
    else
      ds.template run<false>(xb, yb, yo0, yo1, xo0, xi0, ci, C4, w_s, cbn, c_local, has_bias, bias4,
                             epi.clip_lo, epi.clip_hi, epi.round_tf32 != 0);
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

// The same pool for C % 4 == 0 and 16-byte aligned tensors: a thread owns 4 channels of one output
// pixel and reads its window with 128-bit loads; consecutive threads take consecutive channel
// quads, so a warp reads whole 512-byte runs of the NHWC image per tap.  Windows of neighbouring
// output pixels overlap (by (f - s) rows and columns); those re-reads are served by L1 / L2 (the
// loads go through the read-only path), DRAM sees every input line once.  Same arithmetic as
// above: float64 sum over the in-bounds taps in row-major order for avg, `p > cur` for max.
template <bool IS_AVG>
__global__ void __launch_bounds__(256)
pool2d_vec4_kernel(const float4* __restrict__ x, float4* __restrict__ y, tfjs_conv2d_info ci) {
  const int C4 = ci.inChannels >> 2;
  const int64_t total = (int64_t)ci.batchSize * ci.outHeight * ci.outWidth * C4;
  pdl_wait();
  pdl_launch_dependents();
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int d = (int)(t % C4);
    int64_t pix = t / C4;
    const int yc = (int)(pix % ci.outWidth);
    pix /= ci.outWidth;
    const int yr = (int)(pix % ci.outHeight);
    const int b = (int)(pix / ci.outHeight);
    const int xr_corner = yr * ci.strideHeight - ci.padTop;
    const int xc_corner = yc * ci.strideWidth - ci.padLeft;
    const int xr_min = max(0, xr_corner), xr_max = min(ci.inHeight, ci.effectiveFilterHeight + xr_corner);
    const int xc_min = max(0, xc_corner), xc_max = min(ci.inWidth, ci.effectiveFilterWidth + xc_corner);
    float4 mm = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
    double s0 = 0.0, s1 = 0.0, s2 = 0.0, s3 = 0.0;
    int count = 0;
    const float4* img = x + (int64_t)b * ci.inHeight * ci.inWidth * C4 + d;
    for (int xr = xr_min; xr < xr_max; xr += ci.dilationHeight) {
      const float4* row = img + (int64_t)xr * ci.inWidth * C4;
      for (int xc = xc_min; xc < xc_max; xc += ci.dilationWidth) {
        const float4 p = __ldg(row + (int64_t)xc * C4);
        if (IS_AVG) {
          s0 += (double)p.x; s1 += (double)p.y; s2 += (double)p.z; s3 += (double)p.w;
          count++;
        } else {
          if (p.x > mm.x) mm.x = p.x;
          if (p.y > mm.y) mm.y = p.y;
          if (p.z > mm.z) mm.z = p.z;
          if (p.w > mm.w) mm.w = p.w;
        }
      }
    }
    if (IS_AVG) {
      if ((count & (count - 1)) == 0) {
        // 1, 2, 4, 8 ... taps: the reciprocal is a power of two, so multiplying by it is the exact
        // float64 quotient the reference computes, without the long division sequence
        const double r = 1.0 / (double)count;
        mm = make_float4((float)(s0 * r), (float)(s1 * r), (float)(s2 * r), (float)(s3 * r));
      } else {
        const double n = (double)count;
        mm = make_float4((float)(s0 / n), (float)(s1 / n), (float)(s2 / n), (float)(s3 / n));
      }
    }
    y[t] = mm;
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

// Same pool for C % 4 == 0 and 16-byte aligned tensors: a thread owns 4 channels and keeps 7
// 16-byte loads in flight; each channel is still summed tap by tap in float64.
__global__ void global_avgpool_vec4_kernel(const float4* __restrict__ x, float4* __restrict__ y, int batch,
                                           int hw, int C4) {
  const int64_t total = (int64_t)batch * C4;
  pdl_wait();
  pdl_launch_dependents();
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int d = (int)(t % C4);
    const int b = (int)(t / C4);
    const float4* p = x + (int64_t)b * hw * C4 + d;
    double s0 = 0.0, s1 = 0.0, s2 = 0.0, s3 = 0.0;
    int i = 0;
    for (; i + 7 <= hw; i += 7) {
      float4 v[7];
#pragma unroll
      for (int j = 0; j < 7; j++) v[j] = __ldg(p + (int64_t)(i + j) * C4);
#pragma unroll
      for (int j = 0; j < 7; j++) {
        s0 += (double)v[j].x;
        s1 += (double)v[j].y;
        s2 += (double)v[j].z;
        s3 += (double)v[j].w;
      }
    }
    for (; i < hw; i++) {
      const float4 v = __ldg(p + (int64_t)i * C4);
      s0 += (double)v.x;
      s1 += (double)v.y;
      s2 += (double)v.z;
      s3 += (double)v.w;
    }
    const double n = (double)hw;
    y[t] = make_float4((float)(s0 / n), (float)(s1 / n), (float)(s2 / n), (float)(s3 / n));
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
                    (ci.strideHeight == 1 || ci.strideHeight == 2) && epi.activation != TFJS_ACT_PRELU &&
                    (((uintptr_t)x | (uintptr_t)w | (uintptr_t)y) & 15) == 0;
  if (fast && depthwise_image_supported(ci, epi.activation) && (epi.bias == nullptr || ((uintptr_t)epi.bias & 15) == 0))
    return launch_depthwise_image(ctx, x, w, y, ci, epi);
  if (fast) {
    const int C4 = ci.inChannels / 4;
    const int cb = C4 < 128 ? C4 : 128;                // channel quads per block
    const int slices = (C4 + cb - 1) / cb;
    const int groups = 128 / cb;                       // pixel groups per block
    constexpr int MINB = 4, DEPTH1 = 4, DEPTH2 = 6;    // blocks per SM; ring depth for stride 1 / 2
    const int tw = ci.strideHeight == 1 ? 2 : 1;
    const int in_w = (tw - 1) * ci.strideHeight + 3;
    const int depth = ci.strideHeight == 1 ? DEPTH1 : DEPTH2;
    const size_t smem = ((size_t)depth * in_w * 128 + (size_t)9 * cb) * sizeof(float4);
    const int64_t cols = (ci.outWidth + tw - 1) / tw;
    const int resident = ctx->sm_count * MINB;  // one wave of blocks
    // Strips of output rows.  A strip costs its rows plus a start-up of about three row steps
    // (ring fill, halo rows); the blocks of the one resident wave take ceil(items / capacity)
    // strips each.  Pick the strip height that minimises rounds x (rows + start-up): long strips
    // amortise the halo, short ones balance the wave on the small late layers.
    int rows = 8;
    {
      const int64_t capacity = (int64_t)resident * groups / slices > 0 ? (int64_t)resident * groups / slices : 1;
      int64_t best = -1;
      for (int r = 2; r <= ci.outHeight && r <= 32; ++r) {
        const int64_t strips_r = (ci.outHeight + r - 1) / r;
        const int64_t items_r = (int64_t)ci.batchSize * strips_r * cols;
        const int64_t rounds = (items_r + capacity - 1) / capacity;
        const int64_t cost = rounds * (r + 3);
        if (best < 0 || cost < best || (cost == best && r > rows)) {
          best = cost;
          rows = r;
        }
      }
      if (ci.outHeight < 2) rows = 1;
    }
    const int64_t items = (int64_t)ci.batchSize * ((ci.outHeight + rows - 1) / rows) * cols;
    int64_t gx = (items + groups - 1) / groups;
    if (gx > resident / slices) gx = resident / slices > 0 ? resident / slices : 1;
    dim3 grid((unsigned)gx, (unsigned)slices);
#define TFJS_LAUNCH_DW(ACT)                                                                           \
  do {                                                                                                \
    if (ci.strideHeight == 1) {                                                                       \
      auto k = depthwise3x3_strip_kernel<1, 2, ACT, MINB, DEPTH1>;                                     \
      cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                \
      launch_ex(ctx, k, grid, dim3(128), smem, x, w, y, ci, epi, rows, cb);                          \
    } else {                                                                                          \
      auto k = depthwise3x3_strip_kernel<2, 1, ACT, MINB, DEPTH2>;                                     \
      cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                \
      launch_ex(ctx, k, grid, dim3(128), smem, x, w, y, ci, epi, rows, cb);                          \
    }                                                                                                 \
  } while (0)
    switch (epi.activation) {
      case TFJS_ACT_RELU: TFJS_LAUNCH_DW(TFJS_ACT_RELU); break;
      case TFJS_ACT_CLIP: TFJS_LAUNCH_DW(TFJS_ACT_CLIP); break;
      default: TFJS_LAUNCH_DW(TFJS_ACT_LINEAR); break;
    }
#undef TFJS_LAUNCH_DW
    return post_launch(ctx, "depthwiseConv2D (3x3 strip)");
  }
  depthwise_generic_kernel<<<grid_1d(total, 256, ctx->sm_count, 8), 256, 0, ctx->stream>>>(x, w, y, ci, epi);
  return post_launch(ctx, "depthwiseConv2D (generic)");
}

// The same pool over an image stored as IEEE half: a thread owns 4 channels (8 bytes per tap),
// sums tap by tap in float64 in the reference's order, and writes float32.
__global__ void global_avgpool_half_kernel(const uint2* __restrict__ x, float4* __restrict__ y, int batch, int hw,
                                           int C4) {
  const int64_t total = (int64_t)batch * C4;
  pdl_wait();
  pdl_launch_dependents();
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int d = (int)(t % C4);
    const int b = (int)(t / C4);
    const uint2* p = x + (int64_t)b * hw * C4 + d;
    double s0 = 0.0, s1 = 0.0, s2 = 0.0, s3 = 0.0;
    for (int i = 0; i < hw; i++) {
      const uint2 h = __ldg(p + (int64_t)i * C4);
      const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&h.x));
      const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&h.y));
      s0 += (double)a.x; s1 += (double)a.y; s2 += (double)c.x; s3 += (double)c.y;
    }
    const double n = (double)hw;
    y[t] = make_float4((float)(s0 / n), (float)(s1 / n), (float)(s2 / n), (float)(s3 / n));
  }
}

// Global average pool through shared memory: a block stages the hw x 256-channel slab of one image
// with 16-byte asynchronous copies (every copy of the block in flight at once, which is what a
// small batch needs to cover the memory latency), then thread c sums channel c tap by tap in
// float64 in the reference's order, so the result is bit-identical to the kernels above.
constexpr int AVG_SLAB_CH = 256;
__global__ void __launch_bounds__(AVG_SLAB_CH) global_avgpool_slab_kernel(const float* __restrict__ x,
                                                                          float* __restrict__ y, int hw, int C) {
  extern __shared__ __align__(16) float slab[];
  const int chunks = (C + AVG_SLAB_CH - 1) / AVG_SLAB_CH;
  const int b = blockIdx.x / chunks;
  const int c0 = (blockIdx.x % chunks) * AVG_SLAB_CH;
  const int width = min(AVG_SLAB_CH, C - c0);  // multiple of 4
  const int quads = width / 4;
  const float* src = x + (int64_t)b * hw * C + c0;
  const uint32_t dst = (uint32_t)__cvta_generic_to_shared(slab);
  pdl_wait();
  pdl_launch_dependents();
  for (int i = threadIdx.x; i < hw * quads; i += AVG_SLAB_CH) {
    const int tap = i / quads, q = i % quads;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + (uint32_t)(tap * AVG_SLAB_CH + q * 4) * 4),
                 "l"(src + (int64_t)tap * C + q * 4)
                 : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();
  if ((int)threadIdx.x < width) {
    double s = 0.0;
    for (int i = 0; i < hw; i++) s += (double)slab[i * AVG_SLAB_CH + threadIdx.x];
    y[(int64_t)b * C + c0 + threadIdx.x] = (float)(s / (double)hw);
  }
}

bool global_avgpool_half_supported(const tfjs_conv2d_info& ci, int is_avg, const void* x, const void* y) {
  return is_avg && ci.outHeight == 1 && ci.outWidth == 1 && ci.padTop == 0 && ci.padLeft == 0 &&
         ci.dilationHeight == 1 && ci.dilationWidth == 1 && ci.filterHeight == ci.inHeight &&
         ci.filterWidth == ci.inWidth && ci.inChannels % 4 == 0 && ((uintptr_t)x & 7) == 0 && ((uintptr_t)y & 15) == 0;
}

int launch_global_avgpool_half(tfjs_cuda_ctx* ctx, const void* x, float* y, const tfjs_conv2d_info& ci) {
  const int64_t total = (int64_t)ci.batchSize * (ci.inChannels / 4);
  launch_ex(ctx, global_avgpool_half_kernel, dim3(grid_1d(total, 64, ctx->sm_count, 32)), dim3(64), 0,
            (const uint2*)x, (float4*)y, ci.batchSize, ci.inHeight * ci.inWidth, ci.inChannels / 4);
  return post_launch(ctx, "avgPool (global, float16 in)");
}

int launch_pool2d(tfjs_cuda_ctx* ctx, const float* x, float* y, const tfjs_conv2d_info& ci,
                  int is_avg) {
  const int64_t total = (int64_t)ci.batchSize * ci.outHeight * ci.outWidth * ci.inChannels;
  if (total == 0) return TFJS_CUDA_OK;
  const bool global = is_avg && ci.outHeight == 1 && ci.outWidth == 1 && ci.padTop == 0 &&
                      ci.padLeft == 0 && ci.dilationHeight == 1 && ci.dilationWidth == 1 &&
                      ci.filterHeight == ci.inHeight && ci.filterWidth == ci.inWidth;
  const int hw = ci.inHeight * ci.inWidth;
  if (global && ci.inChannels % 4 == 0 && ((uintptr_t)x & 15) == 0 && hw <= 56) {
    const int chunks = (ci.inChannels + AVG_SLAB_CH - 1) / AVG_SLAB_CH;
    const size_t smem = (size_t)hw * AVG_SLAB_CH * sizeof(float);
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(global_avgpool_slab_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_ex(ctx, global_avgpool_slab_kernel, dim3((unsigned)(ci.batchSize * chunks)), dim3(AVG_SLAB_CH), smem, x, y,
              hw, ci.inChannels);
    return post_launch(ctx, "avgPool (global)");
  }
  if (global && ci.inChannels % 4 == 0 && (((uintptr_t)x | (uintptr_t)y) & 15) == 0) {
    launch_ex(ctx, global_avgpool_vec4_kernel, dim3(grid_1d(total / 4, 64, ctx->sm_count, 32)), dim3(64), 0,
              (const float4*)x, (float4*)y, ci.batchSize, ci.inHeight * ci.inWidth, ci.inChannels / 4);
    return post_launch(ctx, "avgPool (global)");
  }
  if (global) {
    global_avgpool_kernel<<<grid_1d(total, 128, ctx->sm_count, 16), 128, 0, ctx->stream>>>(
        x, y, ci.batchSize, ci.inHeight * ci.inWidth, ci.inChannels);
    return post_launch(ctx, "avgPool (global)");
  }
  if (ci.inChannels % 4 == 0 && (((uintptr_t)x | (uintptr_t)y) & 15) == 0) {
    const dim3 grid(grid_1d(total / 4, 256, ctx->sm_count, 8));
    if (is_avg)
      launch_ex(ctx, pool2d_vec4_kernel<true>, grid, dim3(256), 0, (const float4*)x, (float4*)y, ci);
    else
      launch_ex(ctx, pool2d_vec4_kernel<false>, grid, dim3(256), 0, (const float4*)x, (float4*)y, ci);
    return post_launch(ctx, "pool2d (128-bit)");
  }
  pool2d_kernel<<<grid_1d(total, 256, ctx->sm_count, 8), 256, 0, ctx->stream>>>(x, y, ci, is_avg);
  return post_launch(ctx, "pool2d");
}
