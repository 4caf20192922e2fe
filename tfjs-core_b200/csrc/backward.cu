// Gradient kernels of the convolution and pooling ops, so that the engine's tape can
// differentiate the networks this backend runs: KernelBackend.conv2dDerInput / conv2dDerFilter
// (tfjs-core/src/backends/backend.ts:424-429; CPU backend_cpu.ts:1686-1762, 1849-1898),
// depthwiseConv2DDerInput / DerFilter (backend.ts:436-442; CPU :2037-2150), maxPoolBackprop /
// avgPoolBackprop (backend.ts:456-466; CPU :2347-2509) and transpose (backend.ts:216).
//
// These are written for exactness first: every output element is produced by one thread that
// walks the reference's loop nest in the reference's order with a float64 accumulator, so the
// results are bit-identical to MathBackendCPU.  Threads are laid out so that the inner-most
// (channel) index is the fastest-varying one across a warp, which keeps the reads coalesced.
#include "common.cuh"

namespace {

__device__ __forceinline__ int ceil_div_i(int a, int s) {
  // Math.ceil(a / s) for s > 0 and any sign of a
  return a >= 0 ? (a + s - 1) / s : -((-a) / s);
}
// `for (y = lo; y < Math.min(limit, num / s); ++y)` with num / s a real number
__device__ __forceinline__ int upper_bound_i(int limit, int num, int s) {
  const int top = ceil_div_i(num, s);
  return top < limit ? top : limit;
}

// dx[b, xr, xc, d1] = sum over (yr, yc, d2) of dy[b, yr, yc, d2] * w[fh-1-wr, fw-1-wc, d1, d2]
template <bool DEPTHWISE>
__global__ void conv_der_input_kernel(const float* __restrict__ dy, const float* __restrict__ w,
                                      float* __restrict__ dx, tfjs_conv2d_info c) {
  const int fh = c.filterHeight, fw = c.filterWidth, sh = c.strideHeight, sw = c.strideWidth;
  const int top_pad = fh - 1 - c.padTop, left_pad = fw - 1 - c.padLeft;
  const int ch_mul = DEPTHWISE ? c.outChannels / c.inChannels : 1;
  const int64_t w_s2 = DEPTHWISE ? ch_mul : c.outChannels;
  const int64_t w_s1 = (int64_t)c.inChannels * w_s2, w_s0 = (int64_t)fw * w_s1;
  const int64_t total = (int64_t)c.batchSize * c.inHeight * c.inWidth * c.inChannels;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int d1 = (int)(t % c.inChannels);
    int64_t r = t / c.inChannels;
    const int xc = (int)(r % c.inWidth);
    r /= c.inWidth;
    const int xr = (int)(r % c.inHeight);
    const int b = (int)(r / c.inHeight);
    const int xr_corner = xr - top_pad, xc_corner = xc - left_pad;
    const int yr_min = max(0, ceil_div_i(xr_corner, sh)), yr_max = upper_bound_i(c.outHeight, fh + xr_corner, sh);
    const int yc_min = max(0, ceil_div_i(xc_corner, sw)), yc_max = upper_bound_i(c.outWidth, fw + xc_corner, sw);
    double dot = 0.0;
    for (int yr = yr_min; yr < yr_max; ++yr) {
      const int wr = yr * sh - xr_corner;
      for (int yc = yc_min; yc < yc_max; ++yc) {
        const int wc = yc * sw - xc_corner;
        const float* dyp = dy + (((int64_t)b * c.outHeight + yr) * c.outWidth + yc) * c.outChannels;
        const float* wp = w + w_s0 * (fh - 1 - wr) + w_s1 * (fw - 1 - wc) + w_s2 * d1;
        if (DEPTHWISE) {
          for (int dm = 0; dm < ch_mul; ++dm) dot += (double)dyp[d1 * ch_mul + dm] * (double)wp[dm];
        } else {
          for (int d2 = 0; d2 < c.outChannels; ++d2) dot += (double)dyp[d2] * (double)wp[d2];
        }
      }
    }
    dx[t] = (float)dot;
  }
}

// dW[wr, wc, d1, d2] = sum over (b, yr, yc) of x[b, xr, xc, d1] * dy[b, yr, yc, d2].
// grid.y enumerates (wr, wc, d1) (depthwise: (wr, wc)); threads run over d2.
template <bool DEPTHWISE>
__global__ void conv_der_filter_kernel(const float* __restrict__ x, const float* __restrict__ dy,
                                       float* __restrict__ dw, tfjs_conv2d_info c) {
  const int sh = c.strideHeight, sw = c.strideWidth;
  const int ch_mul = DEPTHWISE ? c.outChannels / c.inChannels : 1;
  int64_t row = blockIdx.y;
  int d1_fixed = 0;
  if (!DEPTHWISE) {
    d1_fixed = (int)(row % c.inChannels);
    row /= c.inChannels;
  }
  const int wc = (int)(row % c.filterWidth);
  const int wr = (int)(row / c.filterWidth);
  const int yr_min = max(0, ceil_div_i(c.padTop - wr, sh));
  const int yr_max = upper_bound_i(c.outHeight, c.inHeight + c.padTop - wr, sh);
  const int yc_min = max(0, ceil_div_i(c.padLeft - wc, sw));
  const int yc_max = upper_bound_i(c.outWidth, c.inWidth + c.padLeft - wc, sw);
  for (int d2 = blockIdx.x * blockDim.x + threadIdx.x; d2 < c.outChannels; d2 += gridDim.x * blockDim.x) {
    const int d1 = DEPTHWISE ? d2 / ch_mul : d1_fixed;
    double dot = 0.0;
    for (int b = 0; b < c.batchSize; ++b)
      for (int yr = yr_min; yr < yr_max; ++yr) {
        const int xr = wr + yr * sh - c.padTop;
        for (int yc = yc_min; yc < yc_max; ++yc) {
          const int xc = wc + yc * sw - c.padLeft;
          dot += (double)x[(((int64_t)b * c.inHeight + xr) * c.inWidth + xc) * c.inChannels + d1] *
                 (double)dy[(((int64_t)b * c.outHeight + yr) * c.outWidth + yc) * c.outChannels + d2];
        }
      }
    if (DEPTHWISE)
      dw[(((int64_t)wr * c.filterWidth + wc) * c.inChannels + d1) * ch_mul + d2 % ch_mul] = (float)dot;
    else
      dw[(((int64_t)wr * c.filterWidth + wc) * c.inChannels + d1) * c.outChannels + d2] = (float)dot;
  }
}

// maxPoolPositions (backend_cpu.ts:2347-2398): flat index of the first strictly greatest tap in the
// effective window, -1 if no tap compares greater than -Infinity.
__global__ void max_pool_positions_kernel(const float* __restrict__ x, int32_t* __restrict__ pos,
                                          tfjs_conv2d_info c) {
  const int C = c.inChannels;
  const int64_t total = (int64_t)c.batchSize * c.outHeight * c.outWidth * C;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int d = (int)(t % C);
    int64_t r = t / C;
    const int yc = (int)(r % c.outWidth);
    r /= c.outWidth;
    const int yr = (int)(r % c.outHeight);
    const int b = (int)(r / c.outHeight);
    const int xr_corner = yr * c.strideHeight - c.padTop, xc_corner = yc * c.strideWidth - c.padLeft;
    int xr_min = xr_corner, xc_min = xc_corner;
    while (xr_min < 0) xr_min += c.dilationHeight;
    while (xc_min < 0) xc_min += c.dilationWidth;
    const int xr_max = min(c.inHeight, c.effectiveFilterHeight + xr_corner);
    const int xc_max = min(c.inWidth, c.effectiveFilterWidth + xc_corner);
    float max_value = -INFINITY;
    int max_pos = -1;
    for (int xr = xr_min; xr < xr_max; xr += c.dilationHeight)
      for (int xc = xc_min; xc < xc_max; xc += c.dilationWidth) {
        const float pixel = x[(((int64_t)b * c.inHeight + xr) * c.inWidth + xc) * C + d];
        if (pixel > max_value) {
          max_value = pixel;
          max_pos = (xr - xr_corner) * c.effectiveFilterWidth + (xc - xc_corner);
        }
      }
    pos[t] = max_pos;
  }
}

// maxPoolBackprop / avgPoolBackprop (backend_cpu.ts:2400-2509)
template <bool AVG>
__global__ void pool_backprop_kernel(const float* __restrict__ dy, const int32_t* __restrict__ pos,
                                     float* __restrict__ dx, tfjs_conv2d_info c) {
  const int C = c.inChannels;
  const int efh = c.effectiveFilterHeight, efw = c.effectiveFilterWidth;
  const int pad_left = efw - 1 - c.padLeft, pad_top = efh - 1 - c.padTop;
  const double avg_multiplier = 1.0 / (double)(c.filterHeight * c.filterWidth);
  const int64_t total = (int64_t)c.batchSize * c.inHeight * c.inWidth * C;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int d = (int)(t % C);
    int64_t r = t / C;
    const int dxc = (int)(r % c.inWidth);
    r /= c.inWidth;
    const int dxr = (int)(r % c.inHeight);
    const int b = (int)(r / c.inHeight);
    const int dyr_corner = dxr - pad_top, dyc_corner = dxc - pad_left;
    double dot = 0.0;
    for (int wr = 0; wr < efh; wr += c.dilationHeight) {
      const int num_r = dyr_corner + wr;
      if (num_r < 0 || num_r % c.strideHeight != 0) continue;
      const int dyr = num_r / c.strideHeight;
      if (dyr >= c.outHeight) continue;
      for (int wc = 0; wc < efw; wc += c.dilationWidth) {
        const int num_c = dyc_corner + wc;
        if (num_c < 0 || num_c % c.strideWidth != 0) continue;
        const int dyc = num_c / c.strideWidth;
        if (dyc >= c.outWidth) continue;
        const int64_t yi = (((int64_t)b * c.outHeight + dyr) * c.outWidth + dyc) * C + d;
        if (AVG) {
          dot += (double)dy[yi];
        } else if (efh * efw - 1 - pos[yi] == wr * efw + wc) {
          dot += (double)dy[yi];
        }
      }
    }
    dx[t] = (float)(AVG ? dot * avg_multiplier : dot);
  }
}

// Gradient of clipByValue (ops/unary_ops.ts:456-462): dy where min <= x <= max, else 0.  One
// kernel for the reference's greaterEqual / lessEqual / logicalAnd / where chain.
__global__ void clip_backprop_kernel(const float* __restrict__ dy, const float* __restrict__ x,
                                     float* __restrict__ out, int64_t n, float lo, float hi) {
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < n; t += (int64_t)gridDim.x * blockDim.x)
    out[t] = (x[t] >= lo && x[t] <= hi) ? dy[t] : 0.f;
}

struct TransposeDesc {
  int rank;
  int64_t out_shape[8];
  int64_t in_stride[8];  // stride in x of the axis that becomes output axis i
};

// out[i0, .., i(r-1)] = x at the permuted position (backend_cpu.ts transpose)
__global__ void transpose_kernel(const float* __restrict__ x, float* __restrict__ out, TransposeDesc d,
                                 int64_t n) {
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < n; t += (int64_t)gridDim.x * blockDim.x) {
    int64_t rem = t, src = 0;
    for (int i = d.rank - 1; i >= 0; --i) {
      src += (rem % d.out_shape[i]) * d.in_stride[i];
      rem /= d.out_shape[i];
    }
    out[t] = x[src];
  }
}

inline int grid_for_elems(int64_t n, int threads, int sm_count) {
  int64_t blocks = (n + threads - 1) / threads;
  const int64_t cap = (int64_t)sm_count * 16;
  if (blocks > cap) blocks = cap;
  return (int)(blocks < 1 ? 1 : blocks);
}

int check_info(tfjs_cuda_ctx* ctx, const tfjs_conv2d_info* ci) {
  TFJS_REQUIRE(ctx, ci != nullptr, "convInfo is null");
  TFJS_REQUIRE(ctx, ci->batchSize >= 0 && ci->inHeight >= 0 && ci->inWidth >= 0 && ci->inChannels >= 0 &&
                        ci->outHeight >= 0 && ci->outWidth >= 0 && ci->outChannels >= 0,
               "negative extent in convInfo");
  TFJS_REQUIRE(ctx, ci->strideHeight >= 1 && ci->strideWidth >= 1 && ci->dilationHeight >= 1 &&
                        ci->dilationWidth >= 1 && ci->filterHeight >= 1 && ci->filterWidth >= 1,
               "strides, dilations and filter sizes must be positive");
  return TFJS_CUDA_OK;
}

// x [B, inH, inW, Cin], dy [B, outH, outW, Cout], filter [fH, fW, Cin, Cout or chMul]
int conv_gradient(tfjs_cuda_ctx* ctx, tfjs_tensor_id first_id, tfjs_tensor_id second_id, tfjs_tensor_id out_id,
                  const tfjs_conv2d_info* ci, bool depthwise, bool wrt_input) {
  if (!ctx) return TFJS_CUDA_ERR_INVALID_ARG;
  int rc = check_info(ctx, ci);
  if (rc) return rc;
  TFJS_REQUIRE(ctx, ci->dilationHeight == 1 && ci->dilationWidth == 1,
               "the gradient kernels of the reference do not handle dilation (ops/conv.ts:188-192)");
  TFJS_REQUIRE(ctx, !depthwise || (ci->inChannels > 0 && ci->outChannels % ci->inChannels == 0),
               "depthwise outChannels must be a multiple of inChannels");
  const int64_t x_n = (int64_t)ci->batchSize * ci->inHeight * ci->inWidth * ci->inChannels;
  const int64_t y_n = (int64_t)ci->batchSize * ci->outHeight * ci->outWidth * ci->outChannels;
  const int64_t w_n = (int64_t)ci->filterHeight * ci->filterWidth *
                      (depthwise ? ci->outChannels : (int64_t)ci->inChannels * ci->outChannels);
  TensorEntry *a, *b, *o;
  rc = get_f32(ctx, first_id, wrt_input ? y_n : x_n, wrt_input ? "dy" : "x", &a);
  if (rc) return rc;
  rc = get_f32(ctx, second_id, wrt_input ? w_n : y_n, wrt_input ? "filter" : "dy", &b);
  if (rc) return rc;
  rc = get_f32(ctx, out_id, wrt_input ? x_n : w_n, "gradient output", &o);
  if (rc) return rc;
  TFJS_REQUIRE(ctx, !a->quant.quantized && !b->quant.quantized && !o->quant.quantized,
               "gradient kernels take float32 tensors");
  o->version++;
  if ((wrt_input ? x_n : w_n) == 0) return TFJS_CUDA_OK;
  cudaSetDevice(ctx->device);
  const float *pa = (const float*)a->ptr, *pb = (const float*)b->ptr;
  float* po = (float*)o->ptr;
  if (wrt_input) {
    const int grid = grid_for_elems(x_n, 128, ctx->sm_count);
    if (depthwise)
      conv_der_input_kernel<true><<<grid, 128, 0, ctx->stream>>>(pa, pb, po, *ci);
    else
      conv_der_input_kernel<false><<<grid, 128, 0, ctx->stream>>>(pa, pb, po, *ci);
    return post_launch(ctx, depthwise ? "depthwiseConv2DDerInput" : "conv2dDerInput");
  }
  const int threads = ci->outChannels >= 128 ? 128 : 32;
  dim3 grid((unsigned)((ci->outChannels + threads - 1) / threads),
            (unsigned)(ci->filterHeight * ci->filterWidth * (depthwise ? 1 : ci->inChannels)));
  TFJS_REQUIRE(ctx, grid.y <= 65535u, "filter too large for the gradient kernel");
  if (depthwise)
    conv_der_filter_kernel<true><<<grid, threads, 0, ctx->stream>>>(pa, pb, po, *ci);
  else
    conv_der_filter_kernel<false><<<grid, threads, 0, ctx->stream>>>(pa, pb, po, *ci);
  return post_launch(ctx, depthwise ? "depthwiseConv2DDerFilter" : "conv2dDerFilter");
}

}  // namespace

extern "C" int tfjs_cuda_conv2d_der_input(tfjs_cuda_ctx* ctx, tfjs_tensor_id dy, tfjs_tensor_id filter,
                                          tfjs_tensor_id dx, const tfjs_conv2d_info* info) {
  return conv_gradient(ctx, dy, filter, dx, info, false, true);
}
extern "C" int tfjs_cuda_conv2d_der_filter(tfjs_cuda_ctx* ctx, tfjs_tensor_id x, tfjs_tensor_id dy,
                                           tfjs_tensor_id dw, const tfjs_conv2d_info* info) {
  return conv_gradient(ctx, x, dy, dw, info, false, false);
}
extern "C" int tfjs_cuda_depthwise_conv2d_der_input(tfjs_cuda_ctx* ctx, tfjs_tensor_id dy, tfjs_tensor_id filter,
                                                    tfjs_tensor_id dx, const tfjs_conv2d_info* info) {
  return conv_gradient(ctx, dy, filter, dx, info, true, true);
}
extern "C" int tfjs_cuda_depthwise_conv2d_der_filter(tfjs_cuda_ctx* ctx, tfjs_tensor_id x, tfjs_tensor_id dy,
                                                     tfjs_tensor_id dw, const tfjs_conv2d_info* info) {
  return conv_gradient(ctx, x, dy, dw, info, true, false);
}

extern "C" int tfjs_cuda_pool2d_backprop(tfjs_cuda_ctx* ctx, tfjs_tensor_id dy_id, tfjs_tensor_id x_id,
                                         tfjs_tensor_id dx_id, const tfjs_conv2d_info* ci, int is_avg) {
  if (!ctx) return TFJS_CUDA_ERR_INVALID_ARG;
  int rc = check_info(ctx, ci);
  if (rc) return rc;
  const int64_t x_n = (int64_t)ci->batchSize * ci->inHeight * ci->inWidth * ci->inChannels;
  const int64_t y_n = (int64_t)ci->batchSize * ci->outHeight * ci->outWidth * ci->inChannels;
  TensorEntry *dy, *x, *dx;
  rc = get_f32(ctx, dy_id, y_n, "dy", &dy);
  if (rc) return rc;
  rc = get_f32(ctx, x_id, x_n, "x", &x);
  if (rc) return rc;
  rc = get_f32(ctx, dx_id, x_n, "dx", &dx);
  if (rc) return rc;
  dx->version++;
  if (x_n == 0) return TFJS_CUDA_OK;
  cudaSetDevice(ctx->device);
  const int grid = grid_for_elems(x_n, 256, ctx->sm_count);
  if (is_avg) {
    pool_backprop_kernel<true><<<grid, 256, 0, ctx->stream>>>((const float*)dy->ptr, nullptr, (float*)dx->ptr, *ci);
    return post_launch(ctx, "avgPoolBackprop");
  }
  void* pos;
  size_t cap;
  rc = ctx_alloc(ctx, (size_t)(y_n > 0 ? y_n : 1) * 4, &pos, &cap);
  if (rc) return rc;
  if (y_n > 0) {
    max_pool_positions_kernel<<<grid_for_elems(y_n, 256, ctx->sm_count), 256, 0, ctx->stream>>>(
        (const float*)x->ptr, (int32_t*)pos, *ci);
    rc = post_launch(ctx, "maxPoolPositions");
  }
  if (!rc) {
    pool_backprop_kernel<false><<<grid, 256, 0, ctx->stream>>>((const float*)dy->ptr, (const int32_t*)pos,
                                                                (float*)dx->ptr, *ci);
    rc = post_launch(ctx, "maxPoolBackprop");
  }
  ctx_free(ctx, pos, cap);
  return rc;
}

extern "C" int tfjs_cuda_clip_backprop(tfjs_cuda_ctx* ctx, tfjs_tensor_id dy_id, tfjs_tensor_id x_id,
                                       tfjs_tensor_id out_id, float lo, float hi) {
  if (!ctx) return TFJS_CUDA_ERR_INVALID_ARG;
  TensorEntry *dy, *x, *o;
  int rc = get_f32(ctx, x_id, 0, "x", &x);
  if (rc) return rc;
  rc = get_f32(ctx, dy_id, x->size, "dy", &dy);
  if (rc) return rc;
  rc = get_f32(ctx, out_id, x->size, "clip gradient", &o);
  if (rc) return rc;
  TFJS_REQUIRE(ctx, !x->quant.quantized && !dy->quant.quantized, "gradient kernels take float32 tensors");
  o->version++;
  if (x->size == 0) return TFJS_CUDA_OK;
  cudaSetDevice(ctx->device);
  clip_backprop_kernel<<<grid_for_elems(x->size, 256, ctx->sm_count), 256, 0, ctx->stream>>>(
      (const float*)dy->ptr, (const float*)x->ptr, (float*)o->ptr, x->size, lo, hi);
  return post_launch(ctx, "clipBackprop");
}

extern "C" int tfjs_cuda_transpose(tfjs_cuda_ctx* ctx, tfjs_tensor_id x_id, tfjs_tensor_id out_id, int rank,
                                   const int64_t* shape, const int32_t* perm) {
  if (!ctx) return TFJS_CUDA_ERR_INVALID_ARG;
  TFJS_REQUIRE(ctx, rank >= 0 && rank <= 8 && (rank == 0 || (shape && perm)), "rank out of range");
  TransposeDesc d;
  d.rank = rank;
  int64_t n = 1, stride[8];
  for (int i = rank - 1; i >= 0; --i) {
    TFJS_REQUIRE(ctx, shape[i] >= 0, "negative extent");
    stride[i] = n;
    n *= shape[i];
  }
  bool seen[8] = {false};
  for (int i = 0; i < rank; ++i) {
    TFJS_REQUIRE(ctx, perm[i] >= 0 && perm[i] < rank && !seen[perm[i]], "perm is not a permutation");
    seen[perm[i]] = true;
    d.out_shape[i] = shape[perm[i]];
    d.in_stride[i] = stride[perm[i]];
  }
  TensorEntry *x, *o;
  int rc = get_f32(ctx, x_id, n, "x", &x);
  if (rc) return rc;
  rc = get_f32(ctx, out_id, n, "transpose output", &o);
  if (rc) return rc;
  o->version++;
  if (n == 0) return TFJS_CUDA_OK;
  cudaSetDevice(ctx->device);
  transpose_kernel<<<grid_for_elems(n, 256, ctx->sm_count), 256, 0, ctx->stream>>>((const float*)x->ptr,
                                                                                    (float*)o->ptr, d, n);
  return post_launch(ctx, "transpose");
}
