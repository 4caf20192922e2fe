/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of the gradient kernels of tfjs-core's
 * MathBackendCPU (tfjs-core 1.2.7, src/backends/cpu/backend_cpu.ts), NHWC.  Same loop order and
 * JavaScript number semantics as the reference: `dotProd` is an IEEE float64, each store into
 * the Float32Array result rounds once.  Nothing in the shipped library links or calls this.
 */
#include <math.h>
#include <string.h>

#include "oracle.h"

static int imax(int a, int b) { return a > b ? a : b; }
static int imin(int a, int b) { return a < b ? a : b; }
/* Math.ceil(a / s) and the `< (x) / s` loop bound on integers a, s > 0 */
static int ceil_div(int a, int s) { return (int)ceil((double)a / (double)s); }
static int upper_bound(int limit, int num, int s) {
  /* for (y = ..; y < Math.min(limit, num / s); ++y): y runs while y < num / s (a real number) */
  const double q = (double)num / (double)s;
  int top = (int)ceil(q);
  return imin(limit, top);
}

/* backend_cpu.ts:1686-1762 conv2dDerInput: dx[b, xR, xC, d1] */
void tfo_conv2d_der_input(const float* dy, const float* w, float* dx, const tfo_conv_info* c) {
  const int fh = c->filterHeight, fw = c->filterWidth, sh = c->strideHeight, sw = c->strideWidth;
  const int top_pad = fh - 1 - c->padTop, left_pad = fw - 1 - c->padLeft;
  const int64_t w_s0 = (int64_t)fw * c->inChannels * c->outChannels;
  const int64_t w_s1 = (int64_t)c->inChannels * c->outChannels, w_s2 = c->outChannels;
  const int64_t y_row = (int64_t)c->outWidth * c->outChannels, y_batch = y_row * c->outHeight;
  const int64_t x_row = (int64_t)c->inWidth * c->inChannels, x_batch = x_row * c->inHeight;
  for (int b = 0; b < c->batchSize; ++b)
    for (int d1 = 0; d1 < c->inChannels; ++d1)
      for (int xr = 0; xr < c->inHeight; ++xr) {
        const int xr_corner = xr - top_pad;
        const int yr_min = imax(0, ceil_div(xr_corner, sh));
        const int yr_max = upper_bound(c->outHeight, fh + xr_corner, sh);
        for (int xc = 0; xc < c->inWidth; ++xc) {
          const int xc_corner = xc - left_pad;
          const int yc_min = imax(0, ceil_div(xc_corner, sw));
          const int yc_max = upper_bound(c->outWidth, fw + xc_corner, sw);
          double dot = 0.0;
          for (int yr = yr_min; yr < yr_max; ++yr) {
            const int wr = yr * sh - xr_corner;
            for (int yc = yc_min; yc < yc_max; ++yc) {
              const int wc = yc * sw - xc_corner;
              const float* dyp = dy + b * y_batch + yr * y_row + (int64_t)yc * c->outChannels;
              const float* wp = w + w_s0 * (fh - 1 - wr) + w_s1 * (fw - 1 - wc) + w_s2 * d1;
              for (int d2 = 0; d2 < c->outChannels; ++d2) dot += (double)dyp[d2] * (double)wp[d2];
            }
          }
          dx[b * x_batch + xr * x_row + (int64_t)xc * c->inChannels + d1] = (float)dot;
        }
      }
}

/* backend_cpu.ts:1849-1898 conv2dDerFilter: dW[wR, wC, d1, d2] */
void tfo_conv2d_der_filter(const float* x, const float* dy, float* dw, const tfo_conv_info* c) {
  const int sh = c->strideHeight, sw = c->strideWidth;
  const int64_t y_row = (int64_t)c->outWidth * c->outChannels, y_batch = y_row * c->outHeight;
  const int64_t x_row = (int64_t)c->inWidth * c->inChannels, x_batch = x_row * c->inHeight;
  for (int wr = 0; wr < c->filterHeight; ++wr) {
    const int yr_min = imax(0, ceil_div(c->padTop - wr, sh));
    const int yr_max = upper_bound(c->outHeight, c->inHeight + c->padTop - wr, sh);
    for (int wc = 0; wc < c->filterWidth; ++wc) {
      const int yc_min = imax(0, ceil_div(c->padLeft - wc, sw));
      const int yc_max = upper_bound(c->outWidth, c->inWidth + c->padLeft - wc, sw);
      for (int d1 = 0; d1 < c->inChannels; ++d1)
        for (int d2 = 0; d2 < c->outChannels; ++d2) {
          double dot = 0.0;
          for (int b = 0; b < c->batchSize; ++b)
            for (int yr = yr_min; yr < yr_max; ++yr) {
              const int xr = wr + yr * sh - c->padTop;
              for (int yc = yc_min; yc < yc_max; ++yc) {
                const int xc = wc + yc * sw - c->padLeft;
                dot += (double)x[b * x_batch + xr * x_row + (int64_t)xc * c->inChannels + d1] *
                       (double)dy[b * y_batch + yr * y_row + (int64_t)yc * c->outChannels + d2];
              }
            }
          dw[(((int64_t)wr * c->filterWidth + wc) * c->inChannels + d1) * c->outChannels + d2] = (float)dot;
        }
    }
  }
}

/* backend_cpu.ts:2037-2102 depthwiseConv2DDerInput */
void tfo_depthwise_der_input(const float* dy, const float* w, float* dx, const tfo_conv_info* c) {
  const int fh = c->filterHeight, fw = c->filterWidth, sh = c->strideHeight, sw = c->strideWidth;
  const int top_pad = fh - 1 - c->padTop, left_pad = fw - 1 - c->padLeft;
  const int ch_mul = c->outChannels / c->inChannels;
  const int64_t w_s0 = (int64_t)fw * c->inChannels * ch_mul, w_s1 = (int64_t)c->inChannels * ch_mul, w_s2 = ch_mul;
  const int64_t y_row = (int64_t)c->outWidth * c->outChannels, y_batch = y_row * c->outHeight;
  const int64_t x_row = (int64_t)c->inWidth * c->inChannels, x_batch = x_row * c->inHeight;
  for (int b = 0; b < c->batchSize; ++b)
    for (int d1 = 0; d1 < c->inChannels; ++d1)
      for (int xr = 0; xr < c->inHeight; ++xr) {
        const int xr_corner = xr - top_pad;
        const int yr_min = imax(0, ceil_div(xr_corner, sh));
        const int yr_max = upper_bound(c->outHeight, fh + xr_corner, sh);
        for (int xc = 0; xc < c->inWidth; ++xc) {
          const int xc_corner = xc - left_pad;
          const int yc_min = imax(0, ceil_div(xc_corner, sw));
          const int yc_max = upper_bound(c->outWidth, fw + xc_corner, sw);
          double dot = 0.0;
          for (int yr = yr_min; yr < yr_max; ++yr) {
            const int wr = yr * sh - xr_corner;
            for (int yc = yc_min; yc < yc_max; ++yc) {
              const int wc = yc * sw - xc_corner;
              const float* dyp = dy + b * y_batch + yr * y_row + (int64_t)yc * c->outChannels;
              const float* wp = w + w_s0 * (fh - 1 - wr) + w_s1 * (fw - 1 - wc) + w_s2 * d1;
              for (int dm = 0; dm < ch_mul; ++dm) dot += (double)dyp[d1 * ch_mul + dm] * (double)wp[dm];
            }
          }
          dx[b * x_batch + xr * x_row + (int64_t)xc * c->inChannels + d1] = (float)dot;
        }
      }
}

/* backend_cpu.ts:2104-2150 depthwiseConv2DDerFilter: dW[wR, wC, d1, dm] */
void tfo_depthwise_der_filter(const float* x, const float* dy, float* dw, const tfo_conv_info* c) {
  const int sh = c->strideHeight, sw = c->strideWidth;
  const int ch_mul = c->outChannels / c->inChannels;
  const int64_t y_row = (int64_t)c->outWidth * c->outChannels, y_batch = y_row * c->outHeight;
  const int64_t x_row = (int64_t)c->inWidth * c->inChannels, x_batch = x_row * c->inHeight;
  for (int wr = 0; wr < c->filterHeight; ++wr) {
    const int yr_min = imax(0, ceil_div(c->padTop - wr, sh));
    const int yr_max = upper_bound(c->outHeight, c->inHeight + c->padTop - wr, sh);
    for (int wc = 0; wc < c->filterWidth; ++wc) {
      const int yc_min = imax(0, ceil_div(c->padLeft - wc, sw));
      const int yc_max = upper_bound(c->outWidth, c->inWidth + c->padLeft - wc, sw);
      for (int d2 = 0; d2 < c->outChannels; ++d2) {
        const int d1 = d2 / ch_mul, dm = d2 % ch_mul;
        double dot = 0.0;
        for (int b = 0; b < c->batchSize; ++b)
          for (int yr = yr_min; yr < yr_max; ++yr) {
            const int xr = wr + yr * sh - c->padTop;
            for (int yc = yc_min; yc < yc_max; ++yc) {
              const int xc = wc + yc * sw - c->padLeft;
              dot += (double)x[b * x_batch + xr * x_row + (int64_t)xc * c->inChannels + d1] *
                     (double)dy[b * y_batch + yr * y_row + (int64_t)yc * c->outChannels + d2];
            }
          }
        dw[(((int64_t)wr * c->filterWidth + wc) * c->inChannels + d1) * ch_mul + dm] = (float)dot;
      }
    }
  }
}

/* backend_cpu.ts:2347-2398 maxPoolPositions: flat position inside the effective window, -1 when
 * no tap compares greater than -Infinity (NaN or an empty window). */
static void max_pool_positions(const float* x, int32_t* pos, const tfo_conv_info* c) {
  const int C = c->inChannels;
  const int64_t x_row = (int64_t)c->inWidth * C, x_batch = x_row * c->inHeight;
  const int64_t y_row = (int64_t)c->outWidth * C, y_batch = y_row * c->outHeight;
  for (int b = 0; b < c->batchSize; ++b)
    for (int d = 0; d < C; ++d)
      for (int yr = 0; yr < c->outHeight; ++yr) {
        const int xr_corner = yr * c->strideHeight - c->padTop;
        int xr_min = xr_corner;
        while (xr_min < 0) xr_min += c->dilationHeight;
        const int xr_max = imin(c->inHeight, c->effectiveFilterHeight + xr_corner);
        for (int yc = 0; yc < c->outWidth; ++yc) {
          const int xc_corner = yc * c->strideWidth - c->padLeft;
          int xc_min = xc_corner;
          while (xc_min < 0) xc_min += c->dilationWidth;
          const int xc_max = imin(c->inWidth, c->effectiveFilterWidth + xc_corner);
          double max_value = -INFINITY;
          int max_pos = -1;
          for (int xr = xr_min; xr < xr_max; xr += c->dilationHeight)
            for (int xc = xc_min; xc < xc_max; xc += c->dilationWidth) {
              const double pixel = (double)x[b * x_batch + xr * x_row + (int64_t)xc * C + d];
              if (pixel > max_value) {
                max_value = pixel;
                max_pos = (xr - xr_corner) * c->effectiveFilterWidth + (xc - xc_corner);
              }
            }
          pos[b * y_batch + yr * y_row + (int64_t)yc * C + d] = max_pos;
        }
      }
}

/* backend_cpu.ts:2400-2456 maxPoolBackprop / :2458-2509 avgPoolBackprop.  `pos` is scratch of the
 * output's size (max only). */
void tfo_pool_backprop(const float* dy, const float* x, float* dx, int32_t* pos, const tfo_conv_info* c,
                       int is_avg) {
  const int C = c->inChannels;
  const int efh = c->effectiveFilterHeight, efw = c->effectiveFilterWidth;
  const int pad_left = efw - 1 - c->padLeft, pad_top = efh - 1 - c->padTop;
  const int64_t x_row = (int64_t)c->inWidth * C, x_batch = x_row * c->inHeight;
  const int64_t y_row = (int64_t)c->outWidth * C, y_batch = y_row * c->outHeight;
  const double avg_multiplier = 1.0 / (double)(c->filterHeight * c->filterWidth);
  if (!is_avg) max_pool_positions(x, pos, c);
  for (int b = 0; b < c->batchSize; ++b)
    for (int d = 0; d < C; ++d)
      for (int dxr = 0; dxr < c->inHeight; ++dxr)
        for (int dxc = 0; dxc < c->inWidth; ++dxc) {
          const int dyr_corner = dxr - pad_top, dyc_corner = dxc - pad_left;
          double dot = 0.0;
          for (int wr = 0; wr < efh; wr += c->dilationHeight) {
            const int num_r = dyr_corner + wr;
            if (num_r < 0 || num_r % c->strideHeight != 0) continue;
            const int dyr = num_r / c->strideHeight;
            if (dyr >= c->outHeight) continue;
            for (int wc = 0; wc < efw; wc += c->dilationWidth) {
              const int num_c = dyc_corner + wc;
              if (num_c < 0 || num_c % c->strideWidth != 0) continue;
              const int dyc = num_c / c->strideWidth;
              if (dyc >= c->outWidth) continue;
              const int64_t yi = b * y_batch + dyr * y_row + (int64_t)dyc * C + d;
              if (is_avg) {
                dot += (double)dy[yi];
              } else {
                const int max_pos = efh * efw - 1 - pos[yi];
                if (max_pos == wr * efw + wc) dot += (double)dy[yi];
              }
            }
          }
          dx[b * x_batch + dxr * x_row + (int64_t)dxc * C + d] = (float)(is_avg ? dot * avg_multiplier : dot);
        }
}

/* backend_cpu.ts:1520-1534 step */
void tfo_step(const float* x, float* out, int64_t n, double alpha) {
  for (int64_t i = 0; i < n; ++i) out[i] = isnan(x[i]) ? x[i] : (float)(x[i] > 0 ? 1.0 : alpha);
}
