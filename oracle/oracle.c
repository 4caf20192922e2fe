/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of tfjs-core's MathBackendCPU for the
 * MobileNet inference path (see oracle.h).  The shipped library never calls this.
 *
 * Parity pin: checked against the literal known-answer vectors of the reference's own
 * spec files (extracted into tests/golden/reference_kats.json, checked by
 * tests/test_oracle_golden.py), and cross-checked against an independent float64 numpy
 * implementation (tests/f64_forward.py, by tests/test_oracle_crosscheck.py) on the shapes those
 * vectors do not cover: stride-2 SAME depthwise, 3x3 SAME convolution over many channels,
 * matMul beyond one 48-wide block, the whole MobileNetV1 forward.
 */
#include "oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#define MATMUL_BLOCK 48 /* backend_cpu.ts:83 blockSize */

static int imin(int a, int b) { return a < b ? a : b; }
static int imax(int a, int b) { return a > b ? a : b; }

/* conv_util.ts:391-397 */
static int effective_filter(int f, int d) { return d <= 1 ? f : f + (f - 1) * (d - 1); }

/* conv_util.ts:509-526 conditionalRound; *ok is cleared when the unrounded value is kept
 * and is not an integer (conv_util.ts:306-317 asserts). */
static int conditional_round(double v, int mode, int* ok) {
  switch (mode) {
    case TFO_ROUND_FLOOR: return (int)floor(v);
    case TFO_ROUND_ROUND: return (int)floor(v + 0.5); /* Math.round: half away from -inf */
    case TFO_ROUND_CEIL: return (int)ceil(v);
    default:
      if (v != floor(v)) *ok = 0;
      return (int)v;
  }
}

int tfo_compute_conv2d_info(const int32_t in_shape[4], const int32_t filter_shape[4],
                            int stride_h, int stride_w, int dil_h, int dil_w, int pad_mode,
                            int pad_value, int rounding_mode, int depthwise,
                            tfo_conv_info* o) {
  int ok = 1;
  memset(o, 0, sizeof(*o));
  o->batchSize = in_shape[0];
  o->inHeight = in_shape[1];
  o->inWidth = in_shape[2];
  o->inChannels = in_shape[3];
  o->filterHeight = filter_shape[0];
  o->filterWidth = filter_shape[1];
  o->strideHeight = stride_h;
  o->strideWidth = stride_w;
  o->dilationHeight = dil_h;
  o->dilationWidth = dil_w;
  o->effectiveFilterHeight = effective_filter(o->filterHeight, dil_h);
  o->effectiveFilterWidth = effective_filter(o->filterWidth, dil_w);
  const int fh = o->effectiveFilterHeight, fw = o->effectiveFilterWidth;
  if (pad_mode == TFO_PAD_NUMBER) {
    /* conv_util.ts:408-414: a numeric pad uses filterHeight and strideHeight for BOTH
     * output dimensions (computeOutputShape2D takes one fieldSize and one stride). */
    o->padTop = o->padBottom = o->padLeft = o->padRight = pad_value;
    o->outHeight = conditional_round(
        (double)(o->inHeight - fh + 2 * pad_value) / stride_h + 1, rounding_mode, &ok);
    o->outWidth = conditional_round(
        (double)(o->inWidth - fh + 2 * pad_value) / stride_h + 1, rounding_mode, &ok);
  } else if (pad_mode == TFO_PAD_SAME) {
    o->outHeight = (o->inHeight + stride_h - 1) / stride_h;
    o->outWidth = (o->inWidth + stride_w - 1) / stride_w;
    int pah = imax(0, (o->outHeight - 1) * stride_h + fh - o->inHeight);
    int paw = imax(0, (o->outWidth - 1) * stride_w + fw - o->inWidth);
    o->padTop = pah / 2;
    o->padBottom = pah - o->padTop;
    o->padLeft = paw / 2;
    o->padRight = paw - o->padLeft;
  } else {
    o->outHeight = (int)ceil((double)(o->inHeight - fh + 1) / stride_h);
    o->outWidth = (int)ceil((double)(o->inWidth - fw + 1) / stride_w);
  }
  /* conv_util.ts:151 */
  o->outChannels = depthwise ? filter_shape[3] * o->inChannels : filter_shape[3];
  return ok ? 0 : -1;
}

void tfo_batch_matmul(const float* a, const float* b, float* out, int batch, int a_d1, int a_d2,
                      int b_d1, int b_d2, int ta, int tb) {
  const int shared = ta ? a_d1 : a_d2;
  const int left = ta ? a_d2 : a_d1;
  const int right = tb ? b_d1 : b_d2;
  const int64_t a_batch = (int64_t)a_d1 * a_d2, b_batch = (int64_t)b_d1 * b_d2;
  const int64_t a_outer = ta ? 1 : a_d2, a_inner = ta ? a_d2 : 1;
  const int64_t b_inner = tb ? 1 : b_d2, b_outer = tb ? b_d2 : 1;
  const int64_t size = (int64_t)left * right;
  memset(out, 0, sizeof(float) * (size_t)(size * batch));
  for (int bi = 0; bi < batch; bi++)
    for (int i0 = 0; i0 < left; i0 += MATMUL_BLOCK)
      for (int j0 = 0; j0 < right; j0 += MATMUL_BLOCK)
        for (int k0 = 0; k0 < shared; k0 += MATMUL_BLOCK) {
          const int ib = imin(i0 + MATMUL_BLOCK, left), jb = imin(j0 + MATMUL_BLOCK, right),
                    kb = imin(k0 + MATMUL_BLOCK, shared);
          for (int i = i0; i < ib; i++)
            for (int j = j0; j < jb; j++) {
              double sum = 0.0; /* JS number */
              for (int k = k0; k < kb; k++)
                sum += (double)a[bi * a_batch + i * a_outer + k * a_inner] *
                       (double)b[k * b_inner + j * b_outer + bi * b_batch];
              float* r = &out[bi * size + ((int64_t)i * right + j)];
              *r = (float)((double)*r + sum); /* Float32Array += */
            }
        }
}

void tfo_conv2d(const float* x, const float* w, float* y, const tfo_conv_info* c) {
  const int64_t x_row = (int64_t)c->inWidth * c->inChannels, x_batch = x_row * c->inHeight;
  const int64_t y_row = (int64_t)c->outWidth * c->outChannels, y_batch = y_row * c->outHeight;
  const int64_t w_s0 = (int64_t)c->filterWidth * c->inChannels * c->outChannels;
  const int64_t w_s1 = (int64_t)c->inChannels * c->outChannels;
  memset(y, 0, sizeof(float) * (size_t)(y_batch * c->batchSize));
  for (int b = 0; b < c->batchSize; ++b)
    for (int yr = 0; yr < c->outHeight; ++yr) {
      const int xr_corner = yr * c->strideHeight - c->padTop;
      for (int wr = 0; wr < c->filterHeight; ++wr) {
        const int xr = xr_corner + wr * c->dilationHeight;
        if (xr < 0 || xr >= c->inHeight) continue;
        for (int yc = 0; yc < c->outWidth; ++yc) {
          float* yp = y + b * y_batch + yr * y_row + (int64_t)yc * c->outChannels;
          const int xc_corner = yc * c->strideWidth - c->padLeft;
          for (int wc = 0; wc < c->filterWidth; ++wc) {
            const int xc = xc_corner + wc * c->dilationWidth;
            if (xc < 0 || xc >= c->inWidth) continue;
            const float* xp = x + b * x_batch + xr * x_row + (int64_t)xc * c->inChannels;
            const float* wp = w + wr * w_s0 + wc * w_s1;
            for (int d1 = 0; d1 < c->inChannels; ++d1) {
              const double xv = (double)xp[d1];
              for (int d2 = 0; d2 < c->outChannels; ++d2)
                yp[d2] = (float)((double)yp[d2] + xv * (double)wp[d2]);
              wp += c->outChannels;
            }
          }
        }
      }
    }
}

void tfo_depthwise_conv2d(const float* x, const float* w, float* y, const tfo_conv_info* c) {
  const int ch_mul = c->outChannels / c->inChannels;
  const int64_t x_row = (int64_t)c->inWidth * c->inChannels, x_batch = x_row * c->inHeight;
  const int64_t y_row = (int64_t)c->outWidth * c->outChannels, y_batch = y_row * c->outHeight;
  const int64_t w_s0 = (int64_t)c->filterWidth * c->inChannels * ch_mul;
  const int64_t w_s1 = (int64_t)c->inChannels * ch_mul;
  memset(y, 0, sizeof(float) * (size_t)(y_batch * c->batchSize));
  for (int b = 0; b < c->batchSize; ++b)
    for (int yr = 0; yr < c->outHeight; ++yr) {
      const int xr_corner = yr * c->strideHeight - c->padLeft; /* sic: backend_cpu.ts:2000 */
      for (int wr = 0; wr < c->filterHeight; ++wr) {
        const int xr = xr_corner + wr * c->dilationHeight;
        if (xr < 0 || xr >= c->inHeight) continue;
        for (int yc = 0; yc < c->outWidth; ++yc) {
          float* yp = y + b * y_batch + yr * y_row + (int64_t)yc * c->outChannels;
          const int xc_corner = yc * c->strideWidth - c->padTop; /* sic: :2010 */
          for (int wc = 0; wc < c->filterWidth; ++wc) {
            const int xc = xc_corner + wc * c->dilationWidth;
            if (xc < 0 || xc >= c->inWidth) continue;
            const float* xp = x + b * x_batch + xr * x_row + (int64_t)xc * c->inChannels;
            const float* wp = w + wr * w_s0 + wc * w_s1;
            float* yq = yp;
            for (int d1 = 0; d1 < c->inChannels; ++d1) {
              const double xv = (double)xp[d1];
              for (int q = 0; q < ch_mul; ++q)
                yq[q] = (float)((double)yq[q] + xv * (double)wp[q]);
              yq += ch_mul;
              wp += ch_mul;
            }
          }
        }
      }
    }
}

void tfo_pool(const float* x, float* y, const tfo_conv_info* c, int is_avg) {
  const int C = c->inChannels;
  const int64_t x_col = C, x_row = (int64_t)c->inWidth * C, x_batch = x_row * c->inHeight;
  const int64_t y_col = C, y_row = (int64_t)c->outWidth * C, y_batch = y_row * c->outHeight;
  for (int b = 0; b < c->batchSize; ++b)
    for (int d = 0; d < C; ++d)
      for (int yr = 0; yr < c->outHeight; ++yr) {
        const int xr_corner = yr * c->strideHeight - c->padTop;
        const int xr_min = imax(0, xr_corner);
        const int xr_max = imin(c->inHeight, c->effectiveFilterHeight + xr_corner);
        for (int yc = 0; yc < c->outWidth; ++yc) {
          const int xc_corner = yc * c->strideWidth - c->padLeft;
          const int xc_min = imax(0, xc_corner);
          const int xc_max = imin(c->inWidth, c->effectiveFilterWidth + xc_corner);
          double mm = -INFINITY, avg = 0.0;
          int count = 0;
          for (int xr = xr_min; xr < xr_max; xr += c->dilationHeight) {
            for (int xc = xc_min; xc < xc_max; xc += c->dilationWidth) {
              const double pixel = (double)x[b * x_batch + xr * x_row + xc * x_col + d];
              if (!is_avg && pixel > mm) {
                mm = pixel;
              } else if (is_avg) {
                avg += pixel;
                count++;
              }
            }
            if (isnan(mm)) break; /* :2329, unreachable because NaN > x is false */
          }
          y[b * y_batch + yr * y_row + yc * y_col + d] = (float)(is_avg ? avg / count : mm);
        }
      }
}

static double binary_apply(int op, double a, double b) {
  switch (op) {
    case TFO_ADD: return a + b;
    case TFO_SUB: return a - b;
    case TFO_MUL: return a * b;
    case TFO_DIV: return a / b;
    case TFO_PRELU: return a < 0 ? b * a : a;
  }
  return NAN;
}

int64_t tfo_binary(int op, const float* a, const int32_t* a_shape, int a_rank, const float* b,
                   const int32_t* b_shape, int b_rank, float* out) {
  /* broadcast_util.ts:58-87 assertAndGetBroadcastShape */
  int rank = a_rank > b_rank ? a_rank : b_rank;
  int32_t oshape[8];
  if (rank > 8) return -1;
  for (int i = 0; i < rank; i++) {
    int da = i < a_rank ? a_shape[a_rank - 1 - i] : 1;
    int db = i < b_rank ? b_shape[b_rank - 1 - i] : 1;
    int r;
    if (da == 1) r = db;
    else if (db == 1) r = da;
    else if (da != db) return -1;
    else r = da;
    oshape[rank - 1 - i] = r;
  }
  int64_t n = 1, na = 1, nb = 1;
  for (int i = 0; i < rank; i++) n *= oshape[i];
  for (int i = 0; i < a_rank; i++) na *= a_shape[i];
  for (int i = 0; i < b_rank; i++) nb *= b_shape[i];
  /* broadcast_util.ts:28-41 getBroadcastDims: dims of size 1 stretched to >1 */
  int a_bc[8] = {0}, b_bc[8] = {0}, any = 0;
  for (int i = 0; i < a_rank; i++) {
    int dim = a_rank - 1 - i;
    if (oshape[rank - 1 - i] > 1 && a_shape[dim] == 1) { a_bc[dim] = 1; any = 1; }
  }
  for (int i = 0; i < b_rank; i++) {
    int dim = b_rank - 1 - i;
    if (oshape[rank - 1 - i] > 1 && b_shape[dim] == 1) { b_bc[dim] = 1; any = 1; }
  }
  if (!out) return n;
  if (!any) {
    /* backend_cpu.ts:3527-3530 modulo fast path */
    for (int64_t i = 0; i < n; ++i)
      out[i] = (float)binary_apply(op, (double)a[i % na], (double)b[i % nb]);
    return n;
  }
  for (int64_t i = 0; i < n; ++i) {
    int loc[8];
    int64_t rem = i;
    for (int d = rank - 1; d >= 0; --d) { loc[d] = (int)(rem % oshape[d]); rem /= oshape[d]; }
    int64_t ai = 0, bi = 0;
    for (int d = 0; d < a_rank; d++) ai = ai * a_shape[d] + (a_bc[d] ? 0 : loc[rank - a_rank + d]);
    for (int d = 0; d < b_rank; d++) bi = bi * b_shape[d] + (b_bc[d] ? 0 : loc[rank - b_rank + d]);
    out[i] = (float)binary_apply(op, (double)a[ai], (double)b[bi]);
  }
  return n;
}

void tfo_unary(int op, const float* x, float* out, int64_t n, double p0, double p1) {
  for (int64_t i = 0; i < n; ++i) {
    const double v = (double)x[i];
    double r;
    switch (op) {
      case TFO_RELU: r = isnan(v) ? v : (v > 0 ? v : 0.0); break; /* Math.max(0, v) */
      case TFO_CLIP: r = v > p1 ? p1 : (v < p0 ? p0 : v); break;
      case TFO_EXP: r = exp(v); break;
      case TFO_LOG: r = log(v); break;
      default: r = NAN;
    }
    out[i] = (float)r;
  }
}

void tfo_sum_last(const float* x, float* out, int64_t outer, int64_t inner) {
  for (int64_t i = 0; i < outer; ++i) {
    double s = 0;
    for (int64_t j = 0; j < inner; ++j) s += (double)x[i * inner + j];
    out[i] = (float)s;
  }
}

void tfo_max_last(const float* x, float* out, int64_t outer, int64_t inner) {
  for (int64_t i = 0; i < outer; ++i) {
    float m = x[i * inner];
    for (int64_t j = 0; j < inner; ++j)
      if (x[i * inner + j] > m) m = x[i * inner + j];
    out[i] = m;
  }
}

void tfo_argmax_last(const float* x, int32_t* out, int64_t outer, int64_t inner) {
  for (int64_t i = 0; i < outer; ++i) {
    float m = x[i * inner];
    int32_t mi = 0;
    for (int64_t j = 0; j < inner; ++j)
      if (x[i * inner + j] > m) { m = x[i * inner + j]; mi = (int32_t)j; }
    out[i] = mi;
  }
}

void tfo_softmax_last(const float* x, float* out, int64_t outer, int64_t inner) {
  /* logSumExp (reduction_ops.ts:60-65): xMax = max(x); a = x - xMax; b = exp(a);
   * c = sum(b); d = log(c); lse = xMax + d.  softmax (softmax.ts:60-62): exp(x - lse). */
  for (int64_t i = 0; i < outer; ++i) {
    const float* r = x + i * inner;
    float m = r[0];
    for (int64_t j = 0; j < inner; ++j)
      if (r[j] > m) m = r[j];
    double c = 0;
    for (int64_t j = 0; j < inner; ++j) {
      float a = (float)((double)r[j] - (double)m);
      float b = (float)exp((double)a);
      c += (double)b;
    }
    float cf = (float)c;
    float d = (float)log((double)cf);
    float lse = (float)((double)m + (double)d);
    for (int64_t j = 0; j < inner; ++j) {
      float lr = (float)((double)r[j] - (double)lse);
      out[i * inner + j] = (float)exp((double)lr);
    }
  }
}

void tfo_dequant_u8(const uint8_t* q, int64_t n, double scale, double min, float* out) {
  for (int64_t i = 0; i < n; ++i) out[i] = (float)((double)q[i] * scale + min);
}

static void epilogue(float* y, int64_t n, const float* bias, int64_t bias_n, int act,
                     const float* prelu, int64_t prelu_n) {
  if (bias)
    for (int64_t i = 0; i < n; ++i) y[i] = (float)((double)y[i] + (double)bias[i % bias_n]);
  if (act == TFO_ACT_RELU) {
    tfo_unary(TFO_RELU, y, y, n, 0, 0);
  } else if (act == TFO_ACT_PRELU) {
    for (int64_t i = 0; i < n; ++i)
      y[i] = (float)binary_apply(TFO_PRELU, (double)y[i], (double)prelu[i % prelu_n]);
  }
}

void tfo_fused_matmul(const float* a, const float* b, float* out, int batch, int a_d1, int a_d2,
                      int b_d1, int b_d2, int ta, int tb, const float* bias, int64_t bias_n,
                      int act, const float* prelu, int64_t prelu_n) {
  tfo_batch_matmul(a, b, out, batch, a_d1, a_d2, b_d1, b_d2, ta, tb);
  const int left = ta ? a_d2 : a_d1, right = tb ? b_d1 : b_d2;
  epilogue(out, (int64_t)batch * left * right, bias, bias_n, act, prelu, prelu_n);
}

void tfo_fused_conv2d(const float* x, const float* w, float* y, const tfo_conv_info* c,
                      const float* bias, int64_t bias_n, int act, const float* prelu,
                      int64_t prelu_n) {
  tfo_conv2d(x, w, y, c);
  epilogue(y, (int64_t)c->batchSize * c->outHeight * c->outWidth * c->outChannels, bias, bias_n,
           act, prelu, prelu_n);
}
