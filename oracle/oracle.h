/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of tfjs-core's MathBackendCPU for the
 * MobileNet inference path.  Nothing in the shipped library links, loads or calls this;
 * only tests, the smoke check and the bench's cpu-baseline leg do.
 *
 * Every function restates one routine of the reference (tfjs-core 1.2.7) and cites it.
 * JavaScript number semantics are reproduced: scalar temporaries are IEEE float64, every
 * store into a Float32Array rounds to nearest-even float32.  Build with
 * -O2 -ffp-contract=off and without -ffast-math (see Makefile).
 */
#ifndef TFJS_ORACLE_H_
#define TFJS_ORACLE_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Mirror of Conv2DInfo, tfjs-core/src/ops/conv_util.ts:43-64 (channelsLast only). */
typedef struct {
  int32_t batchSize, inHeight, inWidth, inChannels;
  int32_t outHeight, outWidth, outChannels;
  int32_t strideHeight, strideWidth;
  int32_t dilationHeight, dilationWidth;
  int32_t filterHeight, filterWidth;
  int32_t effectiveFilterHeight, effectiveFilterWidth;
  int32_t padTop, padBottom, padLeft, padRight;
} tfo_conv_info;

enum { TFO_PAD_VALID = 0, TFO_PAD_SAME = 1, TFO_PAD_NUMBER = 2 };
enum { TFO_ROUND_NONE = 0, TFO_ROUND_FLOOR = 1, TFO_ROUND_ROUND = 2, TFO_ROUND_CEIL = 3 };
enum { TFO_ACT_LINEAR = 0, TFO_ACT_RELU = 1, TFO_ACT_PRELU = 2 };
enum { TFO_ADD = 0, TFO_SUB = 1, TFO_MUL = 2, TFO_DIV = 3, TFO_PRELU = 4 };
enum { TFO_RELU = 0, TFO_CLIP = 1, TFO_EXP = 2, TFO_LOG = 3 };

/* conv_util.ts:123-182 computeConv2DInfo (+ getPadAndOutInfo :399-435).  Returns 0, or -1
 * when the numeric-pad output size is not an integer (the reference asserts). */
int tfo_compute_conv2d_info(const int32_t in_shape[4], const int32_t filter_shape[4],
                            int stride_h, int stride_w, int dil_h, int dil_w, int pad_mode,
                            int pad_value, int rounding_mode, int depthwise, tfo_conv_info* out);

/* backend_cpu.ts:491-540 batchMatMul.  a is [batch,d1,d2], b is [batch,e1,e2]. */
void tfo_batch_matmul(const float* a, const float* b, float* out, int batch, int a_d1, int a_d2,
                      int b_d1, int b_d2, int transpose_a, int transpose_b);

/* backend_cpu.ts:1552-1616 conv2d (NHWC). */
void tfo_conv2d(const float* x, const float* w, float* y, const tfo_conv_info* ci);

/* backend_cpu.ts:1979-2035 depthwiseConv2D (including the padLeft/padTop swap). */
void tfo_depthwise_conv2d(const float* x, const float* w, float* y, const tfo_conv_info* ci);

/* backend_cpu.ts:2273-2341 pool. */
void tfo_pool(const float* x, float* y, const tfo_conv_info* ci, int is_avg);

/* backend_cpu.ts:3515-3549 broadcastedBinaryOp with the float32 ops of :440-481, 557-572,
 * 1203-1209.  Returns the output element count, or -1 if shapes do not broadcast. */
int64_t tfo_binary(int op, const float* a, const int32_t* a_shape, int a_rank, const float* b,
                   const int32_t* b_shape, int b_rank, float* out);

/* backend_cpu.ts:1191-1201 relu, :1265-1275 clip, :1094-1103 exp, :1116-1126 log. */
void tfo_unary(int op, const float* x, float* out, int64_t n, double p0, double p1);

/* backend_cpu.ts:590-611 sum, :906-929 max, :686-712 argMax over the inner-most `inner`. */
void tfo_sum_last(const float* x, float* out, int64_t outer, int64_t inner);
void tfo_max_last(const float* x, float* out, int64_t outer, int64_t inner);
void tfo_argmax_last(const float* x, int32_t* out, int64_t outer, int64_t inner);

/* ops/softmax.ts:57-63 + ops/reduction_ops.ts:56-73: the 8-stage chain, each stage rounded. */
void tfo_softmax_last(const float* x, float* out, int64_t outer, int64_t inner);

/* io/io_utils.ts:137-139 uint8 affine dequantisation to float32. */
void tfo_dequant_u8(const uint8_t* q, int64_t n, double scale, double min, float* out);

/* backend_cpu.ts:542-555 fusedBatchMatMul / :1536-1550 fusedConv2d: op, then add(bias),
 * then activation, as three separately rounded passes.  bias may be NULL; bias_n is its
 * element count (broadcast along the inner-most axis by i % bias_n, the reference fast path). */
void tfo_fused_matmul(const float* a, const float* b, float* out, int batch, int a_d1, int a_d2,
                      int b_d1, int b_d2, int transpose_a, int transpose_b, const float* bias,
                      int64_t bias_n, int act, const float* prelu, int64_t prelu_n);
void tfo_fused_conv2d(const float* x, const float* w, float* y, const tfo_conv_info* ci,
                      const float* bias, int64_t bias_n, int act, const float* prelu,
                      int64_t prelu_n);

/* ---- gradient kernels (oracle_backward.c) ---- */
/* backend_cpu.ts:1686-1762 conv2dDerInput and :1849-1898 conv2dDerFilter */
void tfo_conv2d_der_input(const float* dy, const float* w, float* dx, const tfo_conv_info* ci);
void tfo_conv2d_der_filter(const float* x, const float* dy, float* dw, const tfo_conv_info* ci);
/* backend_cpu.ts:2037-2102 depthwiseConv2DDerInput and :2104-2150 depthwiseConv2DDerFilter */
void tfo_depthwise_der_input(const float* dy, const float* w, float* dx, const tfo_conv_info* ci);
void tfo_depthwise_der_filter(const float* x, const float* dy, float* dw, const tfo_conv_info* ci);
/* backend_cpu.ts:2400-2456 maxPoolBackprop (with maxPoolPositions :2347-2398; `pos` is scratch of
 * the pooled output's size) and :2458-2509 avgPoolBackprop */
void tfo_pool_backprop(const float* dy, const float* x, float* dx, int32_t* pos, const tfo_conv_info* ci,
                       int is_avg);
/* backend_cpu.ts:1520-1534 step */
void tfo_step(const float* x, float* out, int64_t n, double alpha);

#ifdef __cplusplus
}
#endif
#endif
