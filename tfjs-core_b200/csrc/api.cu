// extern "C" entry points of the contraction, convolution and pooling kernels: argument
// checking, operand preparation (weight repacking cache, transposes) and kernel selection.
#include "common.cuh"

namespace {

// The derived forms of a weight tensor (dequantised copy, repacked tf32 planes, K-major bytes)
// are computed once and cached on the tensor.  While a graph is being captured a kernel is only
// recorded, not run, so a cache filled during capture would be marked valid without ever having
// been written: an eager call on the same tensor before the first replay would read garbage, and
// every replay would redo the repack.  A miss during capture is therefore refused.
int refuse_miss_during_capture(tfjs_cuda_ctx* ctx, const char* what) {
  if (!ctx->capturing) return TFJS_CUDA_OK;
  return set_error(ctx, TFJS_CUDA_ERR_UNSUPPORTED,
                   "%s of a weight tensor is not prepared yet and cannot be prepared while a graph is being "
                   "captured: run the same calls once eagerly before tfjs_cuda_graph_begin",
                   what);
}

// float32 view of a tensor for kernels that read plain floats; a quantised tensor gets a
// cached dequantised copy (io_utils.ts:139 arithmetic).
int float_view(tfjs_cuda_ctx* ctx, TensorEntry* t, const float** out) {
  if (!t->quant.quantized) {
    *out = (const float*)t->ptr;
    return TFJS_CUDA_OK;
  }
  if (!t->deq || t->deq_version != t->version) {
    int miss = refuse_miss_during_capture(ctx, "the dequantised copy");
    if (miss) return miss;
    if (!t->deq) {
      void* p;
      int rc = ctx_alloc(ctx, (size_t)t->size * 4, &p, &t->deq_capacity);
      if (rc) return rc;
      t->deq = (float*)p;
    }
    int rc = launch_dequant(ctx, (const uint8_t*)t->ptr, t->deq, t->size, t->quant.scale, t->quant.min);
    if (rc) return rc;
    t->deq_version = t->version;
  }
  *out = t->deq;
  return TFJS_CUDA_OK;
}

// K-major tf32 hi/lo planes of a [K, N] operand (or of its [N, K] transpose), cached on the
// tensor entry until the tensor is rewritten.  Weights are constants in inference, so the
// repack runs once per weight tensor.
int packed_weights(tfjs_cuda_ctx* ctx, TensorEntry* w, int64_t offset_elems, int64_t K, int64_t N,
                   bool source_is_nk, bool cacheable, PackedWeights* out, bool* temporary,
                   int row_len = 0, int row_pad = 0, int64_t k_packed = 0) {
  // row_pad > 0: each run of row_len source rows becomes row_pad packed columns (k_packed total)
  const int64_t kp = row_pad > 0 ? k_packed : (K + 3) / 4 * 4;
  PackedWeights& c = w->packed;
  *temporary = !cacheable;
  if (cacheable && c.hi && c.version == w->version && c.n == N && c.k == K &&
      c.transposed_source == source_is_nk && c.row_pad == row_pad) {
    *out = c;
    return TFJS_CUDA_OK;
  }
  if (cacheable) {
    int miss = refuse_miss_during_capture(ctx, "the tensor-core layout");
    if (miss) return miss;
  }
  PackedWeights fresh;
  fresh.n = N;
  fresh.k = K;
  fresh.kp = kp;
  fresh.version = w->version;
  fresh.transposed_source = source_is_nk;
  fresh.row_pad = row_pad;
  void *hi, *lo;
  int rc = ctx_alloc(ctx, (size_t)(N * kp) * 4, &hi, &fresh.capacity);
  if (rc) return rc;
  rc = ctx_alloc(ctx, (size_t)(N * kp) * 4, &lo, &fresh.capacity);
  if (rc) {
    ctx_free(ctx, hi, fresh.capacity);
    return rc;
  }
  fresh.hi = (float*)hi;
  fresh.lo = (float*)lo;
  const bool u8 = w->quant.quantized;
  const void* src = u8 ? (const void*)((const uint8_t*)w->ptr + offset_elems)
                       : (const void*)((const float*)w->ptr + offset_elems);
  if (row_pad > 0)
    rc = launch_pack_weights_rows(ctx, src, u8, w->quant.scale, w->quant.min, K, N, row_len, row_pad, kp,
                                  fresh.hi, fresh.lo);
  else
    rc = launch_pack_weights(ctx, src, u8, w->quant.scale, w->quant.min, K, N,
                             source_is_nk ? 1 : N, source_is_nk ? K : 1, kp, fresh.hi, fresh.lo);
  if (rc) {
    ctx_free(ctx, hi, fresh.capacity);
    ctx_free(ctx, lo, fresh.capacity);
    return rc;
  }
  if (cacheable) {
    if (c.hi) ctx_free(ctx, c.hi, c.capacity);
    if (c.lo) ctx_free(ctx, c.lo, c.capacity);
    c = fresh;
  }
  *out = fresh;
  return TFJS_CUDA_OK;
}

// ---- 16-bit activation storage --------------------------------------------------------------
// An activation tensor may be stored as IEEE half (TFJS_F16).  Kernels with a native half path
// take it as it is; every other kernel sees a float32 temporary (converted before, and for an
// output converted back after), so that any call works on any storage and only the hot path
// needs half-aware kernels.  Temporaries are stream-ordered like every other buffer.
struct F32View {
  const float* ptr = nullptr;
  void* tmp = nullptr;
  size_t cap = 0;
};
int view_as_f32(tfjs_cuda_ctx* ctx, TensorEntry* t, F32View* v) {
  if (t->dtype != TFJS_F16) {
    v->ptr = (const float*)t->ptr;
    return TFJS_CUDA_OK;
  }
  int rc = ctx_alloc(ctx, (size_t)t->size * 4, &v->tmp, &v->cap);
  if (rc) return rc;
  v->ptr = (const float*)v->tmp;
  return launch_convert(ctx, t->ptr, TFJS_F16, v->tmp, TFJS_F32, t->size);
}
void release_view(tfjs_cuda_ctx* ctx, F32View* v) {
  if (v->tmp) ctx_free(ctx, v->tmp, v->cap);
  v->tmp = nullptr;
}
struct F32Out {
  float* ptr = nullptr;
  void* tmp = nullptr;
  size_t cap = 0;
  TensorEntry* dst = nullptr;
};
int out_as_f32(tfjs_cuda_ctx* ctx, TensorEntry* o, F32Out* v) {
  v->dst = o;
  if (o->dtype != TFJS_F16) {
    v->ptr = (float*)o->ptr;
    return TFJS_CUDA_OK;
  }
  int rc = ctx_alloc(ctx, (size_t)o->size * 4, &v->tmp, &v->cap);
  if (rc) return rc;
  v->ptr = (float*)v->tmp;
  return TFJS_CUDA_OK;
}
// Converts the float32 temporary into the half tensor (when there is one) and frees it.
int finish_out(tfjs_cuda_ctx* ctx, F32Out* v, int rc) {
  if (v->tmp) {
    if (!rc) rc = launch_convert(ctx, v->tmp, TFJS_F32, v->dst->ptr, TFJS_F16, v->dst->size);
    ctx_free(ctx, v->tmp, v->cap);
    v->tmp = nullptr;
  }
  return rc;
}

// K-major IEEE half plane [N, kp] of a [K, N] contraction operand, cached on the tensor.
int half_weights(tfjs_cuda_ctx* ctx, TensorEntry* w, int64_t K, int64_t N, const void** plane, int64_t* kp_out) {
  const int64_t kp = (K + 7) / 8 * 8;
  if (!w->w16 || w->w16_version != w->version || w->w16_n != N || w->w16_k != K) {
    int miss = refuse_miss_during_capture(ctx, "the half-precision tensor-core layout");
    if (miss) return miss;
    if (w->w16) ctx_free(ctx, w->w16, w->w16_capacity);
    w->w16 = nullptr;
    int rc = ctx_alloc(ctx, (size_t)(N * kp) * 2, &w->w16, &w->w16_capacity);
    if (rc) return rc;
    rc = launch_pack_weights_f16(ctx, w->ptr, w->quant.quantized, w->quant.scale, w->quant.min, K, N, N, 1, kp,
                                 w->w16);
    if (rc) return rc;
    w->w16_version = w->version;
    w->w16_n = N;
    w->w16_k = K;
    w->w16_kp = kp;
  }
  *plane = w->w16;
  *kp_out = kp;
  return TFJS_CUDA_OK;
}

// Whether the whole-image depthwise kernel takes this call on half storage.
bool depthwise_half_native(const tfjs_conv2d_info& ci, const EpilogueArgs& e, const void* x, const float* w,
                           const void* y) {
  return ci.inChannels % 4 == 0 && depthwise_image_supported(ci, e.activation, true) &&
         (((uintptr_t)x | (uintptr_t)w | (uintptr_t)y) & 15) == 0 &&
         (e.bias == nullptr || ((uintptr_t)e.bias & 15) == 0);
}

void release_temporary(tfjs_cuda_ctx* ctx, const PackedWeights& p, bool temporary) {
  if (!temporary) return;
  ctx_free(ctx, p.hi, p.capacity);
  ctx_free(ctx, p.lo, p.capacity);
}

// out[M, N] = epi(a[M, K] . w), with w a [K, N] (or [N, K] when source_is_nk) operand.
int gemm_dispatch(tfjs_cuda_ctx* ctx, const float* a, int64_t M, int64_t K, TensorEntry* w,
                  int64_t w_offset, bool source_is_nk, bool cacheable, float* out, int64_t N,
                  const EpilogueArgs& epi, bool a_tf32_exact = false) {
  if (ctx->use_tensor_cores && tcgen05_gemm_supported(M, N, K)) {
    if (ctx->dequant_in_gemm && w->quant.quantized && cacheable && w_offset == 0) {
      // Quantised weights stay uint8 in HBM: a K-major byte copy is cached once and the kernel
      // dequantises each tile in shared memory.
      const int64_t kq = (K + 15) / 16 * 16;
      if (!w->packed_q || w->packed_q_version != w->version || w->packed_q_n != N ||
          w->packed_q_k != K || w->packed_q_transposed != source_is_nk) {
        int miss = refuse_miss_during_capture(ctx, "the K-major uint8 layout");
        if (miss) return miss;
        if (w->packed_q) ctx_free(ctx, w->packed_q, w->packed_q_capacity);
        w->packed_q = nullptr;
        void* p;
        int rc = ctx_alloc(ctx, (size_t)(N * kq), &p, &w->packed_q_capacity);
        if (rc) return rc;
        w->packed_q = (uint8_t*)p;
        rc = launch_pack_u8(ctx, (const uint8_t*)w->ptr, K, N, source_is_nk ? 1 : N,
                            source_is_nk ? K : 1, kq, w->packed_q);
        if (rc) return rc;
        w->packed_q_version = w->version;
        w->packed_q_n = N;
        w->packed_q_k = K;
        w->packed_q_kq = kq;
        w->packed_q_transposed = source_is_nk;
      }
      return launch_gemm_tcgen05_u8(ctx, a, M, K, w->packed_q, kq, w->quant.scale, w->quant.min, out,
                                    N, epi, ctx->math_mode, a_tf32_exact);
    }
    PackedWeights pw;
    bool temporary;
    int rc = packed_weights(ctx, w, w_offset, K, N, source_is_nk, cacheable, &pw, &temporary);
    if (rc) return rc;
    rc = launch_gemm_tcgen05(ctx, a, M, K, pw.hi, pw.lo, pw.kp, out, N, epi, ctx->math_mode, a_tf32_exact);
    release_temporary(ctx, pw, temporary);
    return rc;
  }
  const float* wf;
  int rc = float_view(ctx, w, &wf);
  if (rc) return rc;
  wf += w_offset;
  return launch_gemm_simt(ctx, a, wf, out, 1, (int)M, (int)N, (int)K, 0, K, 1, 0,
                          source_is_nk ? 1 : N, source_is_nk ? K : 1, epi);
}

}  // namespace

extern "C" int tfjs_cuda_batch_matmul(tfjs_cuda_ctx* ctx, tfjs_tensor_id a_id, tfjs_tensor_id b_id,
                                      tfjs_tensor_id out_id, int32_t batch, int32_t a_d1,
                                      int32_t a_d2, int32_t b_d1, int32_t b_d2, int transpose_a,
                                      int transpose_b, const tfjs_epilogue* epi) {
  if (!ctx) return TFJS_CUDA_ERR_INVALID_ARG;
  TFJS_REQUIRE(ctx, batch >= 0 && a_d1 >= 0 && a_d2 >= 0 && b_d1 >= 0 && b_d2 >= 0, "negative extent");
  const int64_t K = transpose_a ? a_d1 : a_d2;
  const int64_t M = transpose_a ? a_d2 : a_d1;
  const int64_t Kb = transpose_b ? b_d2 : b_d1;
  const int64_t N = transpose_b ? b_d1 : b_d2;
  // matmul.ts:81-87: inner shapes must match
  TFJS_REQUIRE(ctx, K == Kb, "Error in matMul: inner shapes (%lld) and (%lld) must match",
               (long long)K, (long long)Kb);
  TensorEntry *a, *b, *o;
  int rc = get_f32(ctx, a_id, (int64_t)batch * a_d1 * a_d2, "a", &a);
  if (rc) return rc;
  rc = get_f32(ctx, b_id, (int64_t)batch * b_d1 * b_d2, "b", &b);
  if (rc) return rc;
  rc = get_f32(ctx, out_id, (int64_t)batch * M * N, "matMul output", &o);
  if (rc) return rc;
  TFJS_REQUIRE(ctx, !a->quant.quantized && !o->quant.quantized, "only the b operand may be quantised");
  EpilogueArgs e;
  rc = resolve_epilogue(ctx, epi, N, &e);
  if (rc) return rc;
  o->version++;
  if ((int64_t)batch * M * N == 0) return TFJS_CUDA_OK;  // matmul_test.ts:621-642
  cudaSetDevice(ctx->device);
  const bool tc = ctx->use_tensor_cores && tcgen05_gemm_supported(M, N, K);
  if (!tc) {
    const float* bf;
    rc = float_view(ctx, b, &bf);
    if (rc) return rc;
    return launch_gemm_simt(ctx, (const float*)a->ptr, bf, (float*)o->ptr, batch, (int)M, (int)N, (int)K,
                            (int64_t)a_d1 * a_d2, transpose_a ? 1 : a_d2, transpose_a ? a_d2 : 1,
                            (int64_t)b_d1 * b_d2, transpose_b ? 1 : b_d2, transpose_b ? b_d2 : 1, e);
  }
  // Tensor-core path wants A as [M, K] with K contiguous.
  const float* a_mk = (const float*)a->ptr;
  void* a_scratch = nullptr;
  size_t a_cap = 0;
  if (transpose_a) {
    rc = ctx_alloc(ctx, (size_t)batch * M * K * 4, &a_scratch, &a_cap);
    if (rc) return rc;
    rc = launch_transpose_batched(ctx, (const float*)a->ptr, (float*)a_scratch, batch, (int)K, (int)M);
    if (rc) {
      ctx_free(ctx, a_scratch, a_cap);
      return rc;
    }
    a_mk = (const float*)a_scratch;
  }
  for (int bi = 0; bi < batch && !rc; bi++)
    rc = gemm_dispatch(ctx, a_mk + (int64_t)bi * M * K, M, K, b, (int64_t)bi * K * N, transpose_b != 0,
                       /*cacheable=*/batch == 1, (float*)o->ptr + (int64_t)bi * M * N, N, e);
  if (a_scratch) ctx_free(ctx, a_scratch, a_cap);
  return rc;
}

static int check_conv_info(tfjs_cuda_ctx* ctx, const tfjs_conv2d_info* ci) {
  TFJS_REQUIRE(ctx, ci != nullptr, "convInfo is null");
  TFJS_REQUIRE(ctx, ci->batchSize >= 0 && ci->inHeight >= 0 && ci->inWidth >= 0 && ci->inChannels >= 0 &&
                        ci->outHeight >= 0 && ci->outWidth >= 0 && ci->outChannels >= 0,
               "negative extent in convInfo");
  TFJS_REQUIRE(ctx, ci->strideHeight >= 1 && ci->strideWidth >= 1 && ci->dilationHeight >= 1 &&
                        ci->dilationWidth >= 1 && ci->filterHeight >= 1 && ci->filterWidth >= 1,
               "strides, dilations and filter sizes must be positive");
  return TFJS_CUDA_OK;
}

extern "C" int tfjs_cuda_conv2d(tfjs_cuda_ctx* ctx, tfjs_tensor_id x_id, tfjs_tensor_id w_id,
                                tfjs_tensor_id out_id, const tfjs_conv2d_info* ci,
                                const tfjs_epilogue* epi) {
  if (!ctx) return TFJS_CUDA_ERR_INVALID_ARG;
  int rc = check_conv_info(ctx, ci);
  if (rc) return rc;
  const int64_t pixels = (int64_t)ci->batchSize * ci->outHeight * ci->outWidth;
  TensorEntry *x, *w, *o;
  // x may also be a quantised tensor (uint8 bytes with scale / min): image pixels, decoded by the
  // stem kernel on chip, or through a float32 copy by every other kernel
  TensorEntry* xq = find_tensor(ctx, x_id);
  if (xq && xq->quant.quantized) {
    rc = get_f32(ctx, x_id, (int64_t)ci->batchSize * ci->inHeight * ci->inWidth * ci->inChannels, "x", &x);
  } else {
    rc = get_activation(ctx, x_id, (int64_t)ci->batchSize * ci->inHeight * ci->inWidth * ci->inChannels, "x", &x);
  }
  if (rc) return rc;
  rc = get_f32(ctx, w_id, (int64_t)ci->filterHeight * ci->filterWidth * ci->inChannels * ci->outChannels,
               "filter", &w);
  if (rc) return rc;
  rc = get_activation(ctx, out_id, pixels * ci->outChannels, "conv2d output", &o);
  if (rc) return rc;
  EpilogueArgs e;
  rc = resolve_epilogue(ctx, epi, ci->outChannels, &e);
  if (rc) return rc;
  o->version++;
  if (pixels * ci->outChannels == 0) return TFJS_CUDA_OK;
  cudaSetDevice(ctx->device);
  // A 1x1 stride-1 unpadded convolution over NHWC is the GEMM [B*H*W, Cin] x [Cin, Cout].
  const bool pointwise = ci->filterHeight == 1 && ci->filterWidth == 1 && ci->strideHeight == 1 &&
                         ci->strideWidth == 1 && ci->padTop == 0 && ci->padLeft == 0 &&
                         ci->outHeight == ci->inHeight && ci->outWidth == ci->inWidth;
  const bool x16 = x->dtype == TFJS_F16, o16 = o->dtype == TFJS_F16;
  // Half-precision activations: the pointwise convolution runs on the tensor cores' f16 path,
  // reading x (and writing out, if it is half too) as stored.
  if (x16 && pointwise && ci->inChannels > 0 && ctx->use_tensor_cores && e.activation != TFJS_ACT_PRELU &&
      tcgen05_gemm_f16_supported(pixels, ci->outChannels, ci->inChannels, o16)) {
    const void* plane;
    int64_t kp;
    rc = half_weights(ctx, w, ci->inChannels, ci->outChannels, &plane, &kp);
    if (rc) return rc;
    return launch_gemm_tcgen05_f16(ctx, x->ptr, pixels, ci->inChannels, plane, kp, o->ptr, o16, ci->outChannels, e);
  }
  // The 3-channel 3x3 stem: the image window of a patch arrives by TMA and is rearranged into
  // im2col rows in shared memory (TF32; other modes take the gather path below).  It can store
  // its result as half directly.
  const bool x8 = x->quant.quantized;
  const bool split3 = ctx->math_mode == TFJS_MATH_TF32X3;  // 3xTF32: float32 image in, float32 out
  if (!x16 && ctx->use_tensor_cores && !(split3 && (o16 || x8)) &&
      (x8 ? conv_rgb_u8_tcgen05_supported(*ci, e.activation, ctx->math_mode)
          : conv_rgb_tcgen05_supported(*ci, e.activation, ctx->math_mode))) {
    PackedWeights pw;
    bool temporary;
    rc = packed_weights(ctx, w, 0, 27, ci->outChannels, false, true, &pw, &temporary, 9, 10, 32);
    if (rc) return rc;
    return launch_conv_rgb_tcgen05(ctx, x->ptr, *ci, pw.hi, pw.kp, o->ptr, e, o16, x8, x->quant.scale, x->quant.min,
                                   split3 ? pw.lo : nullptr);
  }
  // Every other kernel computes on float32 storage.
  F32View xv;
  F32Out ov;
  if (x8) {  // decoded copy (cached on the tensor until its bytes change)
    rc = float_view(ctx, x, &xv.ptr);
  } else {
    rc = view_as_f32(ctx, x, &xv);
  }
  if (!rc) rc = out_as_f32(ctx, o, &ov);
  if (rc) {
    release_view(ctx, &xv);
    return finish_out(ctx, &ov, rc);
  }
  auto done = [&](int status) {
    release_view(ctx, &xv);
    return finish_out(ctx, &ov, status);
  };
  if (pointwise && ci->inChannels > 0)
    return done(gemm_dispatch(ctx, xv.ptr, pixels, ci->inChannels, w, 0, false, true, ov.ptr, ci->outChannels, e));
  // Cin a multiple of 32 at stride 1: each filter tap's A tile is one TMA load of the shifted
  // output patch (TF32; 3xTF32 and strided shapes take the gather path below).
  if (ctx->use_tensor_cores && conv_tma_tcgen05_supported(*ci, e.activation, ctx->math_mode)) {
    PackedWeights pw;
    bool temporary;
    rc = packed_weights(ctx, w, 0, (int64_t)ci->filterHeight * ci->filterWidth * ci->inChannels,
                        ci->outChannels, false, true, &pw, &temporary);
    if (rc) return done(rc);
    return done(launch_conv_tma_tcgen05(ctx, xv.ptr, *ci, pw.hi, pw.kp, ov.ptr, e, split3 ? pw.lo : nullptr));
  }
  // Everything else with Cin % 4 == 0 (or a 3-channel, 3-wide filter) is an implicit GEMM: the
  // A tile is gathered from the image by the kernel itself, K = fH * fW * Cin.
  const int mode = ctx->use_tensor_cores ? tcgen05_conv_mode(*ci) : 0;
  if (mode) {
    const int64_t K = (int64_t)ci->filterHeight * ci->filterWidth * ci->inChannels;
    const bool rgb = tcgen05_conv_k(*ci, mode) != K;
    PackedWeights pw;
    bool temporary;
    rc = packed_weights(ctx, w, 0, K, ci->outChannels, false, true, &pw, &temporary,
                        rgb ? ci->filterWidth * ci->inChannels : 0, rgb ? 10 : 0,
                        rgb ? tcgen05_conv_k(*ci, mode) : 0);
    if (rc) return done(rc);
    return done(launch_conv_tcgen05(ctx, mode, xv.ptr, *ci, pw.hi, pw.lo, pw.kp, ov.ptr, e, ctx->math_mode));
  }
  const float* wf;
  rc = float_view(ctx, w, &wf);
  if (rc) return done(rc);
  return done(launch_conv2d_direct(ctx, xv.ptr, wf, ov.ptr, *ci, e));
}

extern "C" int tfjs_cuda_depthwise_conv2d(tfjs_cuda_ctx* ctx, tfjs_tensor_id x_id, tfjs_tensor_id w_id,
                                          tfjs_tensor_id out_id, const tfjs_conv2d_info* ci,
                                          const tfjs_epilogue* epi) {
  if (!ctx) return TFJS_CUDA_ERR_INVALID_ARG;
  int rc = check_conv_info(ctx, ci);
  if (rc) return rc;
  TFJS_REQUIRE(ctx, ci->inChannels == 0 || ci->outChannels % ci->inChannels == 0,
               "depthwise outChannels must be a multiple of inChannels");
  const int64_t out_n = (int64_t)ci->batchSize * ci->outHeight * ci->outWidth * ci->outChannels;
  TensorEntry *x, *w, *o;
  rc = get_activation(ctx, x_id, (int64_t)ci->batchSize * ci->inHeight * ci->inWidth * ci->inChannels, "x", &x);
  if (rc) return rc;
  rc = get_f32(ctx, w_id, (int64_t)ci->filterHeight * ci->filterWidth * ci->outChannels, "filter", &w);
  if (rc) return rc;
  rc = get_activation(ctx, out_id, out_n, "depthwiseConv2D output", &o);
  if (rc) return rc;
  EpilogueArgs e;
  rc = resolve_epilogue(ctx, epi, ci->outChannels, &e);
  if (rc) return rc;
  o->version++;
  if (out_n == 0) return TFJS_CUDA_OK;
  cudaSetDevice(ctx->device);
  const float* wf;
  rc = float_view(ctx, w, &wf);
  if (rc) return rc;
  if (x->dtype == TFJS_F16 && o->dtype == TFJS_F16 && depthwise_half_native(*ci, e, x->ptr, wf, o->ptr))
    return launch_depthwise_image(ctx, x->ptr, wf, o->ptr, *ci, e, true);
  F32View xv;
  F32Out ov;
  rc = view_as_f32(ctx, x, &xv);
  if (!rc) rc = out_as_f32(ctx, o, &ov);
  if (!rc) rc = launch_depthwise(ctx, xv.ptr, wf, ov.ptr, *ci, e);
  release_view(ctx, &xv);
  return finish_out(ctx, &ov, rc);
}

extern "C" int tfjs_cuda_pool2d(tfjs_cuda_ctx* ctx, tfjs_tensor_id x_id, tfjs_tensor_id out_id,
                                const tfjs_conv2d_info* ci, int is_avg) {
  if (!ctx) return TFJS_CUDA_ERR_INVALID_ARG;
  int rc = check_conv_info(ctx, ci);
  if (rc) return rc;
  const int64_t out_n = (int64_t)ci->batchSize * ci->outHeight * ci->outWidth * ci->inChannels;
  TensorEntry *x, *o;
  rc = get_activation(ctx, x_id, (int64_t)ci->batchSize * ci->inHeight * ci->inWidth * ci->inChannels, "x", &x);
  if (rc) return rc;
  rc = get_activation(ctx, out_id, out_n, "pool output", &o);
  if (rc) return rc;
  o->version++;
  if (out_n == 0) return TFJS_CUDA_OK;
  cudaSetDevice(ctx->device);
  // the network's global average pool reads half storage directly (its result is float32)
  if (x->dtype == TFJS_F16 && o->dtype == TFJS_F32 && global_avgpool_half_supported(*ci, is_avg, x->ptr, o->ptr))
    return launch_global_avgpool_half(ctx, x->ptr, (float*)o->ptr, *ci);
  F32View xv;
  F32Out ov;
  rc = view_as_f32(ctx, x, &xv);
  if (!rc) rc = out_as_f32(ctx, o, &ov);
  if (!rc) rc = launch_pool2d(ctx, xv.ptr, ov.ptr, *ci, is_avg);
  release_view(ctx, &xv);
  return finish_out(ctx, &ov, rc);
}

// y = pw_act(conv1x1(dw_act(depthwise(x, dw_filter) + dw_bias), pw_filter) + pw_bias).  Shapes the
// fused tensor-core kernel takes run in one launch without the intermediate in device memory;
// everything else runs the depthwise and the pointwise kernel back to back through a scratch
// buffer.  Either way the arithmetic is that of the two separate calls.
extern "C" int tfjs_cuda_separable_conv2d(tfjs_cuda_ctx* ctx, tfjs_tensor_id x_id, tfjs_tensor_id dw_filter_id,
                                          tfjs_tensor_id pw_filter_id, tfjs_tensor_id out_id,
                                          const tfjs_conv2d_info* dw, int32_t out_channels,
                                          const tfjs_epilogue* dw_epi, const tfjs_epilogue* pw_epi) {
  if (!ctx) return TFJS_CUDA_ERR_INVALID_ARG;
  int rc = check_conv_info(ctx, dw);
  if (rc) return rc;
  TFJS_REQUIRE(ctx, out_channels >= 0, "negative extent");
  TFJS_REQUIRE(ctx, dw->inChannels == 0 || dw->outChannels % dw->inChannels == 0,
               "depthwise outChannels must be a multiple of inChannels");
  const int64_t pixels = (int64_t)dw->batchSize * dw->outHeight * dw->outWidth;
  const int64_t C = dw->outChannels, N = out_channels;
  TensorEntry *x, *wd, *wp, *o;
  rc = get_activation(ctx, x_id, (int64_t)dw->batchSize * dw->inHeight * dw->inWidth * dw->inChannels, "x", &x);
  if (rc) return rc;
  rc = get_f32(ctx, dw_filter_id, (int64_t)dw->filterHeight * dw->filterWidth * C, "depthwise filter", &wd);
  if (rc) return rc;
  rc = get_f32(ctx, pw_filter_id, C * N, "pointwise filter", &wp);
  if (rc) return rc;
  rc = get_activation(ctx, out_id, pixels * N, "separableConv2d output", &o);
  if (rc) return rc;
  EpilogueArgs de, pe;
  rc = resolve_epilogue(ctx, dw_epi, C, &de);
  if (rc) return rc;
  rc = resolve_epilogue(ctx, pw_epi, N, &pe);
  if (rc) return rc;
  o->version++;
  if (pixels * N == 0) return TFJS_CUDA_OK;
  cudaSetDevice(ctx->device);
  const float* wdf;
  rc = float_view(ctx, wd, &wdf);
  if (rc) return rc;
  TFJS_REQUIRE(ctx, C > 0, "separableConv2d needs at least one channel");
  const bool half = x->dtype == TFJS_F16 && o->dtype == TFJS_F16;
  // fuse_separable: 1 fuses where it measures faster than the two kernels (up to 128 channels, and
  // 256 channels at stride 1; at 256 channels and stride 2 the shared memory left beside the
  // weight stages holds too few input windows to cover the DRAM latency), 2 wherever it can
  const bool pays = C <= 128 || (C <= 256 && dw->strideHeight == 1);
  // The fused kernel gets its SAME padding from the zero fill of its window loads and multiplies
  // those zeros by the filter taps, where the reference skips taps outside the image
  // (backend_cpu.ts:2002-2014).  The two agree unless a tap is inf or NaN (0 * inf = NaN), so the
  // fused kernel is taken only for a filter the host wrote with finite values; any other filter
  // goes through the depthwise kernels, which skip those taps.
  // With half storage the arithmetic is TF32 whatever the math mode says: 16-bit storage is the
  // 16-bit precision class.
  const int fused_math = half ? TFJS_MATH_TF32 : ctx->math_mode;
  if ((half || (x->dtype == TFJS_F32 && o->dtype == TFJS_F32)) && ctx->use_tensor_cores && ctx->fuse_separable &&
      (ctx->fuse_separable >= 2 || pays) && known_finite(wd) &&
      sepconv_tcgen05_supported(*dw, N, de.activation, pe.activation, fused_math)) {
    PackedWeights pw;
    bool temporary;
    rc = packed_weights(ctx, wp, 0, C, N, false, true, &pw, &temporary);
    if (rc) return rc;
    return launch_sepconv_tcgen05(ctx, x->ptr, *dw, wdf, de, pw.hi, pw.kp, o->ptr, N, pe, half);
  }
  // Half storage, two kernels: whole-image depthwise into a half intermediate, f16 tensor-core GEMM.
  if (half && ctx->use_tensor_cores && pe.activation != TFJS_ACT_PRELU &&
      tcgen05_gemm_f16_supported(pixels, N, C, true)) {
    void* mid;
    size_t mid_cap;
    rc = ctx_alloc(ctx, (size_t)(pixels * C) * 2, &mid, &mid_cap);
    if (rc) return rc;
    if (depthwise_half_native(*dw, de, x->ptr, wdf, mid)) {
      rc = launch_depthwise_image(ctx, x->ptr, wdf, mid, *dw, de, true);
    } else {
      // no half depthwise kernel for this shape: float32 depthwise on a converted copy
      F32View xv;
      void* mid32 = nullptr;
      size_t mid32_cap = 0;
      rc = view_as_f32(ctx, x, &xv);
      if (!rc) rc = ctx_alloc(ctx, (size_t)(pixels * C) * 4, &mid32, &mid32_cap);
      if (!rc) rc = launch_depthwise(ctx, xv.ptr, wdf, (float*)mid32, *dw, de);
      if (!rc) rc = launch_convert(ctx, mid32, TFJS_F32, mid, TFJS_F16, pixels * C);
      release_view(ctx, &xv);
      if (mid32) ctx_free(ctx, mid32, mid32_cap);
    }
    if (!rc) {
      const void* plane;
      int64_t kp;
      rc = half_weights(ctx, wp, C, N, &plane, &kp);
      if (!rc) rc = launch_gemm_tcgen05_f16(ctx, mid, pixels, C, plane, kp, o->ptr, true, N, pe);
    }
    ctx_free(ctx, mid, mid_cap);
    return rc;
  }
  // float32 storage (or a mix of storages, through converted temporaries)
  F32View xv;
  F32Out ov;
  rc = view_as_f32(ctx, x, &xv);
  if (!rc) rc = out_as_f32(ctx, o, &ov);
  void* mid = nullptr;
  size_t mid_cap = 0;
  if (!rc) rc = ctx_alloc(ctx, (size_t)(pixels * C) * 4, &mid, &mid_cap);
  if (!rc) {
    // The intermediate is private to this call.  When a TF32 tensor-core GEMM reads it, the depthwise
    // kernel rounds its results to tf32 as it stores them (the fused kernel rounds the same values as
    // it builds its A tile), so the GEMM needs no rounding pass of its own.
    const bool round_mid = ctx->use_tensor_cores && ctx->math_mode == TFJS_MATH_TF32 &&
                           tcgen05_gemm_supported(pixels, N, C);
    de.round_tf32 = round_mid ? 1 : 0;
    rc = launch_depthwise(ctx, xv.ptr, wdf, (float*)mid, *dw, de);
    if (!rc)
      rc = gemm_dispatch(ctx, (const float*)mid, pixels, C, wp, 0, false, true, ov.ptr, N, pe, round_mid);
  }
  if (mid) ctx_free(ctx, mid, mid_cap);
  release_view(ctx, &xv);
  return finish_out(ctx, &ov, rc);
}
