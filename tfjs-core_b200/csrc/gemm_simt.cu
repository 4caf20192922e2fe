// CUDA-core GEMM for shapes the tensor-core kernel does not take, plus the operand
// preparation kernels (weight repacking with tf32 hi/lo split, batched transpose).
#include <cuda_fp16.h>

#include "common.cuh"

namespace {

// ---- fp32 GEMM with arbitrary operand strides ------------------------------------------------
// out[b, i, j] = epilogue(sum_k a[b, i, k] * b[b, k, j]).  64x64 tile, 16-deep k slices in
// shared memory, 4x4 outputs per thread, fmaf in ascending k.  Handles every transpose
// combination of batchMatMul (backend_cpu.ts:491-540) through the strides.
constexpr int TM = 64, TN = 64, TK = 16;

__global__ void __launch_bounds__(256)
gemm_simt_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out,
                 int M, int N, int K, int64_t a_batch, int64_t a_row, int64_t a_col,
                 int64_t b_batch, int64_t b_row, int64_t b_col, EpilogueArgs epi) {
  __shared__ float as[TK][TM + 1];
  __shared__ float bs[TK][TN + 1];
  const int bz = blockIdx.z;
  const int m0 = blockIdx.x * TM, n0 = blockIdx.y * TN;  // M tiles on x: up to 2^31 - 1 of them
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const float* ab = a + bz * a_batch;
  const float* bb = b + bz * b_batch;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += TK) {
    for (int i = threadIdx.x; i < TM * TK; i += 256) {
      // pick the faster-varying index along the contiguous dimension of each operand
      int kk, mm;
      if (a_col == 1) { kk = i % TK; mm = i / TK; } else { mm = i % TM; kk = i / TM; }
      const int gm = m0 + mm, gk = k0 + kk;
      as[kk][mm] = (gm < M && gk < K) ? ab[gm * a_row + gk * a_col] : 0.f;
    }
    for (int i = threadIdx.x; i < TN * TK; i += 256) {
      int kk, nn;
      if (b_col == 1) { nn = i % TN; kk = i / TN; } else { kk = i % TK; nn = i / TK; }
      const int gn = n0 + nn, gk = k0 + kk;
      bs[kk][nn] = (gn < N && gk < K) ? bb[gk * b_row + gn * b_col] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; kk++) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; i++) av[i] = as[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; j++) bv[j] = bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
  float* ob = out + (int64_t)bz * M * N;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int gn = n0 + tx * 4 + j;
      if (gn < N) ob[(int64_t)gm * N + gn] = apply_epilogue(acc[i][j], gn, epi);
    }
  }
}

// ---- weight repacking ------------------------------------------------------------------------
// Source: a [K, N] matrix addressed through (k_stride, n_stride), float32 or uint8 affine
// quantised (w = q*scale + min evaluated in float64, io_utils.ts:139).  Destination: K-major
// planes [N, kp]: hi = tf32(w) rounded to nearest, lo = tf32(w - hi); columns k >= K are zero.
// 32x32 shared-memory tile so that both the read and the write are coalesced.
__global__ void pack_weights_kernel(const void* __restrict__ src, int src_is_u8, double scale,
                                    double mn, int K, int N, int64_t k_stride, int64_t n_stride,
                                    int kp, float* __restrict__ hi, float* __restrict__ lo) {
  __shared__ float tile[32][33];
  const int k0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    int k, n;
    if (n_stride == 1) { k = k0 + r; n = n0 + threadIdx.x; } else { n = n0 + r; k = k0 + threadIdx.x; }
    float v = 0.f;
    if (k < K && n < N) {
      const int64_t off = k * k_stride + n * n_stride;
      v = src_is_u8 ? (float)((double)((const uint8_t*)src)[off] * scale + mn)
                    : ((const float*)src)[off];
    }
    tile[k - k0][n - n0] = v;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int n = n0 + r, k = k0 + threadIdx.x;
    if (n < N && k < kp) {
      const float v = tile[threadIdx.x][r];
      const float h = round_tf32(v);
      hi[(int64_t)n * kp + k] = h;
      // A non-finite hi would turn the residual into NaN (inf - inf); keep it zero instead.
      if (lo) lo[(int64_t)n * kp + k] = (fabsf(h) <= 3.4028234e38f) ? round_tf32(v - h) : 0.f;
    }
  }
}

// The same source as one K-major IEEE half plane [N, kp] (round to nearest even), for the
// kind::f16 tensor-core kernel.
__global__ void pack_weights_f16_kernel(const void* __restrict__ src, int src_is_u8, double scale, double mn,
                                        int K, int N, int64_t k_stride, int64_t n_stride, int kp,
                                        __half* __restrict__ dst) {
  __shared__ float tile[32][33];
  const int k0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    int k, n;
    if (n_stride == 1) { k = k0 + r; n = n0 + threadIdx.x; } else { n = n0 + r; k = k0 + threadIdx.x; }
    float v = 0.f;
    if (k < K && n < N) {
      const int64_t off = k * k_stride + n * n_stride;
      v = src_is_u8 ? (float)((double)((const uint8_t*)src)[off] * scale + mn) : ((const float*)src)[off];
    }
    tile[k - k0][n - n0] = v;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int n = n0 + r, k = k0 + threadIdx.x;
    if (n < N && k < kp) dst[(int64_t)n * kp + k] = __float2half_rn(tile[threadIdx.x][r]);
  }
}

// Repack for the Cin == 3 implicit-GEMM gather: destination column k' = wr * row_pad + j holds
// source row k = wr * row_len + j for j < row_len and zero otherwise (each filter row of
// row_len = fW * Cin values is padded to row_pad).  The operand is tiny (27 x N), one thread per
// destination element.
__global__ void pack_weights_rows_kernel(const void* __restrict__ src, int src_is_u8, double scale,
                                         double mn, int K, int N, int row_len, int row_pad, int kp,
                                         float* __restrict__ hi, float* __restrict__ lo) {
  const int64_t total = (int64_t)N * kp;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int n = (int)(i / kp), kd = (int)(i % kp);
    const int wr = kd / row_pad, j = kd % row_pad;
    const int k = wr * row_len + j;
    float v = 0.f;
    if (j < row_len && k < K) {
      const int64_t off = (int64_t)k * N + n;
      v = src_is_u8 ? (float)((double)((const uint8_t*)src)[off] * scale + mn) : ((const float*)src)[off];
    }
    const float h = round_tf32(v);
    hi[i] = h;
    if (lo) lo[i] = (fabsf(h) <= 3.4028234e38f) ? round_tf32(v - h) : 0.f;
  }
}

// uint8 [K, N] (addressed through strides) -> K-major uint8 [N, kq], zero padded in k.
__global__ void pack_u8_kernel(const uint8_t* __restrict__ src, int K, int N, int64_t k_stride,
                               int64_t n_stride, int kq, uint8_t* __restrict__ dst) {
  __shared__ uint8_t tile[32][33];
  const int k0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    int k, n;
    if (n_stride == 1) { k = k0 + r; n = n0 + threadIdx.x; } else { n = n0 + r; k = k0 + threadIdx.x; }
    tile[k - k0][n - n0] = (k < K && n < N) ? src[k * k_stride + n * n_stride] : (uint8_t)0;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int n = n0 + r, k = k0 + threadIdx.x;
    if (n < N && k < kq) dst[(int64_t)n * kq + k] = tile[threadIdx.x][r];
  }
}

// dst[b, c, r] = src[b, r, c]
__global__ void transpose_batched_kernel(const float* __restrict__ src, float* __restrict__ dst,
                                         int rows, int cols) {
  __shared__ float tile[32][33];
  const int64_t base = (int64_t)blockIdx.z * rows * cols;
  const int r0 = blockIdx.y * 32, c0 = blockIdx.x * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int gr = r0 + r, gc = c0 + threadIdx.x;
    if (gr < rows && gc < cols) tile[r][threadIdx.x] = src[base + (int64_t)gr * cols + gc];
  }
  __syncthreads();
  for (int c = threadIdx.y; c < 32; c += blockDim.y) {
    const int gc = c0 + c, gr = r0 + threadIdx.x;
    if (gr < rows && gc < cols) dst[base + (int64_t)gc * rows + gr] = tile[threadIdx.x][c];
  }
}

}  // namespace

int launch_gemm_simt(tfjs_cuda_ctx* ctx, const float* a, const float* b, float* out, int batch,
                     int M, int N, int K, int64_t a_batch, int64_t a_row, int64_t a_col,
                     int64_t b_batch, int64_t b_row, int64_t b_col, const EpilogueArgs& epi) {
  if ((int64_t)batch * M * N == 0) return TFJS_CUDA_OK;
  // row tiles on grid.x (a pointwise convolution over a large batch has millions of rows: M / 64
  // exceeds the 65535 limit of grid.y), column tiles on grid.y
  dim3 grid((M + TM - 1) / TM, (N + TN - 1) / TN, batch);
  if (grid.y > 65535 || grid.z > 65535)
    return set_error(ctx, TFJS_CUDA_ERR_UNSUPPORTED, "matrix too large for the CUDA-core GEMM");
  gemm_simt_kernel<<<grid, 256, 0, ctx->stream>>>(a, b, out, M, N, K, a_batch, a_row, a_col, b_batch,
                                                  b_row, b_col, epi);
  return post_launch(ctx, "batchMatMul (CUDA cores)");
}

int launch_pack_weights_f16(tfjs_cuda_ctx* ctx, const void* src, bool src_is_u8, double scale, double mn,
                            int64_t K, int64_t N, int64_t src_k_stride, int64_t src_n_stride, int64_t kp,
                            void* dst) {
  if (N * kp == 0) return TFJS_CUDA_OK;
  dim3 grid((unsigned)ceil_div64(N, 32), (unsigned)ceil_div64(kp, 32));
  pack_weights_f16_kernel<<<grid, dim3(32, 8), 0, ctx->stream>>>(src, src_is_u8 ? 1 : 0, scale, mn, (int)K, (int)N,
                                                                 src_k_stride, src_n_stride, (int)kp, (__half*)dst);
  return post_launch(ctx, "pack_weights (float16)");
}

int launch_pack_weights(tfjs_cuda_ctx* ctx, const void* src, bool src_is_u8, double scale,
                        double mn, int64_t K, int64_t N, int64_t src_k_stride, int64_t src_n_stride,
                        int64_t kp, float* hi, float* lo) {
  if (N * kp == 0) return TFJS_CUDA_OK;
  dim3 grid((unsigned)ceil_div64(N, 32), (unsigned)ceil_div64(kp, 32));
  pack_weights_kernel<<<grid, dim3(32, 8), 0, ctx->stream>>>(src, src_is_u8 ? 1 : 0, scale, mn, (int)K,
                                                             (int)N, src_k_stride, src_n_stride,
                                                             (int)kp, hi, lo);
  return post_launch(ctx, "pack_weights");
}

int launch_pack_weights_rows(tfjs_cuda_ctx* ctx, const void* src, bool src_is_u8, double scale, double mn,
                             int64_t K, int64_t N, int row_len, int row_pad, int64_t kp, float* hi,
                             float* lo) {
  if (N * kp == 0) return TFJS_CUDA_OK;
  const int blocks = (int)((N * kp + 255) / 256);
  pack_weights_rows_kernel<<<blocks > 1024 ? 1024 : blocks, 256, 0, ctx->stream>>>(
      src, src_is_u8 ? 1 : 0, scale, mn, (int)K, (int)N, row_len, row_pad, (int)kp, hi, lo);
  return post_launch(ctx, "pack_weights (rows)");
}

int launch_pack_u8(tfjs_cuda_ctx* ctx, const uint8_t* src, int64_t K, int64_t N, int64_t k_stride,
                   int64_t n_stride, int64_t kq, uint8_t* dst) {
  if (N * kq == 0) return TFJS_CUDA_OK;
  dim3 grid((unsigned)ceil_div64(N, 32), (unsigned)ceil_div64(kq, 32));
  pack_u8_kernel<<<grid, dim3(32, 8), 0, ctx->stream>>>(src, (int)K, (int)N, k_stride, n_stride, (int)kq, dst);
  return post_launch(ctx, "pack_weights (uint8)");
}

int launch_transpose_batched(tfjs_cuda_ctx* ctx, const float* src, float* dst, int batch, int rows,
                             int cols) {
  if ((int64_t)batch * rows * cols == 0) return TFJS_CUDA_OK;
  dim3 grid((cols + 31) / 32, (rows + 31) / 32, batch);
  transpose_batched_kernel<<<grid, dim3(32, 8), 0, ctx->stream>>>(src, dst, rows, cols);
  return post_launch(ctx, "transpose");
}
