// tfjs_cuda_matmul_static_scratch: the fused tensor-core matMul for callers that must not
// allocate device memory.
//
// The regular entry point (tfjs_cuda_batch_matmul) repacks the b operand into K-major tf32
// hi/lo planes held in buffers from the context's allocator.  Some callers cannot take that
// path: code that runs inside a region where cudaMalloc is forbidden or unaffordable (a
// latency-critical serving loop that has pre-sized every buffer, a host thread that shares the
// device with a framework whose memory pool must not be disturbed, a plugin that is handed raw
// device pointers and owns no allocator).  For them this variant keeps the repacked planes in a
// fixed array that is part of the library image itself, so the call touches no allocator at all:
// no cudaMalloc, no cudaFree, no caching pool, no tensor table.
//
// Costs and rules that follow from that choice:
//  - the array (two planes of kStaticPlaneFloats floats = 8 MiB) is resident on every GPU that
//    loads the library, from load until process exit;
//  - b is limited to n * round_up(k, 4) <= kStaticPlaneFloats elements; larger operands are
//    rejected with TFJS_CUDA_ERR_INVALID_ARG and a message that states the limit;
//  - all calls on a device share the one array.  It still holds the previous call's planes when
//    a call starts; this call overwrites every element it later reads (all n * kp entries of both
//    planes, the zero padding of columns k..kp included), so nothing has to be cleared.  Two
//    calls that overlap on the GPU (different streams or contexts of one device) race on the
//    array: serialise them;
//  - the first call on a device resolves the array's device address (cudaGetSymbolAddress, with
//    that device current).  Make that first call before any stream capture is started.
#include <atomic>

#include "common.cuh"

namespace {

constexpr int64_t kStaticPlaneFloats = 1 << 20;  // 1 Mi floats = 4 MiB per plane

// hi plane followed by lo plane.  In host code this name is only a handle for
// cudaGetSymbolAddress; it is not a device address.
static __device__ __align__(256) float g_static_planes[2 * kStaticPlaneFloats];

constexpr int kMaxDevices = 64;
// resolved device address, per device ordinal; atomic because contexts of different devices may
// be driven from different host threads (two threads resolving the same device store the same value)
std::atomic<float*> g_planes_addr[kMaxDevices];

// Once per device, with that device current.
int resolve_planes(tfjs_cuda_ctx* ctx, float** out) {
  TFJS_REQUIRE(ctx, ctx->device >= 0 && ctx->device < kMaxDevices, "device ordinal out of range");
  if (!g_planes_addr[ctx->device].load(std::memory_order_acquire)) {
    TFJS_CHECK_CUDA(ctx, cudaSetDevice(ctx->device));
    float* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&p, g_static_planes);
    if (e != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return set_error(ctx, TFJS_CUDA_ERR_CUDA, "cudaGetSymbolAddress(static scratch) failed: %s",
                       cudaGetErrorString(e));
    }
    g_planes_addr[ctx->device].store(p, std::memory_order_release);
  }
  *out = g_planes_addr[ctx->device].load(std::memory_order_acquire);
  return TFJS_CUDA_OK;
}

}  // namespace

extern "C" int tfjs_cuda_matmul_static_scratch(tfjs_cuda_ctx* ctx, const float* a, const float* b,
                                               const float* bias, float* out, int64_t m, int64_t k,
                                               int64_t n, int activation, float clip_lo,
                                               float clip_hi) {
  if (!ctx) return TFJS_CUDA_ERR_INVALID_ARG;
  TFJS_REQUIRE(ctx, m >= 0 && k >= 0 && n >= 0, "negative extent");
  TFJS_REQUIRE(ctx, activation == TFJS_ACT_LINEAR || activation == TFJS_ACT_RELU ||
                        activation == TFJS_ACT_CLIP,
               "activation must be linear, relu or clip");
  if (m * n == 0) return TFJS_CUDA_OK;
  TFJS_REQUIRE(ctx, a && b && out, "a, b and out must be device pointers");
  TFJS_REQUIRE(ctx, ctx->device >= 0 && ctx->device < kMaxDevices, "device ordinal out of range");
  TFJS_REQUIRE(ctx, !ctx->capturing || g_planes_addr[ctx->device].load(std::memory_order_acquire),
               "make the first call on a device before starting a stream capture");
  const int64_t kp = (k + 3) / 4 * 4;
  if (n * kp > kStaticPlaneFloats)
    return set_error(ctx, TFJS_CUDA_ERR_INVALID_ARG,
                     "b is too large for the static scratch: n * round_up(k, 4) = %lld exceeds the "
                     "limit of %lld elements; use tfjs_cuda_batch_matmul instead",
                     (long long)(n * kp), (long long)kStaticPlaneFloats);
  if (!tcgen05_gemm_supported(m, n, k))
    return set_error(ctx, TFJS_CUDA_ERR_UNSUPPORTED,
                     "shape %lld x %lld x %lld is not a tensor-core shape (k and n must be multiples "
                     "of 4, n >= 8)", (long long)m, (long long)k, (long long)n);
  TFJS_REQUIRE(ctx, (((uintptr_t)a | (uintptr_t)out) & 15) == 0, "a and out must be 16-byte aligned");
  float* planes = nullptr;
  int rc = resolve_planes(ctx, &planes);
  if (rc) return rc;
  cudaSetDevice(ctx->device);
  float* hi = planes;
  float* lo = planes + kStaticPlaneFloats;
  // b is [k, n] row-major.  Every element of hi/lo[0 .. n*kp) is written here.
  rc = launch_pack_weights(ctx, b, false, 0.0, 0.0, k, n, n, 1, kp, hi, lo);
  if (rc) return rc;
  EpilogueArgs e;
  e.bias = bias;
  e.activation = activation;
  e.clip_lo = clip_lo;
  e.clip_hi = clip_hi;
  return launch_gemm_tcgen05(ctx, a, m, k, hi, lo, kp, out, n, e, ctx->math_mode);
}
