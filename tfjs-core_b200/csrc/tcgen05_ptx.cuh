// Device-side building blocks shared by the tcgen05 kernels: mbarrier / TMA / tcgen05 PTX
// wrappers with bounded waits, shared-memory and instruction descriptors for K-major
// SWIZZLE_128B tf32 operands, the epilogue arithmetic, and the host-side tensor-map encoder.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace {

// Upper bound of every mbarrier wait, in SM clock cycles (~2 s at 1.9 GHz by default).  The
// context option "wait_limit_us" rewrites it; each translation unit that includes this header has
// its own copy, set through set_wait_limit_here().
__constant__ long long g_wait_limit_cycles = 4000000000LL;
#define WAIT_LIMIT_CYCLES g_wait_limit_cycles

inline int set_wait_limit_here(long long cycles) {
  return cudaMemcpyToSymbol(g_wait_limit_cycles, &cycles, sizeof(cycles)) == cudaSuccess ? 0 : -1;
}

// ---- PTX wrappers ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}
// Non-blocking test, for a thread that polls several barriers in turn.
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}
// Bounded wait.  Returns false (and records `code` in the status word) when the barrier did
// not complete within WAIT_LIMIT_CYCLES or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (uint32_t it = 0;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (it > 8) __nanosleep(20);  // leave the issue slots to the warps that have work
    if ((it & 63) == 63) {
      if (*abort_flag) return false;
      if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
        *abort_flag = 1;
        atomicCAS(status, 0, code);
        return false;
      }
    }
  }
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
// Brings a tensor map (a kernel parameter) into the descriptor cache ahead of its first use, so
// that the first load does not wait for the fetch; issued by one thread at kernel start.
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
// Asks the TMA unit to bring a tile into L2 only (no shared memory, no barrier): issued a few
// k-blocks ahead of the real load, it turns that load's DRAM latency into an L2 hit.
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* map, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];" ::"l"(map), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map),
               "r"(src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
// D[tmem] (+)= A[smem] * B[smem], tf32 inputs, fp32 accumulate.
__device__ __forceinline__ void tcgen05_mma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                                 uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Same with IEEE half inputs: A and B tiles hold 16-bit elements, K = 16 per instruction.
__device__ __forceinline__ void tcgen05_mma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                                uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte rows, SWIZZLE_128B, 8-row groups
// 1024 bytes apart.  Bit layout: start address >> 4 in [0,14), leading byte offset >> 4 in
// [16,30) (unused for swizzled K-major), stride byte offset >> 4 in [32,46), descriptor
// version 1 in [46,48), layout type 2 (SWIZZLE_128B) in [61,64).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Instruction descriptor for kind::tf32: D format f32 (1) in [4,6), A and B format tf32 (2) in
// [7,10) and [10,13), both operands K-major (bits 15, 16 = 0), N >> 3 in [17,23), M >> 4 in
// [24,29).
__host__ __device__ constexpr uint32_t make_idesc(int m, int n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// Instruction descriptor for kind::f16 with IEEE half operands: D format f32 (1) in [4,6), A and B
// format f16 (0) in [7,10) and [10,13), both K-major, N >> 3 in [17,23), M >> 4 in [24,29).
__host__ __device__ constexpr uint32_t make_idesc_f16(int m, int n) {
  return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// Bias and activation of one 32x32 output chunk in registers: thread `lane` owns row `lane`,
// v[] holds its 32 accumulator columns.  Arithmetic order follows MathBackendCPU's unfused
// passes: float32(acc) + bias, then the activation (backend_cpu.ts:542-555).  relu is
// Math.max(0, x) and clip is `x > hi ? hi : (x < lo ? lo : x)`: both keep NaN, which the
// NaN-propagating min/max reproduce.  bias_s/alpha_s are this warp's 32 staged values in shared
// memory, read as broadcast float4.  Columns beyond N carry meaningless values; the TMA store
// clips them.
template <int ACT>
__device__ __forceinline__ void finish_chunk(float (&v)[32], bool has_bias, const float* bias_s,
                                             const float* alpha_s, const EpilogueArgs& e) {
#pragma unroll
  for (int j = 0; j < 8; j++) {
    if (has_bias) {
      const float4 b = *reinterpret_cast<const float4*>(bias_s + j * 4);
      v[j * 4 + 0] += b.x;
      v[j * 4 + 1] += b.y;
      v[j * 4 + 2] += b.z;
      v[j * 4 + 3] += b.w;
    }
    if (ACT == TFJS_ACT_PRELU) {
      const float4 a = *reinterpret_cast<const float4*>(alpha_s + j * 4);
      v[j * 4 + 0] = (v[j * 4 + 0] < 0.f) ? a.x * v[j * 4 + 0] : v[j * 4 + 0];
      v[j * 4 + 1] = (v[j * 4 + 1] < 0.f) ? a.y * v[j * 4 + 1] : v[j * 4 + 1];
      v[j * 4 + 2] = (v[j * 4 + 2] < 0.f) ? a.z * v[j * 4 + 2] : v[j * 4 + 2];
      v[j * 4 + 3] = (v[j * 4 + 3] < 0.f) ? a.w * v[j * 4 + 3] : v[j * 4 + 3];
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
      if (ACT == TFJS_ACT_RELU) v[j * 4 + i] = max_nan(v[j * 4 + i], 0.f);
      if (ACT == TFJS_ACT_CLIP) v[j * 4 + i] = min_nan(max_nan(v[j * 4 + i], e.clip_lo), e.clip_hi);
    }
  }
}

// Two float32 -> one word of two IEEE halves (round to nearest even), low half first.
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
// One word of two IEEE halves -> two float32 (exact).
__device__ __forceinline__ void unpack_half2(uint32_t h, float& lo, float& hi) {
  asm("{\n\t.reg .b16 a, b;\n\tmov.b32 {a, b}, %2;\n\tcvt.f32.f16 %0, a;\n\tcvt.f32.f16 %1, b;\n\t}"
      : "=f"(lo), "=f"(hi)
      : "r"(h));
}

__device__ __forceinline__ void cp_async_16_zfill(uint32_t dst, const void* src, bool valid) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(valid ? 16 : 0)
               : "memory");
}
__device__ __forceinline__ void cp_async_8_zfill(uint32_t dst, const void* src, bool valid) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(dst), "l"(src), "r"(valid ? 8 : 0)
               : "memory");
}
__device__ __forceinline__ void cp_async_4_zfill(uint32_t dst, const void* src, bool valid) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(valid ? 4 : 0)
               : "memory");
}
// Packed pairs of float32 (sm_100 f32x2 arithmetic): one instruction per two elements.
__device__ __forceinline__ uint64_t pack_f32x2(uint32_t lo, uint32_t hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, uint32_t& lo, uint32_t& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}

// Byte offset `o` (multiple of 4) of row `r` in a SWIZZLE_128B K-major tile.
__device__ __forceinline__ uint32_t swz(int r, int o) {
  return (uint32_t)(r * 128 + ((((o >> 4) ^ (r & 7)) << 4) | (o & 15)));
}


}  // namespace

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda).
// dims / box are innermost first; strides_bytes has rank - 1 entries (the innermost stride is the
// element size).  Out-of-range elements of a load read as zero.  False when the driver symbol is
// missing or the encode fails.
bool tma_encode_tiled(CUtensorMap* map, CUtensorMapDataType dtype, int rank, const void* base,
                      const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                      CUtensorMapSwizzle swizzle);
