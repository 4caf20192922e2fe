// Tensor-core GEMM for sm_100a: out[M, N] = act(A[M, K] * W[K, N] + bias[N]), float32 in and
// out, TF32 (one pass) or 3xTF32 (three passes on hi/lo splits) on tcgen05 with the
// accumulator in tensor memory.
//
// This is the kernel behind KernelBackend.fusedBatchMatMul and the 1x1 fusedConv2d
// (tfjs-core/src/backends/backend.ts:134-138, 414-418): a pointwise convolution over NHWC is
// the GEMM [B*H*W, Cin] x [Cin, Cout].
//
// Structure (one persistent CTA per SM, warp specialised):
//   warp 8      TMA producer: A tile [128 x 32] and W tile(s) [BLOCK_N x 32] per k-block into a
//               ring of shared-memory stages (SWIZZLE_128B, K-major), mbarrier complete_tx.
//   warps 10-13 (3xTF32 only) split the A stage in place: hi = tf32(a), lo = tf32(a - hi).
//   warp 9      MMA issuer: one thread issues tcgen05.mma (M=128, N=BLOCK_N, K=8) per 32-byte
//               k-step, commits stage release and accumulator-ready barriers.
//   warps 0-7   epilogue: tcgen05.ld the accumulator (two TMEM buffers, so the next tile's
//               MMAs overlap), add bias, apply the activation, stage through swizzled shared
//               memory and write with TMA stores (which clip the M and N tails).
// Every mbarrier wait is bounded; a wait that gives up sets the context's status word and the
// CTA drains and frees its tensor memory.
#include <atomic>

#include "tcgen05_ptx.cuh"

namespace {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 32;                        // 32 fp32 = 128 bytes = one swizzle row
constexpr int A_STAGE_BYTES = BLOCK_M * BLOCK_K * 4;  // 16 KB
constexpr int C_CHUNK_BYTES = 32 * 32 * 4;         // one warp's 32x32 output chunk
constexpr int EPI_WARPS = 8;                      // two warps per TMEM lane quarter
constexpr int C_STAGING_BYTES = EPI_WARPS * C_CHUNK_BYTES;
constexpr int BIAS_STAGING_BYTES = EPI_WARPS * 256;  // per warp: 32 bias values + 32 prelu slopes
constexpr int SMEM_LIMIT = 232448;                 // 227 KB
constexpr int BARRIER_BYTES = 1024;
constexpr int LUT_BYTES = 2048;  // uint8 weights: 256 dequantised tf32 hi values + 256 lo values

constexpr int WQ_SLOTS = 2;  // uint8 weights: ring of dequantised weight tiles
__host__ __device__ constexpr int stage_bytes(int block_n, bool split, bool wq = false) {
  // wq: a stage holds the A tile and the raw uint8 weight tile (block_n rows of 32 bytes); the
  // dequantised tf32 tiles live in their own short ring, so that many small stages can be in
  // flight while only WQ_SLOTS expanded tiles take up shared memory
  return wq ? A_STAGE_BYTES * (split ? 2 : 1) + block_n * BLOCK_K
            : (A_STAGE_BYTES + block_n * BLOCK_K * 4) * (split ? 2 : 1);
}
__host__ __device__ constexpr int wq_ring_bytes(int block_n, bool split, bool wq) {
  return wq ? WQ_SLOTS * block_n * BLOCK_K * 4 * (split ? 2 : 1) + LUT_BYTES : 0;
}
// The ring takes everything the 227 KB allow.  No room is set aside for aligning the dynamic
// shared-memory window to 1024 bytes (which SWIZZLE_128B tiles need): the window of a kernel
// without static shared memory starts 1024-aligned, the launch asks for up to 1 KB of slack where
// the layout leaves it, and a CTA that finds it would not fit reports STATUS_SMEM_LAYOUT and
// returns before touching anything.  At BLOCK_N = 256 this is the difference between 3 and 4
// stages of 48 KB, i.e. a third more bytes in flight on the layers that are bound by load latency.
__host__ __device__ constexpr int num_stages(int block_n, bool split, bool wq = false) {
  int s = (SMEM_LIMIT - C_STAGING_BYTES - BIAS_STAGING_BYTES - BARRIER_BYTES -
           wq_ring_bytes(block_n, split, wq)) / stage_bytes(block_n, split, wq);
  return s > 8 ? 8 : s;
}
__host__ __device__ constexpr int layout_bytes(int block_n, bool split, bool wq) {
  return wq_ring_bytes(block_n, split, wq) + num_stages(block_n, split, wq) * stage_bytes(block_n, split, wq) +
         C_STAGING_BYTES + BIAS_STAGING_BYTES + BARRIER_BYTES;
}

// Geometry of an implicit-GEMM convolution: row m of the A matrix is output pixel
// (b, yo, xo) = unflatten(m), column kk is filter tap (wr, wc) and input channel ci.
struct ConvGeom {
  const float* x;
  int inH, inW, Cin, outH, outW;
  int sH, sW, dH, dW, padT, padL, fH, fW;
};

struct GemmParams {
  int M, N, K;
  int num_m_tiles, num_n_tiles, num_k_blocks;
  int* status;
  EpilogueArgs epi;
  ConvGeom conv;  // AMODE != A_MATRIX only
  double q_scale, q_min;  // WQ only: w = q * q_scale + q_min, evaluated in float64
  // WQ, TF32: set when the host has checked, for all 256 byte values, that one float32 fma
  // followed by the tf32 rounding gives the same bits as the float64 evaluation
  float q_scale32, q_min32;
  int q_arith;
  // diagnostic: the producer does not issue the loads of its last k-block, so the consumers'
  // bounded waits run out (nothing is left in flight, the kernel gives up cleanly)
  int withhold_last_load;
};

// How the A operand reaches shared memory.
constexpr int A_MATRIX = 0;     // dense [M, K] matrix, TMA
constexpr int A_CONV_VEC = 1;   // NHWC image, Cin % 4 == 0: 16-byte cp.async gathers, K = (wr, wc, ci)
constexpr int A_CONV_RGB = 2;   // NHWC image, Cin == 3, 3 columns wide filter: one 32-wide k-block,
                                // K' = wr * 10 + wc * 3 + ci (each filter row padded to 10 floats so
                                // that its 36 contiguous source bytes can move as 8-byte pieces)

// WQ: the weights arrive as raw uint8 affine-quantised bytes (K-major [N, Kq], map_w_hi is a
// uint8 tensor map) and are dequantised in shared memory by the converter warps, k-block by
// k-block, inside the main loop: w = float32(float64(q) * scale + min) (io_utils.ts:139), then
// the tf32 hi (/lo) split straight into the swizzled operand tile the tensor core reads.
// Threads per CTA: 10 warps, plus 4 converter / gather warps, or 8 converter warps when the
// weights are dequantised in the loop.
// `converts`: the A stage is rewritten in shared memory before the tensor core reads it (3xTF32
// split, or round-to-nearest of a TF32 operand), which takes the four helper warps.
__host__ __device__ constexpr int cta_threads(bool converts, int amode, bool wq) {
  return wq ? 576 : ((converts || amode != A_MATRIX) ? 448 : 320);
}

// How the A operand is prepared for the tensor core, which reads the upper 19 bits of each
// float32 (sign, exponent, 10 mantissa bits) and so TRUNCATES whatever it is given:
constexpr int PREC_TF32_ASIS = 0;   // one pass; the caller guarantees A holds tf32-exact values
                                    // (low 13 mantissa bits zero), e.g. a producer kernel rounded
                                    // them, or (conv modes) the gather threads round each row
constexpr int PREC_3XTF32 = 1;      // hi = rna(a), lo = rna(a - hi); three passes
constexpr int PREC_TF32_ROUND = 2;  // one pass; helper warps round A to nearest (ties away) in
                                    // shared memory first, so that the operand error is unbiased
constexpr int PREC_F16 = 3;         // A and W are IEEE half matrices (16-bit activation storage): one
                                    // kind::f16 pass, a k-block is 64 elements (the same 128-byte rows)

// cta_threads' first argument: does the variant rewrite its A stages in shared memory
__host__ __device__ constexpr bool converts_a(int prec) { return prec == PREC_3XTF32 || prec == PREC_TF32_ROUND; }

// OUT16: the result is stored as IEEE half (rows of a 32-column chunk are 64 bytes, unswizzled)
template <int BLOCK_N, int PREC, int AMODE, bool WQ, bool OUT16 = false>
__global__ void __launch_bounds__(cta_threads(converts_a(PREC), AMODE, WQ), 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a,
                    const __grid_constant__ CUtensorMap map_w_hi,
                    const __grid_constant__ CUtensorMap map_w_lo,
                    const __grid_constant__ CUtensorMap map_c, GemmParams p) {
  static_assert(!WQ || AMODE == A_MATRIX, "in-loop dequantisation is implemented for the matrix mode");
  static_assert(PREC != PREC_TF32_ROUND || AMODE == A_MATRIX, "the gather threads of the conv modes round their own rows");
  static_assert(PREC != PREC_F16 || (AMODE == A_MATRIX && !WQ), "half operands: dense matrix mode only");
  static_assert(!OUT16 || PREC == PREC_F16, "half output goes with half operands");
  constexpr bool SPLIT = PREC == PREC_3XTF32;
  constexpr bool ROUND = PREC == PREC_TF32_ROUND;
  constexpr bool HALF = PREC == PREC_F16;
  constexpr int KB_ELEMS = HALF ? 64 : BLOCK_K;  // elements per k-block: 128 bytes either way
  constexpr int STAGES = num_stages(BLOCK_N, SPLIT, WQ);
  constexpr int NCONV = cta_threads(converts_a(PREC), AMODE, WQ) - 320;  // converter (or gather) threads
  constexpr int B_STAGE_BYTES = BLOCK_N * BLOCK_K * 4;
  constexpr int Q_STAGE_BYTES = BLOCK_N * BLOCK_K;  // uint8 tile
  // Two accumulator buffers (the epilogue drains one while the MMAs fill the other).  In 3xTF32
  // each buffer is a pair: the hi*hi products accumulate in one tile and the small lo*hi + hi*lo
  // correction terms in another, and the epilogue adds the two in float32.  The tensor core
  // truncates when it aligns an addend to the running sum, so keeping the corrections out of the
  // large sum removes two thirds of those truncations from it.
  constexpr int ACC_COLS = SPLIT ? 2 * BLOCK_N : BLOCK_N;  // TMEM columns per buffer
  constexpr uint32_t TMEM_COLS = 2 * ACC_COLS;             // a power of two >= 64
  static_assert(TMEM_COLS <= 512, "tensor memory has 512 columns");
  constexpr uint32_t TX_BYTES = (AMODE == A_MATRIX ? A_STAGE_BYTES : 0) +
                                (WQ ? Q_STAGE_BYTES : B_STAGE_BYTES * (SPLIT ? 2 : 1));
  static_assert(STAGES >= 2, "pipeline needs at least two stages");

  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment by an offset on the __shared__ array itself: the pointers derived from
  // it stay in the shared address space (an integer round trip would make every access generic)
  const uint32_t align_pad = (1024u - (smem_u32(smem_raw) & 1023u)) & 1023u;
  {
    uint32_t window;
    asm("mov.u32 %0, %%dynamic_smem_size;" : "=r"(window));
    if (align_pad + (uint32_t)layout_bytes(BLOCK_N, SPLIT, WQ) > window) {  // uniform over the CTA
      if (threadIdx.x == 0) atomicCAS(p.status, 0, STATUS_SMEM_LAYOUT);
      return;
    }
  }
  uint8_t* smem = smem_raw + align_pad;
  uint8_t* a_hi = smem;
  uint8_t* a_lo = a_hi + STAGES * A_STAGE_BYTES;  // SPLIT only
  // tf32 weight tiles: one per stage, or (WQ) a ring of WQ_SLOTS tiles filled by the converters
  constexpr int B_TILES = WQ ? WQ_SLOTS : STAGES;
  uint8_t* b_hi = a_hi + STAGES * A_STAGE_BYTES * (SPLIT ? 2 : 1);
  uint8_t* b_lo = b_hi + B_TILES * B_STAGE_BYTES;  // SPLIT only
  uint8_t* b_q = b_hi + B_TILES * B_STAGE_BYTES * (SPLIT ? 2 : 1);  // WQ only: raw bytes per stage
  uint8_t* c_stage = b_q + (WQ ? STAGES * Q_STAGE_BYTES : 0);
  uint8_t* bias_stage = c_stage + C_STAGING_BYTES;
  uint64_t* bars = (uint64_t*)(bias_stage + BIAS_STAGING_BYTES);
  uint64_t* full_bar = bars;                  // [STAGES] TMA -> consumers
  uint64_t* empty_bar = bars + STAGES;        // [STAGES] MMA -> TMA
  uint64_t* conv_bar = bars + 2 * STAGES;     // [STAGES] converters -> MMA (SPLIT)
  uint64_t* tmem_full_bar = bars + 3 * STAGES;   // [2] MMA -> epilogue
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;  // [2] epilogue -> MMA
  uint64_t* slot_full_bar = tmem_empty_bar + 2;  // [WQ_SLOTS] converters -> MMA (WQ)
  uint64_t* slot_empty_bar = slot_full_bar + WQ_SLOTS;  // [WQ_SLOTS] MMA -> converters (WQ)
  uint32_t* tmem_ptr_holder = (uint32_t*)(slot_empty_bar + WQ_SLOTS);
  volatile int* abort_flag = (volatile int*)(tmem_ptr_holder + 1);
  float* lut_hi = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + BARRIER_BYTES);  // WQ only
  float* lut_lo = lut_hi + 256;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.num_m_tiles * p.num_n_tiles;
  if (threadIdx.x == 32 * 8) {  // the producer warp's first lane: descriptors on their way before the set-up below
    if (AMODE == A_MATRIX) prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_w_hi);
    if (SPLIT) prefetch_tensormap(&map_w_lo);
    prefetch_tensormap(&map_c);
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      // the TMA producer's expect_tx arrival, plus one arrival per gather thread in conv modes (a
      // thread hands its row over as soon as its own copies have landed; one arrival per warp
      // would make every row wait for the slowest of its warp and measured 7 % slower)
      mbar_init(smem_u32(&full_bar[s]), AMODE == A_MATRIX ? 1 : 129);
      mbar_init(smem_u32(&empty_bar[s]), 1);
      mbar_init(smem_u32(&conv_bar[s]), 4);  // one arrival per converter warp
    }
    for (int d = 0; d < WQ_SLOTS; d++) {
      mbar_init(smem_u32(&slot_full_bar[d]), NCONV / 32 > 0 ? NCONV / 32 : 1);  // one arrival per converter warp
      mbar_init(smem_u32(&slot_empty_bar[d]), 1);
    }
    for (int a = 0; a < 2; a++) {
      mbar_init(smem_u32(&tmem_full_bar[a]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[a]), BLOCK_N >= 64 ? EPI_WARPS : 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 9) {
    // Tensor memory: the whole warp allocates, the same warp frees at the end.
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_ptr_holder)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (WQ && threadIdx.x >= 320) {
    // A byte has 256 values: dequantise each once per CTA, w = float32(float64(q)*scale + min)
    // (io_utils.ts:139), and keep its tf32 hi / lo split; the main loop only looks bytes up.
    for (int q = threadIdx.x - 320; q < 256; q += NCONV) {
      const float w = (float)((double)q * p.q_scale + p.q_min);
      const float h = round_tf32(w);
      lut_hi[q] = h;
      lut_lo[q] = (fabsf(h) <= 3.4028234e38f) ? round_tf32(w - h) : 0.f;
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_ptr_holder;
  // everything above touched only shared and tensor memory; global memory from here on
  pdl_wait();
  pdl_launch_dependents();

  if (warp == 8) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      // The ring holds few A tiles when the weight tile is large (3 stages at BLOCK_N = 256), too
      // few bytes in flight to cover DRAM latency.  A second cursor runs PREFETCH k-blocks ahead of
      // the loads and pulls the A tiles into L2, so that the loads themselves are L2 hits.
      // (Only where an A tile is worked on for long: K >= 512, or K >= 256 with two or more column
      // tiles.  On the other short-K layers, which run at the DRAM roofline anyway, the extra
      // requests measured slower.)
      const int PREFETCH = (AMODE == A_MATRIX && STAGES <= 6 &&
                            (p.num_k_blocks >= 16 || (p.num_k_blocks >= 8 && p.num_n_tiles >= 2)))
                               ? 8
                               : 0;
      int ptile = blockIdx.x, pkb = 0;
      for (int i = 0; i < PREFETCH && ptile < num_tiles; i++) {
        tma_prefetch_2d(&map_a, pkb * KB_ELEMS, (ptile / p.num_n_tiles) * BLOCK_M);
        if (++pkb == p.num_k_blocks) { pkb = 0; ptile += gridDim.x; }
      }
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile / p.num_n_tiles) * BLOCK_M;
        const int n0 = (tile % p.num_n_tiles) * BLOCK_N;
        for (int kb = 0; kb < p.num_k_blocks; kb++) {
          if (PREFETCH > 0 && ptile < num_tiles) {
            tma_prefetch_2d(&map_a, pkb * KB_ELEMS, (ptile / p.num_n_tiles) * BLOCK_M);
            if (++pkb == p.num_k_blocks) { pkb = 0; ptile += gridDim.x; }
          }
          ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag, p.status, 1);
          if (!ok) break;
          if (p.withhold_last_load && kb + 1 == p.num_k_blocks && tile + (int)gridDim.x >= num_tiles) {
            ok = false;  // the consumers now wait for a stage that never fills
            break;
          }
          const uint32_t bar = smem_u32(&full_bar[stage]);
          mbar_arrive_expect_tx(bar, TX_BYTES);
          if (AMODE == A_MATRIX)
            tma_load_2d(smem_u32(a_hi + stage * A_STAGE_BYTES), &map_a, bar, kb * KB_ELEMS, m0);
          if (WQ) {
            tma_load_2d(smem_u32(b_q + stage * Q_STAGE_BYTES), &map_w_hi, bar, kb * BLOCK_K, n0);
          } else {
            tma_load_2d(smem_u32(b_hi + stage * B_STAGE_BYTES), &map_w_hi, bar, kb * KB_ELEMS, n0);
            if (SPLIT)
              tma_load_2d(smem_u32(b_lo + stage * B_STAGE_BYTES), &map_w_lo, bar, kb * BLOCK_K, n0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 9) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = HALF ? make_idesc_f16(BLOCK_M, BLOCK_N) : make_idesc(BLOCK_M, BLOCK_N);
      int stage = 0;
      uint32_t phase = 0;
      int slot = 0;  // WQ: position in the ring of dequantised weight tiles
      uint32_t slot_phase = 0;
      bool ok = true;
      int local = 0;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, local++) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        ok = mbar_wait(smem_u32(&tmem_empty_bar[acc]), acc_phase ^ 1, abort_flag, p.status, 2);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + acc * ACC_COLS;
        const uint32_t tmem_corr = tmem_d + BLOCK_N;  // 3xTF32 only
        for (int kb = 0; kb < p.num_k_blocks; kb++) {
          ok = mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag, p.status, 3);
          if (ok && WQ)
            ok = mbar_wait(smem_u32(&slot_full_bar[slot]), slot_phase, abort_flag, p.status, 4);
          else if (ok && (SPLIT || ROUND) && AMODE == A_MATRIX)
            ok = mbar_wait(smem_u32(&conv_bar[stage]), phase, abort_flag, p.status, 4);
          if (!ok) break;
          tcgen05_fence_after();
          const int b_tile = WQ ? slot : stage;
          const uint32_t a_hi_s = smem_u32(a_hi + stage * A_STAGE_BYTES);
          const uint32_t a_lo_s = smem_u32(a_lo + stage * A_STAGE_BYTES);
          const uint32_t b_hi_s = smem_u32(b_hi + b_tile * B_STAGE_BYTES);
          const uint32_t b_lo_s = smem_u32(b_lo + b_tile * B_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BLOCK_K / 8; k++) {
            const uint32_t koff = k * 32;  // 8 tf32 = 32 bytes inside the 128-byte swizzle row
            const uint32_t accum = (kb > 0 || k > 0) ? 1u : 0u;
            if (SPLIT) {
              tcgen05_mma_tf32(tmem_corr, make_smem_desc(a_lo_s + koff), make_smem_desc(b_hi_s + koff), idesc, accum);
              tcgen05_mma_tf32(tmem_corr, make_smem_desc(a_hi_s + koff), make_smem_desc(b_lo_s + koff), idesc, 1u);
              tcgen05_mma_tf32(tmem_d, make_smem_desc(a_hi_s + koff), make_smem_desc(b_hi_s + koff), idesc, accum);
            } else if (HALF) {  // 16 halves = the same 32 bytes per instruction
              tcgen05_mma_f16(tmem_d, make_smem_desc(a_hi_s + koff), make_smem_desc(b_hi_s + koff), idesc, accum);
            } else {
              tcgen05_mma_tf32(tmem_d, make_smem_desc(a_hi_s + koff), make_smem_desc(b_hi_s + koff), idesc, accum);
            }
          }
          tcgen05_commit(smem_u32(&empty_bar[stage]));  // frees the stage once the MMAs have read it
          if (WQ) {
            tcgen05_commit(smem_u32(&slot_empty_bar[slot]));
            if (++slot == WQ_SLOTS) { slot = 0; slot_phase ^= 1; }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) tcgen05_commit(smem_u32(&tmem_full_bar[acc]));  // accumulator complete
      }
    }
  } else if (warp >= 10) {
    if (AMODE != A_MATRIX) {
      // ---------------- conv gather warps (one thread per tile row) ----------------
      // Each thread copies its own row of every A stage with cp.async (zero-filled where the tap
      // falls outside the image or beyond K), keeps LAG stages in flight, and hands a stage over
      // to the MMA warp once its copies have landed: for 3xTF32 it first splits its row into
      // tf32 hi/lo in place (the row is private to the thread), then fences the generic-proxy
      // writes for the tensor core and arrives on the stage's full barrier.
      const ConvGeom& g = p.conv;
      const int t = threadIdx.x - 320;  // 0..127
      constexpr int LAG = STAGES >= 4 ? 3 : STAGES - 1;
      int stage = 0, hand_stage = 0;
      uint32_t phase = 0;
      int in_flight = 0;
      bool ok = true;
      auto hand_over = [&](int s) {
        if (SPLIT) {
          float4* hi4 = reinterpret_cast<float4*>(a_hi + s * A_STAGE_BYTES + t * 128);
          float4* lo4 = reinterpret_cast<float4*>(a_lo + s * A_STAGE_BYTES + t * 128);
#pragma unroll
          for (int i = 0; i < 8; i++) {
            float4 v = hi4[i], h, l;
            h.x = round_tf32(v.x); h.y = round_tf32(v.y); h.z = round_tf32(v.z); h.w = round_tf32(v.w);
            l.x = (fabsf(h.x) <= 3.4028234e38f) ? round_tf32(v.x - h.x) : 0.f;
            l.y = (fabsf(h.y) <= 3.4028234e38f) ? round_tf32(v.y - h.y) : 0.f;
            l.z = (fabsf(h.z) <= 3.4028234e38f) ? round_tf32(v.z - h.z) : 0.f;
            l.w = (fabsf(h.w) <= 3.4028234e38f) ? round_tf32(v.w - h.w) : 0.f;
            hi4[i] = h;
            lo4[i] = l;
          }
        } else {
          // TF32: round the row to nearest, the tensor core would truncate it
          float4* hi4 = reinterpret_cast<float4*>(a_hi + s * A_STAGE_BYTES + t * 128);
#pragma unroll
          for (int i = 0; i < 8; i++) {
            float4 v = hi4[i];
            v.x = round_tf32_for_mma(v.x); v.y = round_tf32_for_mma(v.y);
            v.z = round_tf32_for_mma(v.z); v.w = round_tf32_for_mma(v.w);
            hi4[i] = v;
          }
        }
        fence_proxy_async_smem();
        mbar_arrive(smem_u32(&full_bar[s]));
      };
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m = (tile / p.num_n_tiles) * BLOCK_M + t;
        const bool row_valid = m < p.M;
        const int pix = row_valid ? m : 0;
        const int xo = pix % g.outW;
        const int yo = (pix / g.outW) % g.outH;
        const int b = pix / (g.outW * g.outH);
        const int yi0 = yo * g.sH - g.padT, xi0 = xo * g.sW - g.padL;
        const float* xb = g.x + (int64_t)b * g.inH * g.inW * g.Cin;
        int ci = 0, wc = 0, wr = 0;  // tap cursor of the vector gather (advances with kk)
        for (int kb = 0; kb < p.num_k_blocks; kb++) {
          ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag, p.status, 7);
          if (!ok) break;
          const uint32_t row = smem_u32(a_hi + stage * A_STAGE_BYTES);
          if (AMODE == A_CONV_VEC) {
#pragma unroll
            for (int j = 0; j < 8; j++) {
              const int yi = yi0 + wr * g.dH, xi = xi0 + wc * g.dW;
              const bool v = row_valid && wr < g.fH && yi >= 0 && yi < g.inH && xi >= 0 && xi < g.inW;
              const float* src = v ? xb + ((int64_t)yi * g.inW + xi) * g.Cin + ci : g.x;
              cp_async_16_zfill(row + swz(t, j * 16), src, v);
              ci += 4;
              if (ci >= g.Cin) { ci = 0; if (++wc == g.fW) { wc = 0; ++wr; } }
            }
          } else {
            // Cin == 3, fW == 3, dW == 1: filter row wr is 9 contiguous floats of input row yi
#pragma unroll
            for (int r3 = 0; r3 < 3; r3++) {
              const int yi = yi0 + r3 * g.dH;
              const bool rv = row_valid && r3 < g.fH && yi >= 0 && yi < g.inH;
              const float* src = rv ? xb + ((int64_t)yi * g.inW + xi0) * 3 : g.x;
              const bool all_cols = xi0 >= 0 && xi0 + 3 <= g.inW;
              const int o = r3 * 40;  // destination byte offset of this filter row
              if (rv && all_cols && (((uintptr_t)src) & 7) == 0) {
#pragma unroll
                for (int q = 0; q < 4; q++) cp_async_8_zfill(row + swz(t, o + q * 8), src + q * 2, true);
                cp_async_4_zfill(row + swz(t, o + 32), src + 8, true);
              } else {
#pragma unroll
                for (int e = 0; e < 9; e++) {
                  const int xi = xi0 + e / 3;
                  const bool v = rv && xi >= 0 && xi < g.inW;
                  cp_async_4_zfill(row + swz(t, o + e * 4), v ? src + e : g.x, v);
                }
              }
              cp_async_4_zfill(row + swz(t, o + 36), g.x, false);  // pad float of the filter row
            }
            cp_async_8_zfill(row + swz(t, 120), g.x, false);       // k' = 30, 31
          }
          asm volatile("cp.async.commit_group;" ::: "memory");
          if (++in_flight > LAG) {
            asm volatile("cp.async.wait_group %0;" ::"n"(LAG) : "memory");
            hand_over(hand_stage);
            if (++hand_stage == STAGES) hand_stage = 0;
            --in_flight;
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      while (in_flight > 0 && ok) {
        hand_over(hand_stage);
        if (++hand_stage == STAGES) hand_stage = 0;
        --in_flight;
      }
    } else if (SPLIT || ROUND || WQ) {
      // ---------------- converter warps (matrix mode) ----------------
      // 3xTF32: split the A stage in place into tf32 hi / lo.  TF32 with rounding: round the A
      // stage in place.  WQ: dequantise the uint8 weight tile of the stage into the swizzled tf32
      // hi (/lo) tile(s).
      const int t = threadIdx.x - 320;  // 0..127
      int stage = 0;
      uint32_t phase = 0;
      int slot = 0;
      uint32_t slot_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        for (int kb = 0; kb < p.num_k_blocks; kb++) {
          ok = mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag, p.status, 5);
          if (ok && WQ)
            ok = mbar_wait(smem_u32(&slot_empty_bar[slot]), slot_phase ^ 1, abort_flag, p.status, 6);
          if (!ok) break;
          if (SPLIT) {
            float4* hi4 = reinterpret_cast<float4*>(a_hi + stage * A_STAGE_BYTES);
            float4* lo4 = reinterpret_cast<float4*>(a_lo + stage * A_STAGE_BYTES);
#pragma unroll
            for (int i = 0; i < A_STAGE_BYTES / 16 / NCONV; i++) {
              const int idx = t + i * NCONV;  // element-wise: the swizzled placement is preserved
              float4 v = hi4[idx], h, l;
              h.x = round_tf32(v.x); h.y = round_tf32(v.y); h.z = round_tf32(v.z); h.w = round_tf32(v.w);
              // a non-finite hi keeps lo at zero (inf - inf would poison the product with NaN)
              l.x = (fabsf(h.x) <= 3.4028234e38f) ? round_tf32(v.x - h.x) : 0.f;
              l.y = (fabsf(h.y) <= 3.4028234e38f) ? round_tf32(v.y - h.y) : 0.f;
              l.z = (fabsf(h.z) <= 3.4028234e38f) ? round_tf32(v.z - h.z) : 0.f;
              l.w = (fabsf(h.w) <= 3.4028234e38f) ? round_tf32(v.w - h.w) : 0.f;
              hi4[idx] = h;
              lo4[idx] = l;
            }
          }
          if (ROUND) {
            float4* hi4 = reinterpret_cast<float4*>(a_hi + stage * A_STAGE_BYTES);
#pragma unroll
            for (int i = 0; i < A_STAGE_BYTES / 16 / NCONV; i++) {
              const int idx = t + i * NCONV;
              float4 v = hi4[idx];
              v.x = round_tf32_for_mma(v.x); v.y = round_tf32_for_mma(v.y);
              v.z = round_tf32_for_mma(v.z); v.w = round_tf32_for_mma(v.w);
              hi4[idx] = v;
            }
          }
          if (WQ) {
            // the uint8 tile is [BLOCK_N rows][32 bytes]; a thread dequantises 16 bytes at a time
            const uint8_t* q_tile = b_q + stage * Q_STAGE_BYTES;
            uint8_t* w_hi = b_hi + slot * B_STAGE_BYTES;
            uint8_t* w_lo = b_lo + slot * B_STAGE_BYTES;
            if (!SPLIT && p.q_arith) {
              // arithmetic form: byte -> float through the 2^23 mantissa trick, one fma, then
              // round-to-nearest (ties away) to tf32 on the bit pattern
              const uint32_t s32 = __float_as_uint(p.q_scale32), m32 = __float_as_uint(p.q_min32);
              const uint64_t s2 = pack_f32x2(s32, s32), m2 = pack_f32x2(m32, m32);
              const uint64_t neg_magic2 = pack_f32x2(0xCB000000u, 0xCB000000u);  // -2^23 twice
              for (int c = t; c < BLOCK_N * 2; c += NCONV) {
                const int n = c >> 1, half = c & 1;
                const uint4 raw = *reinterpret_cast<const uint4*>(q_tile + n * 32 + half * 16);
                const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                  uint32_t h[4];
#pragma unroll
                  for (int e = 0; e < 4; e += 2) {
                    // 0x4B0000qq is the float 2^23 + q: subtracting 2^23 leaves q exactly
                    const uint64_t r2 = pack_f32x2(__byte_perm(words[j], 0x4B000000u, 0x7540u + e),
                                                   __byte_perm(words[j], 0x4B000000u, 0x7541u + e));
                    unpack_f32x2(fma_f32x2(add_f32x2(r2, neg_magic2), s2, m2), h[e], h[e + 1]);
                    // the tensor core reads the upper 19 bits only, so adding half a tf32 ulp
                    // to the bit pattern is the round-to-nearest (ties away)
                    h[e] += 0x1000u;
                    h[e + 1] += 0x1000u;
                  }
                  *reinterpret_cast<uint4*>(w_hi + swz(n, (half * 16 + j * 4) * 4)) = make_uint4(h[0], h[1], h[2], h[3]);
                }
              }
            } else {
              for (int c = t; c < BLOCK_N * 2; c += NCONV) {
                const int n = c >> 1, half = c & 1;
                const uint4 raw = *reinterpret_cast<const uint4*>(q_tile + n * 32 + half * 16);
                const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                  float h[4], l[4];
#pragma unroll
                  for (int e = 0; e < 4; e++) {
                    const uint32_t q = (words[j] >> (8 * e)) & 0xffu;
                    h[e] = lut_hi[q];
                    if (SPLIT) l[e] = lut_lo[q];
                  }
                  const uint32_t off = swz(n, (half * 16 + j * 4) * 4);
                  *reinterpret_cast<float4*>(w_hi + off) = make_float4(h[0], h[1], h[2], h[3]);
                  if (SPLIT) *reinterpret_cast<float4*>(w_lo + off) = make_float4(l[0], l[1], l[2], l[3]);
                }
              }
            }
          }
          fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor core
          // One arrival per warp, by lane 0 once all its lanes have fenced (a hundred single-thread
          // arrivals on one barrier queue up in the shared-memory pipe; it measured the same here).
          __syncwarp();
          if (WQ) {
            if (lane == 0) mbar_arrive(smem_u32(&slot_full_bar[slot]));
            if (++slot == WQ_SLOTS) { slot = 0; slot_phase ^= 1; }
          } else {
            if (lane == 0) mbar_arrive(smem_u32(&conv_bar[stage]));
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else {
    // ---------------- epilogue warps 0-7 ----------------
    // Warps w and w+4 share TMEM lane quarter w%4 (rows 32*(w%4) .. +31 of the tile) and split
    // the tile's 32-column chunks between them: warp half h takes chunks h, h+2, h+4, ...
    constexpr int CHUNKS = BLOCK_N / 32;
    constexpr int MY_CHUNKS = CHUNKS >= 2 ? CHUNKS / 2 : 1;
    const int quarter = warp & 3;
    const int half = warp >> 2;
    if (CHUNKS >= 2 || half == 0) {
      uint8_t* stage_buf = c_stage + warp * C_CHUNK_BYTES;
      float* bias_s = reinterpret_cast<float*>(bias_stage + warp * 256);
      float* alpha_s = bias_s + 32;
      const bool has_bias = p.epi.bias != nullptr;
      const bool has_alpha = p.epi.activation == TFJS_ACT_PRELU;
      int local = 0;
      int store_parity = 0;  // OUT16: which half of the staging buffer the next chunk uses
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, local++) {
        const int m0 = (tile / p.num_n_tiles) * BLOCK_M;
        const int n0 = (tile % p.num_n_tiles) * BLOCK_N;
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        // One coalesced load per chunk fetches its 32 bias values (and prelu slopes), issued
        // before waiting for the accumulator so that the latency hides behind the MMAs.
        float bias_l[MY_CHUNKS], alpha_l[MY_CHUNKS];
#pragma unroll
        for (int i = 0; i < MY_CHUNKS; i++) {
          const int cl = n0 + (CHUNKS >= 2 ? 2 * i + half : 0) * 32 + lane;
          bias_l[i] = 0.f;
          alpha_l[i] = 0.f;
          if (has_bias) bias_l[i] = p.epi.bias_scalar ? __ldg(p.epi.bias) : (cl < p.N ? __ldg(p.epi.bias + cl) : 0.f);
          if (has_alpha) alpha_l[i] = p.epi.prelu_scalar ? __ldg(p.epi.prelu) : (cl < p.N ? __ldg(p.epi.prelu + cl) : 0.f);
        }
        ok = mbar_wait(smem_u32(&tmem_full_bar[acc]), acc_phase, abort_flag, p.status, 6);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tcgen05_fence_after();
        // TMEM address: lane in bits [16,32), column in [0,16)
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * ACC_COLS;
        bool released = false;
#pragma unroll
        for (int i = 0; i < MY_CHUNKS; i++) {
          const int chunk = CHUNKS >= 2 ? 2 * i + half : 0;
          const int c0 = n0 + chunk * 32;
          if (c0 >= p.N) break;  // the rest of this warp's chunks lie beyond the last column
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + chunk * 32, r);
          __syncwarp();
          bias_s[lane] = bias_l[i];
          if (has_alpha) alpha_s[lane] = alpha_l[i];
          tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int k = 0; k < 32; k++) v[k] = __uint_as_float(r[k]);
          if (SPLIT) {
            // add the correction tile (lo*hi + hi*lo) to the hi*hi tile
            tmem_ld_32x32b_x32(taddr + BLOCK_N + chunk * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int k = 0; k < 32; k++) v[k] += __uint_as_float(r[k]);
          }
          __syncwarp();
          if (i == MY_CHUNKS - 1) {
            // this warp's last read of the accumulator: hand it back to the MMA warp right away
            tcgen05_fence_before();
            if (lane == 0) mbar_arrive(smem_u32(&tmem_empty_bar[acc]));
            released = true;
          }
          switch (p.epi.activation) {
            case TFJS_ACT_RELU: finish_chunk<TFJS_ACT_RELU>(v, has_bias, bias_s, alpha_s, p.epi); break;
            case TFJS_ACT_PRELU: finish_chunk<TFJS_ACT_PRELU>(v, has_bias, bias_s, alpha_s, p.epi); break;
            case TFJS_ACT_CLIP: finish_chunk<TFJS_ACT_CLIP>(v, has_bias, bias_s, alpha_s, p.epi); break;
            default: finish_chunk<TFJS_ACT_LINEAR>(v, has_bias, bias_s, alpha_s, p.epi); break;
          }
          // the staging buffer must have been read by this warp's previous TMA store (a half
          // chunk is 2 KB of the 4 KB buffer: its two halves alternate and one store may be pending)
          if (lane == 0) {
            if (OUT16) tma_store_wait_read<1>(); else tma_store_wait_read<0>();
          }
          __syncwarp();
          if (OUT16) {
            // half output: 32 columns are 64 bytes per row, stored unswizzled
            store_parity ^= 1;
            uint8_t* dst = stage_buf + store_parity * 2048 + lane * 64;
#pragma unroll
            for (int j = 0; j < 4; j++)
              *reinterpret_cast<uint4*>(dst + (j << 4)) =
                  make_uint4(pack_half2(v[j * 8 + 0], v[j * 8 + 1]), pack_half2(v[j * 8 + 2], v[j * 8 + 3]),
                             pack_half2(v[j * 8 + 4], v[j * 8 + 5]), pack_half2(v[j * 8 + 6], v[j * 8 + 7]));
          } else {
            // SWIZZLE_128B placement expected by the store's tensor map: 16-byte chunk j of row
            // `lane` lives at chunk (j ^ (lane & 7)).
            uint8_t* dst = stage_buf + lane * 128;
#pragma unroll
            for (int j = 0; j < 8; j++)
              *reinterpret_cast<float4*>(dst + ((j ^ (lane & 7)) << 4)) =
                  make_float4(v[j * 4 + 0], v[j * 4 + 1], v[j * 4 + 2], v[j * 4 + 3]);
          }
          fence_proxy_async_smem();  // generic-proxy writes -> visible to the TMA engine
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&map_c, smem_u32(stage_buf + (OUT16 ? store_parity * 2048 : 0)), c0, m0 + quarter * 32);
            tma_store_commit();
          }
        }
        if (!released) {
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&tmem_empty_bar[acc]));
        }
      }
    }
    if (lane == 0) tma_store_wait_all();
  }

  // A wait that gave up leaves copies and MMAs of this CTA in flight: give them time to land
  // before the shared and tensor memory they target is released.
  if (*abort_flag) {
    for (int i = 0; i < 100; i++) __nanosleep(1000);
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 9) {
    __syncwarp();
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS)
                 : "memory");
  }
}

// ---- host side ------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn lookup_encode_fn() {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
      q == cudaDriverEntryPointSuccess)
    return (EncodeTiledFn)p;
  cudaGetLastError();
  return nullptr;
}

EncodeTiledFn get_encode_fn() {
  static const EncodeTiledFn fn = lookup_encode_fn();  // initialised once, safely across host threads
  return fn;
}

// 2-D row-major matrix [rows, cols] (cols contiguous) of float32 or IEEE half, box [box_rows,
// box_cols]; SWIZZLE_128B unless `plain`.
bool encode_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
               uint32_t box_cols, bool half = false, bool plain = false) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * (half ? 2 : 4)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, half ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
            const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            plain ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BLOCK_N, int PREC, int AMODE, bool WQ = false, bool OUT16 = false>
int launch_variant(tfjs_cuda_ctx* ctx, const CUtensorMap& ma, const CUtensorMap& mh, const CUtensorMap& ml,
                   const CUtensorMap& mc, const GemmParams& p) {
  constexpr bool SPLIT = PREC == PREC_3XTF32;
  constexpr int layout = layout_bytes(BLOCK_N, SPLIT, WQ);
  static_assert(layout <= SMEM_LIMIT, "shared memory budget exceeded");
  constexpr int smem_bytes = layout + 1024 <= SMEM_LIMIT ? layout + 1024 : SMEM_LIMIT;
  auto kernel = gemm_tcgen05_kernel<BLOCK_N, PREC, AMODE, WQ, OUT16>;
  // the attribute is per device and per kernel; contexts of several devices may call from several
  // host threads, so the flags are atomic (setting the attribute twice is harmless)
  static std::atomic<bool> configured[64];
  if (!configured[ctx->device & 63].load(std::memory_order_acquire)) {
    TFJS_CHECK_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    configured[ctx->device & 63].store(true, std::memory_order_release);
  }
  const int tiles = p.num_m_tiles * p.num_n_tiles;
  const int grid = tiles < ctx->sm_count ? tiles : ctx->sm_count;
  launch_ex(ctx, kernel, dim3(grid), dim3(cta_threads(converts_a(PREC), AMODE, WQ)), smem_bytes, ma, mh, ml, mc, p);
  if (PREC == PREC_F16) return post_launch(ctx, "gemm_tcgen05 (F16)");
  if (WQ) return post_launch(ctx, SPLIT ? "gemm_tcgen05 (3xTF32, uint8 weights)" : "gemm_tcgen05 (TF32, uint8 weights)");
  if (AMODE == A_MATRIX) return post_launch(ctx, SPLIT ? "gemm_tcgen05 (3xTF32)" : "gemm_tcgen05 (TF32)");
  return post_launch(ctx, SPLIT ? "conv2d_tcgen05 (3xTF32)" : "conv2d_tcgen05 (TF32)");
}

// prec: PREC_3XTF32 is limited to 128 columns (two tile pairs fill tensor memory)
template <int AMODE, bool WQ>
int launch_mode(tfjs_cuda_ctx* ctx, int block_n, int prec, const CUtensorMap& ma, const CUtensorMap& mh,
                const CUtensorMap& ml, const CUtensorMap& mc, const GemmParams& p) {
#define TFJS_GEMM_CASE(BN)                                                                            \
  case BN:                                                                                            \
    if (prec == PREC_3XTF32) return launch_variant<BN, PREC_3XTF32, AMODE, WQ>(ctx, ma, mh, ml, mc, p); \
    if (AMODE == A_MATRIX && prec == PREC_TF32_ROUND)                                                 \
      return launch_variant<BN, AMODE == A_MATRIX ? PREC_TF32_ROUND : PREC_TF32_ASIS, AMODE, WQ>(ctx, ma, mh, ml, mc, p); \
    return launch_variant<BN, PREC_TF32_ASIS, AMODE, WQ>(ctx, ma, mh, ml, mc, p);
  switch (block_n) {
    TFJS_GEMM_CASE(32)
    TFJS_GEMM_CASE(64)
    TFJS_GEMM_CASE(128)
    default:
      if (AMODE == A_MATRIX && prec == PREC_TF32_ROUND)
        return launch_variant<256, AMODE == A_MATRIX ? PREC_TF32_ROUND : PREC_TF32_ASIS, AMODE, WQ>(ctx, ma, mh, ml, mc, p);
      return launch_variant<256, PREC_TF32_ASIS, AMODE, WQ>(ctx, ma, mh, ml, mc, p);
  }
#undef TFJS_GEMM_CASE
}

// True when, for every byte value q, tf32(fma(float(q), float(scale), float(min))) has the same
// bits as tf32(float32(double(q) * scale + min)): the kernel may then dequantise with float32
// arithmetic and still feed the tensor core exactly what the float64 formula would.
bool dequant_exact_in_float32(double scale, double min) {
  const float s32 = (float)scale, m32 = (float)min;
  for (int q = 0; q < 256; q++) {
    const float want = (float)((double)q * scale + min);
    const float got = fmaf((float)q, s32, m32);
    uint32_t wb, gb;
    memcpy(&wb, &want, 4);
    memcpy(&gb, &got, 4);
    if ((wb & 0x7f800000u) == 0x7f800000u || (gb & 0x7f800000u) == 0x7f800000u) return false;
    if (((wb + 0x1000u) & 0xffffe000u) != ((gb + 0x1000u) & 0xffffe000u)) return false;
  }
  return true;
}

// uint8 K-major [rows, cols] matrix, box [box_rows, 32 bytes], no swizzle.
bool encode_2d_u8(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols};
  cuuint32_t box[2] = {BLOCK_K, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Shared by the matrix and the convolution entry points.  `a` is the dense A matrix
// (A_MATRIX) or null; K is the contraction length as laid out in the packed weights.
int launch_common(tfjs_cuda_ctx* ctx, int amode, const float* a, const ConvGeom* conv, int64_t M, int64_t K,
                  const float* w_hi, const float* w_lo, int64_t kp, float* out, int64_t N,
                  const EpilogueArgs& epi, int math_mode, bool a_tf32_exact, const uint8_t* w_q = nullptr,
                  double q_scale = 0.0, double q_min = 0.0) {
  const bool split = math_mode == TFJS_MATH_TF32X3;
  // TF32: a dense A matrix is rounded to nearest in shared memory unless its producer already did
  const int prec = split ? PREC_3XTF32 : ((amode == A_MATRIX && !a_tf32_exact) ? PREC_TF32_ROUND : PREC_TF32_ASIS);
  TFJS_REQUIRE(ctx, w_q != nullptr || !split || w_lo != nullptr, "3xTF32 needs the residual weight plane");
  // Large problems go to the CTA-pair kernel (256 x 256 tiles, half of the weight tile per SM).
  // (With on-chip rounding of A the pair kernel only wins on long contractions: 203 vs 211 us at
  // K = 512, 176 vs 187 at 1024, but 230 vs 219 at 128.)
  if (amode == A_MATRIX && w_q && prec == PREC_TF32_ASIS && ctx->gemm_pair && kp == K &&
      gemm_pair_supported(ctx, M, K, N))
    return launch_gemm_tcgen05_pair(ctx, a, M, K, nullptr, nullptr, kp, out, N, epi, true, w_q, q_scale, q_min);
  if (amode == A_MATRIX && !w_q && ctx->gemm_pair && kp == K && gemm_pair_supported(ctx, M, K, N) &&
      (prec != PREC_TF32_ROUND || K >= 512 || ctx->gemm_pair >= 2))
    return launch_gemm_tcgen05_pair(ctx, a, M, K, w_hi, split ? w_lo : nullptr, kp, out, N, epi,
                                    prec == PREC_TF32_ASIS);
  int block_n;
  if (N <= 32) block_n = 32;
  else if (N <= 64) block_n = 64;
  else if (N <= 128 || split) block_n = 128;
  else block_n = (N % 256 == 0 || N > 512) ? 256 : 128;
  // When the widest tile leaves the machine under-filled, a narrower one may finish sooner.  Cost of
  // a candidate = waves x (k-blocks x cycles per k-block + epilogue); a k-block is bound by the
  // shared-memory traffic of its operands (written by TMA, read by the tensor core: measured
  // about 2.9 cycles per 128-byte operand row), the epilogue by the tile's width.  A narrower
  // tile must win by 10 % to be taken, because it re-reads A more often.
  const int64_t m_tiles = ceil_div64(M, BLOCK_M);
  if (m_tiles * ceil_div64(N, block_n) < 2 * (int64_t)ctx->sm_count) {
    const int64_t k_blocks = ceil_div64(K, BLOCK_K);
    auto cost = [&](int bn) {
      const int64_t waves = ceil_div64(m_tiles * ceil_div64(N, bn), ctx->sm_count);
      const double kb_cycles = 2.9 * (BLOCK_M + (split ? 2 : 1) * bn);
      return (double)waves * ((double)k_blocks * kb_cycles + 6.0 * bn + 600.0);
    };
    int best = block_n;
    double best_cost = cost(block_n);
    for (int bn = block_n / 2; bn >= 32; bn /= 2) {
      const double c = cost(bn);
      if (c < 0.9 * best_cost) {
        best = bn;
        best_cost = c;
      }
    }
    block_n = best;
  }
  if (ctx->gemm_block_n && !(split && ctx->gemm_block_n > 128)) block_n = ctx->gemm_block_n;

  CUtensorMap ma, mh, ml, mc;
  bool ok = encode_2d(&mc, out, (uint64_t)M, (uint64_t)N, 32, 32);
  if (w_q) {
    ok = ok && encode_2d_u8(&mh, w_q, (uint64_t)N, (uint64_t)kp, (uint32_t)block_n);
    ml = mh;
  } else {
    ok = ok && encode_2d(&mh, w_hi, (uint64_t)N, (uint64_t)kp, (uint32_t)block_n, BLOCK_K) &&
         encode_2d(&ml, split ? w_lo : w_hi, (uint64_t)N, (uint64_t)kp, (uint32_t)block_n, BLOCK_K);
  }
  if (ok && amode == A_MATRIX) ok = encode_2d(&ma, a, (uint64_t)M, (uint64_t)K, BLOCK_M, BLOCK_K);
  else ma = mh;  // unused by the conv modes
  if (!ok) return set_error(ctx, TFJS_CUDA_ERR_CUDA, "cuTensorMapEncodeTiled failed");

  GemmParams p;
  p.M = (int)M;
  p.N = (int)N;
  p.K = (int)K;
  p.num_m_tiles = (int)m_tiles;
  p.num_n_tiles = (int)ceil_div64(N, block_n);
  p.num_k_blocks = (int)ceil_div64(K, BLOCK_K);
  p.status = ctx->d_status;
  p.epi = epi;
  if (conv) p.conv = *conv;
  else memset(&p.conv, 0, sizeof(p.conv));
  p.q_scale = q_scale;
  p.q_min = q_min;
  p.q_scale32 = (float)q_scale;
  p.q_min32 = (float)q_min;
  p.q_arith = (w_q && !split && dequant_exact_in_float32(q_scale, q_min)) ? 1 : 0;
  p.withhold_last_load = (ctx->test_withhold_last_load && amode == A_MATRIX) ? 1 : 0;
  if (w_q) return launch_mode<A_MATRIX, true>(ctx, block_n, prec, ma, mh, mh, mc, p);
  switch (amode) {
    case A_CONV_VEC: return launch_mode<A_CONV_VEC, false>(ctx, block_n, prec, ma, mh, ml, mc, p);
    case A_CONV_RGB: return launch_mode<A_CONV_RGB, false>(ctx, block_n, prec, ma, mh, ml, mc, p);
    default: return launch_mode<A_MATRIX, false>(ctx, block_n, prec, ma, mh, ml, mc, p);
  }
}

// A and W as IEEE half matrices (K-major W [N, kp], kp a multiple of 8); out is float32 or half.
int launch_half(tfjs_cuda_ctx* ctx, const void* a, int64_t M, int64_t K, const void* w16, int64_t kp, void* out,
                bool out16, int64_t N, const EpilogueArgs& epi) {
  int block_n = N <= 32 ? 32 : (N <= 64 ? 64 : (N <= 128 ? 128 : ((N % 256 == 0 || N > 512) ? 256 : 128)));
  const int64_t m_tiles = ceil_div64(M, BLOCK_M);
  if (m_tiles * ceil_div64(N, block_n) < 2 * (int64_t)ctx->sm_count) {
    // the same waves x (k-blocks x operand bytes + epilogue) model as the float32 kernel
    const int64_t k_blocks = ceil_div64(K, 64);
    auto cost = [&](int bn) {
      const int64_t waves = ceil_div64(m_tiles * ceil_div64(N, bn), ctx->sm_count);
      return (double)waves * ((double)k_blocks * 2.9 * (BLOCK_M + bn) + 6.0 * bn + 600.0);
    };
    int best = block_n;
    double best_cost = cost(block_n);
    for (int bn = block_n / 2; bn >= 32; bn /= 2)
      if (cost(bn) < 0.9 * best_cost) {
        best = bn;
        best_cost = cost(bn);
      }
    block_n = best;
  }
  CUtensorMap ma, mw, mc;
  const bool ok = encode_2d(&ma, a, (uint64_t)M, (uint64_t)K, BLOCK_M, 64, true) &&
                  encode_2d(&mw, w16, (uint64_t)N, (uint64_t)kp, (uint32_t)block_n, 64, true) &&
                  (out16 ? encode_2d(&mc, out, (uint64_t)M, (uint64_t)N, 32, 32, true, true)
                         : encode_2d(&mc, out, (uint64_t)M, (uint64_t)N, 32, 32));
  if (!ok) return set_error(ctx, TFJS_CUDA_ERR_CUDA, "cuTensorMapEncodeTiled failed");
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = (int)M;
  p.N = (int)N;
  p.K = (int)K;
  p.num_m_tiles = (int)m_tiles;
  p.num_n_tiles = (int)ceil_div64(N, block_n);
  p.num_k_blocks = (int)ceil_div64(K, 64);
  p.status = ctx->d_status;
  p.epi = epi;
#define TFJS_HALF_CASE(BN)                                                                       \
  case BN:                                                                                       \
    return out16 ? launch_variant<BN, PREC_F16, A_MATRIX, false, true>(ctx, ma, mw, mw, mc, p)   \
                 : launch_variant<BN, PREC_F16, A_MATRIX, false, false>(ctx, ma, mw, mw, mc, p);
  switch (block_n) {
    TFJS_HALF_CASE(32)
    TFJS_HALF_CASE(64)
    TFJS_HALF_CASE(128)
    default:
      return out16 ? launch_variant<256, PREC_F16, A_MATRIX, false, true>(ctx, ma, mw, mw, mc, p)
                   : launch_variant<256, PREC_F16, A_MATRIX, false, false>(ctx, ma, mw, mw, mc, p);
  }
#undef TFJS_HALF_CASE
}

}  // namespace

int set_wait_limit_gemm(long long cycles) { return set_wait_limit_here(cycles); }

bool tma_encode_tiled(CUtensorMap* map, CUtensorMapDataType dtype, int rank, const void* base,
                      const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                      CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn || rank < 1 || rank > 5) return false;
  cuuint64_t d[5], st[4];
  cuuint32_t b[5], estr[5];
  for (int i = 0; i < rank; i++) {
    d[i] = dims[i];
    b[i] = box[i];
    estr[i] = 1;
    if (i + 1 < rank) st[i] = strides_bytes[i];
  }
  return fn(map, dtype, (cuuint32_t)rank, const_cast<void*>(base), d, st, b, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool tcgen05_gemm_supported(int64_t M, int64_t N, int64_t K) {
  // TMA needs 16-byte row strides; tiles smaller than one MMA are left to the CUDA cores.
  return M >= 1 && N >= 8 && K >= 4 && K % 4 == 0 && N % 4 == 0 && M < (1ll << 31) &&
         N < (1ll << 31) && K < (1ll << 31) && get_encode_fn() != nullptr;
}

int launch_gemm_tcgen05(tfjs_cuda_ctx* ctx, const float* a, int64_t M, int64_t K, const float* w_hi,
                        const float* w_lo, int64_t kp, float* out, int64_t N, const EpilogueArgs& epi,
                        int math_mode, bool a_tf32_exact) {
  return launch_common(ctx, A_MATRIX, a, nullptr, M, K, w_hi, w_lo, kp, out, N, epi, math_mode, a_tf32_exact);
}

bool tcgen05_gemm_f16_supported(int64_t M, int64_t N, int64_t K, bool out16) {
  // TMA needs 16-byte row strides: 8 halves per row of A, W and (if half) the output
  return M >= 1 && N >= 8 && K >= 8 && K % 8 == 0 && N % (out16 ? 8 : 4) == 0 && M < (1ll << 31) &&
         N < (1ll << 31) && K < (1ll << 31) && get_encode_fn() != nullptr;
}

int launch_gemm_tcgen05_f16(tfjs_cuda_ctx* ctx, const void* a, int64_t M, int64_t K, const void* w16, int64_t kp,
                            void* out, bool out16, int64_t N, const EpilogueArgs& epi) {
  return launch_half(ctx, a, M, K, w16, kp, out, out16, N, epi);
}

// Matrix-mode GEMM whose weights are raw uint8 bytes, K-major [N, kq] (kq a multiple of 16),
// dequantised inside the main loop.
int launch_gemm_tcgen05_u8(tfjs_cuda_ctx* ctx, const float* a, int64_t M, int64_t K, const uint8_t* w_q,
                           int64_t kq, double scale, double min, float* out, int64_t N,
                           const EpilogueArgs& epi, int math_mode, bool a_tf32_exact) {
  return launch_common(ctx, A_MATRIX, a, nullptr, M, K, nullptr, nullptr, kq, out, N, epi, math_mode,
                       a_tf32_exact, w_q, scale, min);
}

// Which implicit-GEMM gather, if any, can take this convolution (0 = none).
int tcgen05_conv_mode(const tfjs_conv2d_info& ci) {
  const int64_t M = (int64_t)ci.batchSize * ci.outHeight * ci.outWidth;
  const int64_t N = ci.outChannels;
  if (M < 1 || M >= (1ll << 31) || N < 8 || N % 4 != 0 || get_encode_fn() == nullptr) return 0;
  if ((int64_t)ci.batchSize * ci.inHeight * ci.inWidth * ci.inChannels >= (1ll << 31)) return 0;
  if (ci.inChannels == 3 && ci.filterWidth == 3 && ci.filterHeight <= 3 && ci.dilationWidth == 1) return A_CONV_RGB;
  if (ci.inChannels >= 4 && ci.inChannels % 4 == 0) return A_CONV_VEC;
  return 0;
}

// Contraction length of the packed weights for a conv mode (see the K layouts above).
int64_t tcgen05_conv_k(const tfjs_conv2d_info& ci, int mode) {
  if (mode == A_CONV_RGB) return 32;
  return (int64_t)ci.filterHeight * ci.filterWidth * ci.inChannels;
}

int launch_conv_tcgen05(tfjs_cuda_ctx* ctx, int mode, const float* x, const tfjs_conv2d_info& ci,
                        const float* w_hi, const float* w_lo, int64_t kp, float* out,
                        const EpilogueArgs& epi, int math_mode) {
  ConvGeom g;
  g.x = x;
  g.inH = ci.inHeight; g.inW = ci.inWidth; g.Cin = ci.inChannels;
  g.outH = ci.outHeight; g.outW = ci.outWidth;
  g.sH = ci.strideHeight; g.sW = ci.strideWidth; g.dH = ci.dilationHeight; g.dW = ci.dilationWidth;
  g.padT = ci.padTop; g.padL = ci.padLeft; g.fH = ci.filterHeight; g.fW = ci.filterWidth;
  const int64_t M = (int64_t)ci.batchSize * ci.outHeight * ci.outWidth;
  return launch_common(ctx, mode, nullptr, &g, M, tcgen05_conv_k(ci, mode), w_hi, w_lo, kp, out,
                       ci.outChannels, epi, math_mode, false);
}
