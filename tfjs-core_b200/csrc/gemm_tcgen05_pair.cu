// Tensor-core GEMM on CTA pairs (tcgen05 cta_group::2): out[M, N] = act(A[M, K] * W[K, N] + bias[N])
// for the deep pointwise convolutions (tfjs-core/src/backends/backend.ts:414-418 fusedConv2d with a
// 1x1 filter, :134-138 fusedBatchMatMul), float32 in and out.  Three precisions: one TF32 pass on an
// A whose producer already rounded it to tf32, one TF32 pass with A rounded to nearest on chip, and
// 3xTF32 (A split into tf32 hi / lo on chip, hi and lo weight planes, three passes).
//
// Why pairs.  The single-CTA kernel computes a 128 x 256 tile per SM and has to bring 128 rows of A
// and 256 rows of W into its shared memory per k-block: 48 KB for 128 x 256 x 32 multiply-adds.  Its
// main loop runs at about 2.9 cycles per 128-byte operand row, i.e. it is bound by the bytes that
// arrive in (and are read back out of) the SM's shared memory, with the tensor pipe half idle.  A
// pair of CTAs on the two SMs of a cluster computes a 256 x 256 tile together: each CTA supplies its
// own 128 rows of A and only HALF of the W tile (128 rows), and the tensor cores of both SMs read
// both halves.  That is 32 KB per SM and k-block for the same 128 x 256 x 32 multiply-adds per SM,
// the W traffic out of L2 halves, and the shared memory holds 6 stages instead of 4.
//
// Structure (both CTAs of a pair run the same code; rank 0 is the leader):
//   warp 8      TMA producer, in each CTA: its A tile [128 x 32] and its half of the W tile
//               [128 x 32] per k-block into a ring of local stages.  The loads of both CTAs complete
//               on the LEADER's full barrier (the .cta_group::2 form of the tensor load; every CTA fetches its own bytes).
//   warp 9      MMA issuer, leader only: one thread issues tcgen05.mma.cta_group::2 (M = 256,
//               N = 256, K = 8) per 32-byte k-step and commits stage-release and accumulator-ready
//               barriers in both CTAs (one tcgen05.commit per barrier; the peer's through its
//               shared::cluster address).
//   warps 10-13 (rounding and 3xTF32 variants) converters, in each CTA: its A load completes on a
//               barrier of its own CTA; they round the stage in place, or split it into a hi and a lo
//               tile, and arrive on the leader's converter barrier.  3xTF32 keeps three stages of
//               64 KB and ONE accumulator buffer (a main and a correction tile, all 512 columns).
//   warps 0-7   epilogue, in each CTA: its 128 rows x 256 columns of the accumulator (two buffers
//               of 256 tensor-memory columns, so the next tile's MMAs overlap), bias, activation,
//               swizzled staging, 128-bit row stores.  Both CTAs hand the buffer back on the leader's barrier.
// Every mbarrier wait is bounded.  A wait that gives up sets the status word; the CTA leaves its
// loops and still takes part in the two cluster barriers, so its peer (whose own waits then run out
// as well) is not left behind, and the pair frees its tensor memory.
#include <atomic>

#include "tcgen05_ptx.cuh"

namespace {

constexpr int CTA_M = 128;    // rows of A (and of the output) per CTA
constexpr int PAIR_M = 256;   // rows per pair tile
constexpr int TILE_N = 256;   // columns per pair tile
constexpr int HALF_N = 128;   // rows of the K-major W tile that each CTA stages
constexpr int BLOCK_K = 32;   // 32 fp32 = 128 bytes = one swizzle row
constexpr int A_BYTES = CTA_M * BLOCK_K * 4;   // 16 KB
constexpr int B_BYTES = HALF_N * BLOCK_K * 4;  // 16 KB
// How A is prepared for the tensor core (which reads the upper 19 bits of each float32):
constexpr int PAIR_ASIS = 0;   // one pass, A already holds tf32-exact values
constexpr int PAIR_SPLIT = 1;  // 3xTF32: converter warps split A into hi / lo, three passes
constexpr int PAIR_ROUND = 2;  // one pass, converter warps round A to nearest in shared memory first
constexpr int PAIR_WQ = 3;     // one pass, A tf32-exact, weights arrive as raw uint8 affine-quantised bytes
                               // (each CTA its 128 rows x 32 bytes per k-block) and the converter warps
                               // dequantise them in shared memory, k-block by k-block, inside the main loop:
                               // w = float32(float64(q) * scale + min) (io_utils.ts:139), rounded to tf32,
                               // straight into the swizzled operand tile the tensor cores read
constexpr int Q_BYTES = HALF_N * BLOCK_K;  // 4 KB: this CTA's half of the uint8 weight tile
constexpr int WQ_SLOTS = 3;                // ring of dequantised weight half-tiles (16 KB each)
// SPLIT (3xTF32): a stage also holds the lo parts of A (written by the converter warps) and of the
// weight half (loaded), so three stages of 64 KB instead of six of 32 KB.
__host__ __device__ constexpr int num_stages(bool split) { return split ? 3 : 6; }
constexpr int EPI_WARPS = 8;
constexpr int C_CHUNK_BYTES = 32 * 32 * 4;
constexpr int C_STAGING_BYTES = EPI_WARPS * C_CHUNK_BYTES;
constexpr int BIAS_STAGING_BYTES = EPI_WARPS * 256;
constexpr int BARRIER_BYTES = 1024;
constexpr int LAYOUT_BYTES = 6 * (A_BYTES + B_BYTES) + C_STAGING_BYTES + BIAS_STAGING_BYTES + BARRIER_BYTES;
constexpr int SMEM_LIMIT = 232448;  // 227 KB
static_assert(LAYOUT_BYTES <= SMEM_LIMIT, "shared memory budget exceeded");
// 10 warps, plus (SPLIT) four converter warps that split each A stage into tf32 hi / lo
// (eight of them when they dequantise uint8 weights)
__host__ __device__ constexpr int cta_threads(int prec) { return prec == 0 ? 320 : (prec == 3 ? 576 : 448); }
// Tensor memory, all 512 columns either way: two accumulator buffers of 256 columns, or (SPLIT) one
// buffer made of a main tile (hi*hi) and a correction tile (lo*hi + hi*lo) that the epilogue adds.
constexpr uint32_t TMEM_COLS = 512;

struct PairParams {
  double q_scale, q_min;  // PAIR_WQ: w = q * q_scale + q_min, evaluated in float64
  // set when the host has checked, for all 256 byte values, that one float32 fma followed by the
  // tf32 rounding gives the same bits as the float64 evaluation
  float q_scale32, q_min32;
  int q_arith;
  int M, N, K;
  int num_m_tiles, num_n_tiles, num_k_blocks;
  float* out;
  // diagnostic: neither producer issues the loads of its last k-block, so the consumers' bounded
  // waits run out (nothing is left in flight, both CTAs give up cleanly)
  int withhold_last_load;
  int* status;
  EpilogueArgs epi;
};

// ---- cluster-level PTX -----------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx_cluster(uint32_t cluster_addr, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_addr),
               "r"(bytes)
               : "memory");
}
// TMA load whose completion is counted on a barrier that may live in the peer CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t cluster_bar, int x,
                                                 int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(x), "r"(y)
      : "memory");
}
// one barrier (anywhere in the cluster) arrives once all MMAs issued so far by this thread are done
__device__ __forceinline__ void tcgen05_commit_pair(uint32_t cluster_bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar)
               : "memory");
}
__device__ __forceinline__ void tcgen05_mma_tf32_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                      uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <int PREC>
__global__ void __launch_bounds__(cta_threads(PREC), 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                         const __grid_constant__ CUtensorMap map_w_lo, PairParams p) {
  constexpr bool SPLIT = PREC == PAIR_SPLIT;
  constexpr bool WQ = PREC == PAIR_WQ;
  constexpr bool CONVERTS = PREC == PAIR_SPLIT || PREC == PAIR_ROUND;  // A passes through this CTA's converter warps
  constexpr int STAGES = num_stages(SPLIT);
  constexpr int NUM_ACC = SPLIT ? 1 : 2;
  constexpr uint32_t ACC_COLS = SPLIT ? 2 * TILE_N : TILE_N;  // tensor-memory columns per buffer
  // bytes that one CTA's loads complete on the leader's full barrier per stage
  constexpr uint32_t STAGE_TX = SPLIT ? 2 * B_BYTES : (CONVERTS ? B_BYTES : (WQ ? A_BYTES : A_BYTES + B_BYTES));
  extern __shared__ uint8_t smem_raw[];
  const uint32_t align_pad = (1024u - (smem_u32(smem_raw) & 1023u)) & 1023u;
  uint32_t window;
  asm("mov.u32 %0, %%dynamic_smem_size;" : "=r"(window));
  // the same in both CTAs of a pair; a pair that cannot lay out its stages does nothing but the
  // two cluster barriers
  const bool layout_ok = align_pad + (uint32_t)LAYOUT_BYTES <= window;
  uint8_t* smem = smem_raw + align_pad;
  uint8_t* a_st = smem;                                         // [STAGES] A (SPLIT: its hi part after the split)
  uint8_t* a_lo_st = a_st + STAGES * A_BYTES;                   // [STAGES] SPLIT only
  uint8_t* b_st = a_lo_st + (SPLIT ? STAGES * A_BYTES : 0);     // [STAGES] this CTA's half of the weight tile
  uint8_t* b_lo_st = b_st + STAGES * B_BYTES;                   // [STAGES] SPLIT only
  // PAIR_WQ: b_st is a ring of WQ_SLOTS dequantised half-tiles instead, the raw bytes of every stage follow
  uint8_t* q_st = b_st + WQ_SLOTS * B_BYTES;                    // [STAGES] WQ only
  float* lut = reinterpret_cast<float*>(q_st + STAGES * Q_BYTES);  // [256] WQ only
  uint8_t* c_stage = WQ ? reinterpret_cast<uint8_t*>(lut) + 1024 : b_lo_st + (SPLIT ? STAGES * B_BYTES : 0);
  uint8_t* bias_stage = c_stage + C_STAGING_BYTES;
  uint64_t* bars = (uint64_t*)(bias_stage + BIAS_STAGING_BYTES);
  uint64_t* full_bar = bars;                     // [STAGES] leader's: both CTAs' loads -> MMA
  uint64_t* empty_bar = bars + STAGES;           // [STAGES] in each CTA: MMA -> local producer
  uint64_t* a_full_bar = bars + 2 * STAGES;      // [STAGES] SPLIT, in each CTA: its A load -> its converters
  uint64_t* conv_bar = bars + 3 * STAGES;        // [STAGES] SPLIT, leader's: both CTAs' converters -> MMA
  uint64_t* tmem_full_bar = bars + 4 * STAGES;   // [2] in each CTA: MMA -> local epilogue
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;  // [2] leader's: both CTAs' epilogues -> MMA
  uint64_t* slot_full_bar = tmem_empty_bar + 2;  // [WQ_SLOTS] WQ, leader's: both CTAs' converters -> MMA
  uint64_t* slot_empty_bar = slot_full_bar + WQ_SLOTS;  // [WQ_SLOTS] WQ, in each CTA: MMA -> local converters
  uint32_t* tmem_ptr_holder = (uint32_t*)(slot_empty_bar + WQ_SLOTS);
  volatile int* abort_flag = (volatile int*)(tmem_ptr_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int num_tiles = p.num_m_tiles * p.num_n_tiles;
  if (threadIdx.x == 32 * 8) {  // the producer warp's first lane: descriptors on their way before the set-up below
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_w);
    if (SPLIT) prefetch_tensormap(&map_w_lo);
  }

  if (layout_ok) {
    if (threadIdx.x == 0) {
      for (int s = 0; s < STAGES; s++) {
        mbar_init(smem_u32(&full_bar[s]), 2);  // one arrive.expect_tx from the producer of each CTA
        mbar_init(smem_u32(&empty_bar[s]), 1);
        mbar_init(smem_u32(&a_full_bar[s]), 1);
        mbar_init(smem_u32(&conv_bar[s]), 2 * 4);  // one arrival per converter warp of each CTA
      }
      for (int a = 0; a < 2; a++) {
        mbar_init(smem_u32(&tmem_full_bar[a]), 1);
        mbar_init(smem_u32(&tmem_empty_bar[a]), 2 * EPI_WARPS);
      }
      for (int d = 0; d < WQ_SLOTS; d++) {
        mbar_init(smem_u32(&slot_full_bar[d]), 2 * 8);  // one arrival per converter warp of each CTA
        mbar_init(smem_u32(&slot_empty_bar[d]), 1);
      }
      *abort_flag = 0;
      fence_barrier_init();
    }
    if (warp == 9) {
      // Tensor memory of both SMs: warp 9 of each CTA takes part in the allocation, and the same
      // warps free it at the end.
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                       smem_u32(tmem_ptr_holder)),
                   "r"(TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
  } else if (threadIdx.x == 0) {
    atomicCAS(p.status, 0, STATUS_SMEM_LAYOUT);
  }
  if (WQ && layout_ok && threadIdx.x >= 320) {
    // a byte has 256 values: dequantise each once per CTA; the main loop only looks bytes up
    for (int q = threadIdx.x - 320; q < 256; q += 256)
      lut[q] = round_tf32((float)((double)q * p.q_scale + p.q_min));
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything arrives on them
  tcgen05_fence_after();
  const uint32_t tmem_base = layout_ok ? *tmem_ptr_holder : 0u;
  // everything above touched only shared and tensor memory; global memory from here on
  pdl_wait();
  pdl_launch_dependents();

  if (!layout_ok) {
    // nothing to do
  } else if (warp == 8) {
    // ---------------- TMA producer (each CTA loads its own operands) ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      // No L2 prefetch cursor ahead of the loads, unlike the single-CTA kernel: its requests compete
      // with the loads (TF32, six stages: 6-12 % slower with it; 3xTF32, three stages: 5 % slower).
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        const int m0 = (tile / p.num_n_tiles) * PAIR_M + (int)rank * CTA_M;
        const int n0 = (tile % p.num_n_tiles) * TILE_N + (int)rank * HALF_N;
        for (int kb = 0; kb < p.num_k_blocks; kb++) {
          ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag, p.status, 31);
          if (!ok) break;
          if (p.withhold_last_load && kb + 1 == p.num_k_blocks && tile + num_pairs >= num_tiles) {
            ok = false;  // the consumers now wait for a stage that never fills
            break;
          }
          const uint32_t bar = map_to_cta(smem_u32(&full_bar[stage]), 0);
          mbar_arrive_expect_tx_cluster(bar, STAGE_TX);
          if (CONVERTS) {
            // A goes to this CTA's own converters first; the weight halves (hi and lo) to the leader
            const uint32_t abar = smem_u32(&a_full_bar[stage]);
            mbar_arrive_expect_tx(abar, A_BYTES);
            tma_load_2d(smem_u32(a_st + stage * A_BYTES), &map_a, abar, kb * BLOCK_K, m0);
            tma_load_2d_pair(smem_u32(b_st + stage * B_BYTES), &map_w, bar, kb * BLOCK_K, n0);
            if (SPLIT) tma_load_2d_pair(smem_u32(b_lo_st + stage * B_BYTES), &map_w_lo, bar, kb * BLOCK_K, n0);
          } else if (WQ) {
            // A to the leader; this CTA's 4 KB of weight bytes to its own converters
            const uint32_t qbar = smem_u32(&a_full_bar[stage]);
            mbar_arrive_expect_tx(qbar, Q_BYTES);
            tma_load_2d_pair(smem_u32(a_st + stage * A_BYTES), &map_a, bar, kb * BLOCK_K, m0);
            tma_load_2d(smem_u32(q_st + stage * Q_BYTES), &map_w, qbar, kb * BLOCK_K, n0);
          } else {
            tma_load_2d_pair(smem_u32(a_st + stage * A_BYTES), &map_a, bar, kb * BLOCK_K, m0);
            tma_load_2d_pair(smem_u32(b_st + stage * B_BYTES), &map_w, bar, kb * BLOCK_K, n0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 9) {
    // ---------------- MMA issuer (leader only) ----------------
    if (rank == 0 && lane == 0) {
      constexpr uint32_t idesc = make_idesc(PAIR_M, TILE_N);
      int stage = 0;
      uint32_t phase = 0;
      int slot = 0;  // WQ: position in the ring of dequantised weight tiles
      uint32_t slot_phase = 0;
      bool ok = true;
      int local = 0;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, local++) {
        const int acc = local % NUM_ACC;
        const uint32_t acc_phase = (local / NUM_ACC) & 1;
        ok = mbar_wait(smem_u32(&tmem_empty_bar[acc]), acc_phase ^ 1, abort_flag, p.status, 32);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + acc * ACC_COLS;
        const uint32_t tmem_corr = tmem_d + TILE_N;  // SPLIT only
        for (int kb = 0; kb < p.num_k_blocks; kb++) {
          ok = mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag, p.status, 33);
          if (ok && CONVERTS) {
            // (the converters of both CTAs made their stores visible to the tensor cores with
            // fence.proxy.async before they arrived; this side needs the wait and the tcgen05 fence
            // below, no cluster-scope fence of its own: one per k-block in this thread cost 20 %)
            ok = mbar_wait(smem_u32(&conv_bar[stage]), phase, abort_flag, p.status, 35);
          }
          if (ok && WQ) ok = mbar_wait(smem_u32(&slot_full_bar[slot]), slot_phase, abort_flag, p.status, 37);
          if (!ok) break;
          tcgen05_fence_after();
          const uint32_t a_s = smem_u32(a_st + stage * A_BYTES);
          const uint32_t b_s = smem_u32(b_st + (WQ ? slot : stage) * B_BYTES);
          const uint32_t a_lo_s = smem_u32(a_lo_st + stage * A_BYTES);
          const uint32_t b_lo_s = smem_u32(b_lo_st + stage * B_BYTES);
#pragma unroll
          for (int k = 0; k < BLOCK_K / 8; k++) {
            const uint32_t koff = k * 32;  // 8 tf32 = 32 bytes inside the 128-byte swizzle row
            const uint32_t accum = (kb > 0 || k > 0) ? 1u : 0u;
            if (SPLIT) {
              // the small terms accumulate in their own tile, away from the large sum's alignment truncations
              tcgen05_mma_tf32_pair(tmem_corr, make_smem_desc(a_lo_s + koff), make_smem_desc(b_s + koff), idesc, accum);
              tcgen05_mma_tf32_pair(tmem_corr, make_smem_desc(a_s + koff), make_smem_desc(b_lo_s + koff), idesc, 1u);
            }
            tcgen05_mma_tf32_pair(tmem_d, make_smem_desc(a_s + koff), make_smem_desc(b_s + koff), idesc, accum);
          }
          // the stage is free in both CTAs once these MMAs have read it
          const uint32_t eb = smem_u32(&empty_bar[stage]);
          tcgen05_commit_pair(eb);
          tcgen05_commit_pair(map_to_cta(eb, 1));
          if (WQ) {  // and so is the dequantised tile, for the converters of both CTAs
            const uint32_t sb = smem_u32(&slot_empty_bar[slot]);
            tcgen05_commit_pair(sb);
            tcgen05_commit_pair(map_to_cta(sb, 1));
            if (++slot == WQ_SLOTS) { slot = 0; slot_phase ^= 1; }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) {  // accumulator complete: wake the epilogue of both CTAs
          const uint32_t fb = smem_u32(&tmem_full_bar[acc]);
          tcgen05_commit_pair(fb);
          tcgen05_commit_pair(map_to_cta(fb, 1));
        }
      }
    }
  } else if (warp >= 10 && WQ) {
    // ---------------- converter warps (each CTA dequantises its own half of the weight tile) ----------------
    const int t = threadIdx.x - 320;  // 0..255
    int stage = 0, slot = 0;
    uint32_t phase = 0, slot_phase = 0;
    bool ok = true;
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      for (int kb = 0; kb < p.num_k_blocks; kb++) {
        ok = mbar_wait(smem_u32(&a_full_bar[stage]), phase, abort_flag, p.status, 38);
        if (ok) ok = mbar_wait(smem_u32(&slot_empty_bar[slot]), slot_phase ^ 1, abort_flag, p.status, 39);
        if (!ok) break;
        // the uint8 tile is [128 rows][32 bytes]; thread t dequantises the 16 bytes of half t & 1 of row t >> 1
        const uint8_t* q_tile = q_st + stage * Q_BYTES;
        uint8_t* w_tile = b_st + slot * B_BYTES;
        const int n = t >> 1, half = t & 1;
        const uint4 raw = *reinterpret_cast<const uint4*>(q_tile + n * 32 + half * 16);
        const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
        if (p.q_arith) {
          // arithmetic form: byte -> float through the 2^23 mantissa trick, one fma, then
          // round-to-nearest (ties away) to tf32 on the bit pattern
          const uint32_t s32 = __float_as_uint(p.q_scale32), m32 = __float_as_uint(p.q_min32);
          const uint64_t s2 = pack_f32x2(s32, s32), m2 = pack_f32x2(m32, m32);
          const uint64_t neg_magic2 = pack_f32x2(0xCB000000u, 0xCB000000u);  // -2^23 twice
#pragma unroll
          for (int j = 0; j < 4; j++) {
            uint32_t h[4];
#pragma unroll
            for (int e = 0; e < 4; e += 2) {
              // 0x4B0000qq is the float 2^23 + q: subtracting 2^23 leaves q exactly
              const uint64_t r2 = pack_f32x2(__byte_perm(words[j], 0x4B000000u, 0x7540u + e),
                                             __byte_perm(words[j], 0x4B000000u, 0x7541u + e));
              unpack_f32x2(fma_f32x2(add_f32x2(r2, neg_magic2), s2, m2), h[e], h[e + 1]);
              h[e] += 0x1000u;  // the tensor core reads the upper 19 bits only: this is the rounding
              h[e + 1] += 0x1000u;
            }
            *reinterpret_cast<uint4*>(w_tile + swz(n, (half * 16 + j * 4) * 4)) = make_uint4(h[0], h[1], h[2], h[3]);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 4; j++) {
            float h[4];
#pragma unroll
            for (int e = 0; e < 4; e++) h[e] = lut[(words[j] >> (8 * e)) & 0xffu];
            *reinterpret_cast<float4*>(w_tile + swz(n, (half * 16 + j * 4) * 4)) = make_float4(h[0], h[1], h[2], h[3]);
          }
        }
        fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor cores
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&slot_full_bar[slot]), 0));
        if (++slot == WQ_SLOTS) { slot = 0; slot_phase ^= 1; }
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp >= 10) {
    // ---------------- converter warps (each CTA prepares its own A stages) ----------------
    // 3xTF32: hi = tf32(a) in place, lo = tf32(a - hi) into the stage's lo tile.  TF32 with rounding:
    // a is rounded to nearest in place.  Element-wise, so the swizzled placement is preserved.  A non-finite hi keeps lo at zero (inf - inf would poison
    // the product with NaN).
    if (CONVERTS) {
      const int t = threadIdx.x - 320;  // 0..127
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        for (int kb = 0; kb < p.num_k_blocks; kb++) {
          ok = mbar_wait(smem_u32(&a_full_bar[stage]), phase, abort_flag, p.status, 36);
          if (!ok) break;
          float4* hi4 = reinterpret_cast<float4*>(a_st + stage * A_BYTES);
          float4* lo4 = reinterpret_cast<float4*>(a_lo_st + stage * A_BYTES);
#pragma unroll
          for (int i = 0; i < A_BYTES / 16 / 128; i++) {
            const int idx = t + i * 128;
            float4 v = hi4[idx], h, l;
            if (!SPLIT) {  // TF32: round to nearest where the tensor core would truncate
              v.x = round_tf32_for_mma(v.x); v.y = round_tf32_for_mma(v.y);
              v.z = round_tf32_for_mma(v.z); v.w = round_tf32_for_mma(v.w);
              hi4[idx] = v;
              continue;
            }
            h.x = round_tf32(v.x); h.y = round_tf32(v.y); h.z = round_tf32(v.z); h.w = round_tf32(v.w);
            l.x = (fabsf(h.x) <= 3.4028234e38f) ? round_tf32(v.x - h.x) : 0.f;
            l.y = (fabsf(h.y) <= 3.4028234e38f) ? round_tf32(v.y - h.y) : 0.f;
            l.z = (fabsf(h.z) <= 3.4028234e38f) ? round_tf32(v.z - h.z) : 0.f;
            l.w = (fabsf(h.w) <= 3.4028234e38f) ? round_tf32(v.w - h.w) : 0.f;
            hi4[idx] = h;
            lo4[idx] = l;
          }
          fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor cores
          __syncwarp();
          // (plain remote arrive: the stores above are already performed in this SM's shared memory
          // and ordered for its tensor core by the proxy fence; an arrive with .release.cluster
          // costs the converters about a microsecond per stage and made them the bottleneck)
          if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&conv_bar[stage]), 0));
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else {
    // ---------------- epilogue warps 0-7 (each CTA: its 128 rows, all 256 columns) ----------------
    // Warps w and w+4 share TMEM lane quarter w%4 and split the eight 32-column chunks: warp half h
    // takes chunks h, h+2, h+4, h+6.
    constexpr int MY_CHUNKS = TILE_N / 64;
    const int quarter = warp & 3;
    const int half = warp >> 2;
    uint8_t* stage_buf = c_stage + warp * C_CHUNK_BYTES;
    float* bias_s = reinterpret_cast<float*>(bias_stage + warp * 256);
    float* alpha_s = bias_s + 32;
    const bool has_bias = p.epi.bias != nullptr;
    const bool has_alpha = p.epi.activation == TFJS_ACT_PRELU;
    int local = 0;
    bool ok = true;
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, local++) {
      const int m0 = (tile / p.num_n_tiles) * PAIR_M + (int)rank * CTA_M;
      const int n0 = (tile % p.num_n_tiles) * TILE_N;
      const int acc = local % NUM_ACC;
      const uint32_t acc_phase = (local / NUM_ACC) & 1;
      float bias_l[MY_CHUNKS], alpha_l[MY_CHUNKS];
#pragma unroll
      for (int i = 0; i < MY_CHUNKS; i++) {
        const int cl = n0 + (2 * i + half) * 32 + lane;
        bias_l[i] = 0.f;
        alpha_l[i] = 0.f;
        if (has_bias) bias_l[i] = p.epi.bias_scalar ? __ldg(p.epi.bias) : (cl < p.N ? __ldg(p.epi.bias + cl) : 0.f);
        if (has_alpha) alpha_l[i] = p.epi.prelu_scalar ? __ldg(p.epi.prelu) : (cl < p.N ? __ldg(p.epi.prelu + cl) : 0.f);
      }
      ok = mbar_wait(smem_u32(&tmem_full_bar[acc]), acc_phase, abort_flag, p.status, 34);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      // TMEM address: lane in bits [16,32), column in [0,16)
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * ACC_COLS;
#pragma unroll
      for (int i = 0; i < MY_CHUNKS; i++) {
        const int chunk = 2 * i + half;
        const int c0 = n0 + chunk * 32;
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
          tmem_ld_32x32b_x32(taddr + TILE_N + chunk * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int k = 0; k < 32; k++) v[k] += __uint_as_float(r[k]);
        }
        __syncwarp();
        if (i == MY_CHUNKS - 1) {
          // this warp's last read of the accumulator: hand it back to the leader's MMA warp
          tcgen05_fence_before();
          if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty_bar[acc]), 0));
        }
        switch (p.epi.activation) {
          case TFJS_ACT_RELU: finish_chunk<TFJS_ACT_RELU>(v, has_bias, bias_s, alpha_s, p.epi); break;
          case TFJS_ACT_PRELU: finish_chunk<TFJS_ACT_PRELU>(v, has_bias, bias_s, alpha_s, p.epi); break;
          case TFJS_ACT_CLIP: finish_chunk<TFJS_ACT_CLIP>(v, has_bias, bias_s, alpha_s, p.epi); break;
          default: finish_chunk<TFJS_ACT_LINEAR>(v, has_bias, bias_s, alpha_s, p.epi); break;
        }
        // Through the warp's staging buffer (rows of 128 bytes, 16-byte chunk j of row r at chunk
        // j ^ (r & 7), which keeps both passes free of bank conflicts) and out with 128-bit stores,
        // four whole rows per warp instruction.  Stores issued by the warps measured 2 % faster here
        // than TMA stores, which queue up behind the loads in the same unit.
        __syncwarp();
        uint8_t* dst = stage_buf + lane * 128;
#pragma unroll
        for (int j = 0; j < 8; j++)
          *reinterpret_cast<float4*>(dst + ((j ^ (lane & 7)) << 4)) =
              make_float4(v[j * 4 + 0], v[j * 4 + 1], v[j * 4 + 2], v[j * 4 + 3]);
        __syncwarp();
        const int rr = lane >> 3, cc = lane & 7;
#pragma unroll
        for (int it = 0; it < 8; it++) {
          const int row = it * 4 + rr;
          const float4 val = *reinterpret_cast<const float4*>(stage_buf + row * 128 + ((cc ^ (row & 7)) << 4));
          const int gm = m0 + quarter * 32 + row;
          if (gm < p.M) *reinterpret_cast<float4*>(p.out + (size_t)gm * p.N + c0 + cc * 4) = val;
        }
      }
    }
  }

  // A wait that gave up leaves copies and MMAs in flight: give them time to land before the
  // shared and tensor memory they target is released.
  if (layout_ok && *abort_flag) {
    for (int i = 0; i < 100; i++) __nanosleep(1000);
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA frees tensor memory or exits while the other may still use it
  if (layout_ok && warp == 9) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// True when, for every byte value q, tf32(fma(float(q), float(scale), float(min))) has the same
// bits as tf32(float32(double(q) * scale + min)): the kernel may then dequantise with float32
// arithmetic and still feed the tensor cores exactly what the float64 formula would.
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

bool encode_matrix(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                   uint32_t box_cols) {
  const uint64_t dims[2] = {cols, rows};
  const uint64_t strides[1] = {cols * 4};
  const uint32_t box[2] = {box_cols, box_rows};
  return tma_encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, base, dims, strides, box,
                          CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace

int set_wait_limit_gemm_pair(long long cycles) { return set_wait_limit_here(cycles); }

// The pair kernel takes whole 256-column tiles and 32-deep k-blocks, and only pays when there are
// enough tiles to fill the pairs of the device about twice (below that the single-CTA kernel's
// smaller tiles spread over more SMs).
bool gemm_pair_supported(const tfjs_cuda_ctx* ctx, int64_t M, int64_t K, int64_t N) {
  if (!(N % TILE_N == 0 && K % BLOCK_K == 0 && K >= 128 && M >= PAIR_M && M < (1ll << 31) && N < (1ll << 31)))
    return false;
  const int64_t tiles = ceil_div64(M, PAIR_M) * (N / TILE_N);
  return ctx->gemm_pair >= 2 || tiles >= (int64_t)ctx->sm_count;
}

namespace {

template <int PREC>
int launch_pair_variant(tfjs_cuda_ctx* ctx, const CUtensorMap& ma, const CUtensorMap& mw, const CUtensorMap& mw_lo,
                        const PairParams& p) {
  constexpr int smem_bytes = LAYOUT_BYTES + 1024 <= SMEM_LIMIT ? LAYOUT_BYTES + 1024 : SMEM_LIMIT;
  constexpr bool SPLIT = PREC == PAIR_SPLIT;
  auto kernel = gemm_tcgen05_pair_kernel<PREC>;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(cta_threads(PREC));
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  // per device: the dynamic shared-memory opt-in and how many pairs can be resident at once
  static std::atomic<int> resident_pairs[64];
  int max_pairs = resident_pairs[ctx->device & 63].load(std::memory_order_acquire);
  if (max_pairs == 0) {
    TFJS_CHECK_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    cfg.gridDim = dim3(2 * (unsigned)(ctx->sm_count / 2));
    cfg.numAttrs = 1;
    int clusters = 0;
    TFJS_CHECK_CUDA(ctx, cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg));
    TFJS_REQUIRE(ctx, clusters >= 1, "no CTA pair of the pair GEMM fits on this device");
    max_pairs = clusters < ctx->sm_count / 2 ? clusters : ctx->sm_count / 2;
    resident_pairs[ctx->device & 63].store(max_pairs, std::memory_order_release);
  }
  const int tiles = p.num_m_tiles * p.num_n_tiles;
  const int pairs = tiles < max_pairs ? tiles : max_pairs;
  cfg.gridDim = dim3(2 * (unsigned)pairs);
  cfg.numAttrs = ctx->use_pdl ? 2 : 1;
  cudaLaunchKernelEx(&cfg, kernel, ma, mw, mw_lo, p);
  if (PREC == PAIR_WQ) return post_launch(ctx, "gemm_tcgen05 (TF32, uint8 weights, CTA pairs)");
  return post_launch(ctx, SPLIT ? "gemm_tcgen05 (3xTF32, CTA pairs)" : "gemm_tcgen05 (TF32, CTA pairs)");
}

}  // namespace

// W is the K-major tf32 plane [N, kp] of the packed weights.  With w_lo (the residual plane): 3xTF32,
// A is split into hi / lo on chip.  Without: one TF32 pass; a_tf32_exact says that A's producer
// already rounded it to tf32, otherwise the converter warps round it in shared memory.
int launch_gemm_tcgen05_pair(tfjs_cuda_ctx* ctx, const float* a, int64_t M, int64_t K, const float* w_hi,
                             const float* w_lo, int64_t kp, float* out, int64_t N, const EpilogueArgs& epi,
                             bool a_tf32_exact, const uint8_t* w_q, double q_scale, double q_min) {
  // w_q: the weights as K-major uint8 bytes [N, kp] (then w_hi / w_lo are unused, TF32 only, A tf32-exact)
  CUtensorMap ma, mw, mw_lo;
  bool ok = encode_matrix(&ma, a, (uint64_t)M, (uint64_t)K, CTA_M, BLOCK_K);
  if (w_q) {
    const uint64_t dims[2] = {(uint64_t)kp, (uint64_t)N};
    const uint64_t strides[1] = {(uint64_t)kp};
    const uint32_t box[2] = {BLOCK_K, HALF_N};
    ok = ok && tma_encode_tiled(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, w_q, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
    mw_lo = mw;
  } else {
    ok = ok && encode_matrix(&mw, w_hi, (uint64_t)N, (uint64_t)kp, HALF_N, BLOCK_K) &&
         encode_matrix(&mw_lo, w_lo ? w_lo : w_hi, (uint64_t)N, (uint64_t)kp, HALF_N, BLOCK_K);
  }
  if (!ok) return set_error(ctx, TFJS_CUDA_ERR_CUDA, "cuTensorMapEncodeTiled failed");
  PairParams p;
  p.q_scale = q_scale;
  p.q_min = q_min;
  p.q_scale32 = (float)q_scale;
  p.q_min32 = (float)q_min;
  p.q_arith = (w_q && dequant_exact_in_float32(q_scale, q_min)) ? 1 : 0;
  p.M = (int)M;
  p.N = (int)N;
  p.K = (int)K;
  p.num_m_tiles = (int)ceil_div64(M, PAIR_M);
  p.num_n_tiles = (int)(N / TILE_N);
  p.num_k_blocks = (int)(K / BLOCK_K);
  p.status = ctx->d_status;
  p.out = out;
  p.withhold_last_load = ctx->test_withhold_last_load ? 1 : 0;
  p.epi = epi;
  if (w_q) return launch_pair_variant<PAIR_WQ>(ctx, ma, mw, mw_lo, p);
  if (w_lo) return launch_pair_variant<PAIR_SPLIT>(ctx, ma, mw, mw_lo, p);
  if (a_tf32_exact) return launch_pair_variant<PAIR_ASIS>(ctx, ma, mw, mw_lo, p);
  return launch_pair_variant<PAIR_ROUND>(ctx, ma, mw, mw_lo, p);
}
