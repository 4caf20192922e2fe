// Fused depthwise-separable block for sm_100a:
//   y = act2( pointwise1x1( act1( depthwise3x3(x) + bias1 ) ) + bias2 )
// i.e. KernelBackend.depthwiseConv2D (+ add, clip) followed by fusedConv2d with a 1x1 filter
// (tfjs-core/src/backends/backend.ts:431-434, 414-418; the op pair of tf.separableConv2d,
// ops/conv.ts:574-654, with MobileNet's bias and relu6 between the two).  The depthwise output
// never reaches device memory: it is computed into shared memory as the A operand of the
// pointwise GEMM, which runs on tcgen05 with its accumulator in tensor memory.
//
// One persistent CTA per SM works on patches of 8 x 16 output pixels (= the 128 rows of one MMA):
//   warp 8      producer: per 32-channel k-block, TMA-loads the pointwise weight tile
//               [BLOCK_N x 32] and the input window of the patch ((8-1)*S+3 rows x (16-1)*S+3
//               columns x 32 channels; in two halves of 4 patch rows for stride 2) through a 4-D
//               tensor map whose out-of-range reads return zero, which is SAME padding.  At
//               stride 1 the two kinds of load advance independently, so that the window loads,
//               which carry the DRAM latency, are not held back behind the weight ring.
//   warps 10-17 depthwise: a thread owns 4 channels of a block of output pixels (2 rows x 4
//               columns at stride 1, where the warps form two groups that take alternate
//               k-blocks; 2 adjacent pixels at stride 2), accumulates the 9 taps in the
//               reference's order with one fmaf per tap, adds the bias, applies the activation
//               and writes 16 bytes per pixel of the swizzled K-major A tile (two slots, so the
//               next k-block is computed while the tensor core reads the current one).
//   warp 9      one thread issues tcgen05.mma (M = 128, N = BLOCK_N, K = 8) into one of two TMEM
//               accumulators and commits the barriers that free the slots.
//   warps 0-7   epilogue: tcgen05.ld, bias, activation, swizzled staging, 4-D TMA store of
//               [2 rows x 16 columns x 32 channels] boxes (the store clips patches that overhang
//               the image).
// The arithmetic is that of the two separate kernels, operation for operation, so the results are
// bit-identical to running them back to back.  Every mbarrier wait is bounded.
#include <atomic>

#include "tcgen05_ptx.cuh"

namespace {

constexpr int PH = 8, PW = 16;                    // output patch
constexpr int BLOCK_K = 32;
constexpr int A_TILE_BYTES = 128 * BLOCK_K * 4;   // 16 KB
constexpr int A_SLOTS = 2;
// MODE_RGB in 3xTF32 (see the list of modes below): an A slot holds the hi and the lo tile, a weight
// stage the hi and the lo plane of the filter.
constexpr int MODE_RGB3 = 3;
// MODE_CONV in 3xTF32: the stage the TMA load filled becomes the hi tile, the helper warps write the
// lo tile behind it (a stage is 32 KB), the filter arrives as hi and lo planes.
constexpr int MODE_CONV3 = 5;
__host__ __device__ constexpr bool is_conv(int mode) { return mode == 2 || mode == MODE_CONV3; }
__host__ __device__ constexpr bool is_split3(int mode) { return mode == MODE_RGB3 || mode == MODE_CONV3; }
// Stride-1 depthwise blocks of 256 columns build the A tile IN PLACE: a window (10 x 18 x 128 B = 23 KB) is larger
// than the tile made from it (16 KB), so once the threads of a group have all read their window
// taps into registers (a named barrier) they write the tile over the start of the same stage, the
// tensor core reads it there, and the commit of those MMAs frees the stage for the next load.
// That saves the separate A slots (32 KB), which buys two more window stages: the number of
// window bytes in flight is what bounds these blocks.
// (Only at 256 columns, where the 64 KB of weight stages otherwise leave room for two window stages:
// four in place.  With narrower tiles the ring already holds four, and in place measured slower:
// a stage then stays occupied until its MMAs retire, and the group barrier costs overlap.)
// (Not with half input: its 11.5 KB window is smaller than the 16 KB tile, and four of them fit anyway.)
__host__ __device__ constexpr bool a_in_place(int block_n, int s, int mode, bool in16 = false) {
  return mode == 0 && s == 1 && block_n >= 256 && !in16;
}
__host__ __device__ constexpr int a_slot_bytes(int block_n, int s, int mode, bool in16 = false) {
  return (a_in_place(block_n, s, mode, in16) || is_conv(mode)) ? 0 : A_SLOTS * A_TILE_BYTES * (mode == MODE_RGB3 ? 2 : 1);
}
constexpr int EPI_WARPS = 8;
constexpr int C_CHUNK_BYTES = 32 * 32 * 4;
constexpr int C_STAGING_BYTES = EPI_WARPS * C_CHUNK_BYTES;
constexpr int BIAS_STAGING_BYTES = EPI_WARPS * 128;
constexpr int DW_THREADS = 256;
// The depthwise / im2col threads work as one group of 256 on every k-block (stride-2 depthwise) or as
// two groups of 128 on alternate k-blocks.  With two groups every A slot, raw stage and barrier
// belongs to one group only: a parity wait is only safe for a thread that watches every phase of
// its barrier, and a group does not see the phases of the k-blocks it skips.
__host__ __device__ constexpr int dw_groups(int s, int mode) { return (is_conv(mode) || (mode == 0 && s == 2)) ? 1 : 2; }
constexpr int THREADS = 320 + DW_THREADS;
constexpr int MAX_C = 256;                        // depthwise channels (= K of the GEMM)
constexpr int DW_TABLE_BYTES = 10 * MAX_C * 4;    // 9 filter taps + bias per channel
constexpr int BARRIER_BYTES = 512;
constexpr int SMEM_LIMIT = 232448;

// One raw stage = the input window of PART_ROWS patch rows x 16 columns x 32 channels (every
// pixel a full 128-byte line, so that the window reads are free of bank conflicts).  Stride 2
// doubles the window, so its patch is loaded as two halves of 4 rows.
constexpr int MODE_DW = 0;   // depthwise 3x3 over 32-channel k-blocks feeding the GEMM
constexpr int MODE_RGB = 1;  // dense 3x3 convolution of a 3-channel image: the window rows are turned
                             // into im2col rows (K' = 10 * filter row + 3 * filter column + channel)
                             // MODE_RGB3 (= 3, above) is the same in 3xTF32: the im2col threads write a
                             // tf32 hi and a lo tile, the filter arrives as hi and lo planes, and every
                             // k-step issues hi*hi, lo*hi and hi*lo into the one accumulator (K' is 27
                             // terms long, so the correction terms need no accumulator of their own)
constexpr int MODE_CONV = 2; // dense convolution, Cin a multiple of 32, stride 1: the A tile of k-block
                             // (filter row, filter column, 32-channel group) is the patch shifted by that
                             // tap, loaded by TMA straight into the swizzled layout the tensor core reads;
                             // no thread touches the operands (zero fill of the load is the padding)

// IN16: the input image is stored as IEEE half (16-bit activation storage): a pixel of a k-block
// is a 64-byte line, a window stage half as large.
// IN8 (MODE_RGB only): the image is stored as one unsigned byte per value (pixels), decoded on chip
// as q * scale + min through a 256-entry table; ROW_FLOATS then counts bytes.
template <int S, int MODE, bool IN16 = false, bool IN8 = false>
struct Raw {
  static constexpr int ELEM = IN8 ? 1 : (IN16 ? 2 : 4);
  static constexpr int PIX_BYTES = BLOCK_K * ELEM;       // one pixel of a 32-channel k-block (MODE_DW)
  static constexpr int PARTS = MODE == MODE_DW ? S : 1;  // raw stages per k-block
  static constexpr int PART_ROWS = PH / PARTS;           // patch rows per raw stage
  static constexpr int ROWS = (PART_ROWS - 1) * S + 3;
  static constexpr int COLS = (PW - 1) * S + 3;
  // floats per window row: 32 channels per pixel, or (RGB) 3 per pixel plus up to 3 floats of
  // slack in front so that the copy can start on a 16-byte boundary, rounded up to 16 bytes
  static constexpr int ROW_FLOATS = MODE == MODE_DW ? COLS * BLOCK_K
                                    : (IN8 ? (COLS * 3 + 15 + 15) / 16 * 16 : (COLS * 3 + 3 + 3) / 4 * 4);
  static constexpr int BYTES = is_conv(MODE) ? A_TILE_BYTES : ROWS * ROW_FLOATS * ELEM;   // what the load deposits
  static constexpr int STRIDE = MODE == MODE_CONV3 ? 2 * A_TILE_BYTES : (BYTES + 1023) / 1024 * 1024;
  static constexpr int GROUP_THREADS = DW_THREADS / dw_groups(S, MODE);
  static constexpr int TR = S == 1 ? 2 : 1;                            // a thread's block of outputs: rows
  static constexpr int TC = PW * PART_ROWS * 8 / (TR * GROUP_THREADS);  // and columns (4 / 2)
};

// Weight tiles come from L2 and need little lookahead; at stride 2 and 128 columns two stages
// instead of three make room for a third 38 KB window stage, and the windows carry the DRAM latency.
__host__ __device__ constexpr int w_stages(int block_n, int s, int mode) {
  return block_n >= 256 ? 2 : (block_n >= 128 ? ((mode == 0 && s == 2) ? 2 : 3) : 4);
}
__host__ __device__ constexpr bool is_rgb(int mode) { return mode == MODE_RGB || mode == MODE_RGB3; }
__host__ __device__ constexpr int w_stage_bytes(int block_n, int mode) {
  return block_n * BLOCK_K * 4 * (is_split3(mode) ? 2 : 1);
}
__host__ __device__ constexpr int epi_arrivals(int block_n) { return block_n >= 64 ? EPI_WARPS : 4; }
template <int S, int MODE, bool IN16 = false, bool IN8 = false>
__host__ __device__ constexpr int raw_stages(int block_n) {
  int left = SMEM_LIMIT - 1024 - a_slot_bytes(block_n, S, MODE, IN16) - w_stages(block_n, S, MODE) * w_stage_bytes(block_n, MODE) -
             C_STAGING_BYTES - BIAS_STAGING_BYTES - DW_TABLE_BYTES - BARRIER_BYTES;
  int n = left / Raw<S, MODE, IN16, IN8>::STRIDE;
  // Window loads carry the DRAM latency: about 90 KB must be in flight per SM to keep the memory
  // system busy (four 23 KB float32 windows; with half-size windows that takes eight stages).
  const int cap = (MODE == MODE_DW && !IN16) ? 4 : 8;
  n = n > cap ? cap : n;
  return n / dw_groups(S, MODE) * dw_groups(S, MODE);  // the same number of stages for every group
}

struct SepParams {
  int B, inH, inW, C, outH, outW, N;
  int pad_r, pad_c;                 // first input row / column of output (0, 0) is -pad
  int tiles_y, tiles_x, num_tiles, num_k_blocks;
  const float* dw_filter;           // [3, 3, C, 1]
  const float* dw_bias;             // [C] or null
  int dw_bias_scalar;
  int dw_act;
  float dw_lo, dw_hi;
  EpilogueArgs epi;                 // of the pointwise convolution
  int rgb_off;                      // MODE_RGB: floats (bytes for byte input) between the 16-byte aligned copy start and the window
  double q_scale, q_min;            // MODE_RGB with byte input: value = q * q_scale + q_min
  int fh, fw, dil_h, dil_w, cin_groups;  // MODE_CONV: filter size, dilation, Cin / 32
  int* status;
};

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0,
                                            int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0,
                                            int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ float lds32(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2,
                                             int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(map),
               "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
__device__ __forceinline__ float4 lds128(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}
// the same 16 bytes as two packed float pairs (x, y) and (z, w)
__device__ __forceinline__ void lds128_pairs(uint32_t addr, uint64_t& lo, uint64_t& hi) {
  asm volatile("ld.shared.v2.b64 {%0, %1}, [%2];" : "=l"(lo), "=l"(hi) : "r"(addr));
}
__device__ __forceinline__ void sts128(uint32_t addr, const float4& v) {
  asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}
// Four channels of a window pixel as two packed float pairs, from float32 (16 bytes) or IEEE half
// (8 bytes, converted exactly).
template <bool IN16>
__device__ __forceinline__ void lds_quad_pairs(uint32_t addr, uint64_t& lo, uint64_t& hi) {
  if (!IN16) {
    lds128_pairs(addr, lo, hi);
  } else {
    uint32_t a, b;
    asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(a), "=r"(b) : "r"(addr));
    float x, y, z, w;
    unpack_half2(a, x, y);
    unpack_half2(b, z, w);
    lo = pack_f32x2(__float_as_uint(x), __float_as_uint(y));
    hi = pack_f32x2(__float_as_uint(z), __float_as_uint(w));
  }
}

template <int ACT>
__device__ __forceinline__ float dw_activate(float v, float lo, float hi) {
  if (ACT == TFJS_ACT_RELU) return max_nan(v, 0.f);
  if (ACT == TFJS_ACT_CLIP) return min_nan(max_nan(v, lo), hi);
  return v;
}

// Depthwise 3x3 of one raw stage by one group of threads: thread t computes a block of TR output
// rows x TC columns (2 x 4 at stride 1, 1 x 2 at stride 2) x 4 channels from the window in shared
// memory and writes it into the A tile.  `table` holds the 9 filter taps and the bias of every
// channel ([10][C] floats).  The block shares window rows between its output rows and filter
// taps between all its pixels, which is what bounds the kernel: every 16-byte read costs a
// quarter-warp wavefront of the shared-memory pipe.  The window is walked row by row and entry by
// entry, so each output still accumulates its taps in the order (wR, wC) ascending.
template <int S, int ACT, bool IN16>
__device__ __forceinline__ void dw_part(uint32_t raw, uint32_t a_tile, uint32_t table, int t, int part, int kb,
                                        const SepParams& p, bool has_bias, int sync_id) {
  using R = Raw<S, MODE_DW, IN16>;
  constexpr int TR = R::TR, TC = R::TC;
  constexpr int GROUPS_PER_ROW = PW / TC;
  constexpr int WROWS = (TR - 1) * S + 3, WIN = (TC - 1) * S + 3;
  static_assert((R::PART_ROWS / TR) * GROUPS_PER_ROW * 8 == R::GROUP_THREADS, "one block per thread");
  const int q = t & 7;                         // channel quad of the k-block
  const int g = t >> 3;
  const int r0 = (g / GROUPS_PER_ROW) * TR;    // first output row inside this part
  const int c0 = (g % GROUPS_PER_ROW) * TC;
  const int ch = kb * BLOCK_K + q * 4;
  // the four channels travel as two packed float pairs: one fma.rn.f32x2 does two of the taps'
  // multiply-adds, each lane rounding exactly like fmaf
  uint64_t acc[TR][TC][2];
  uint64_t f[3][3][2];
#pragma unroll
  for (int o = 0; o < TR; o++)
#pragma unroll
    for (int j = 0; j < TC; j++) acc[o][j][0] = acc[o][j][1] = 0ull;
#pragma unroll
  for (int ir = 0; ir < WROWS; ir++) {
    if (ir < 3) {
#pragma unroll
      for (int wc = 0; wc < 3; wc++)
        lds128_pairs(table + (uint32_t)(((ir * 3 + wc) * p.C + ch) * 4), f[ir][wc][0], f[ir][wc][1]);
    }
    const uint32_t row = raw + (uint32_t)((((r0 * S + ir) * R::COLS) + c0 * S) * R::PIX_BYTES + q * 4 * R::ELEM);
#pragma unroll
    for (int i = 0; i < WIN; i++) {
      uint64_t in0, in1;
      lds_quad_pairs<IN16>(row + i * R::PIX_BYTES, in0, in1);
#pragma unroll
      for (int o = 0; o < TR; o++) {
        const int dr = ir - o * S;  // filter row of this window row for output row o
        if (dr < 0 || dr > 2) continue;
#pragma unroll
        for (int wc = 2; wc >= 0; wc--) {
          const int d = i - wc;     // = j * S for the output column j this entry is tap wc of
          if (d < 0 || d % S != 0 || d / S >= TC) continue;
          acc[o][d / S][0] = fma_f32x2(in0, f[dr][wc][0], acc[o][d / S][0]);
          acc[o][d / S][1] = fma_f32x2(in1, f[dr][wc][1], acc[o][d / S][1]);
        }
      }
    }
  }
  uint64_t b0, b1;
  lds128_pairs(table + (uint32_t)((9 * p.C + ch) * 4), b0, b1);
  // When the tile is written over its own window (sync_id > 0), every thread of the group must
  // have its window taps in registers first.
  if (sync_id > 0) asm volatile("bar.sync %0, %1;" ::"r"(sync_id), "n"(R::GROUP_THREADS) : "memory");
#pragma unroll
  for (int o = 0; o < TR; o++) {
    const int m0 = (part * R::PART_ROWS + r0 + o) * PW + c0;  // first of this row's rows of the A tile
#pragma unroll
    for (int j = 0; j < TC; j++) {
      if (has_bias) {
        acc[o][j][0] = add_f32x2(acc[o][j][0], b0);
        acc[o][j][1] = add_f32x2(acc[o][j][1], b1);
      }
      uint32_t ox, oy, oz, ow;
      unpack_f32x2(acc[o][j][0], ox, oy);
      unpack_f32x2(acc[o][j][1], oz, ow);
      // rounded to the nearest tf32 value: the tensor core reads the upper 19 bits only, and
      // truncating these (non-negative, after relu6) values would bias every sum downwards
      float4 v;
      v.x = round_tf32_after_arith(dw_activate<ACT>(__uint_as_float(ox), p.dw_lo, p.dw_hi));
      v.y = round_tf32_after_arith(dw_activate<ACT>(__uint_as_float(oy), p.dw_lo, p.dw_hi));
      v.z = round_tf32_after_arith(dw_activate<ACT>(__uint_as_float(oz), p.dw_lo, p.dw_hi));
      v.w = round_tf32_after_arith(dw_activate<ACT>(__uint_as_float(ow), p.dw_lo, p.dw_hi));
      sts128(a_tile + swz(m0 + j, q * 16), v);
    }
  }
}

// MODE_RGB: thread t of a group turns the 3 x 9 window floats of output pixel t (3 filter rows of 3 pixels
// x 3 channels, contiguous in the NHWC image) into row t of the A tile, in the K' order the repacked
// filter uses: floats 10*wr + 3*wc + ci, with zeros at 9, 19 and 29..31.
// (y0, x0): input row / column of the tile's first window element.  Byte input only: the zero fill
// of a load outside the image is the BYTE 0, which decodes to `min`, not to the 0.0 that padding
// means, so taps outside the image are set to zero here.
template <int S, bool IN8, bool SPLIT3 = false>
__device__ __forceinline__ void rgb_part(uint32_t raw, uint32_t a_tile, int t, const SepParams& p, uint32_t lut,
                                         int y0, int x0) {
  using R = Raw<S, MODE_RGB, false, IN8>;
  const int r = t / PW, c = t % PW;
  float v[3][9];
#pragma unroll
  for (int dr = 0; dr < 3; dr++) {
    if (IN8) {
      // pixel bytes -> float through the table of decoded (and tf32-rounded) values
      const uint32_t row = raw + (uint32_t)((r * S + dr) * R::ROW_FLOATS + p.rgb_off + c * S * 3);
      const int yi = y0 + r * S + dr;
      const bool row_in = yi >= 0 && yi < p.inH;
#pragma unroll
      for (int j = 0; j < 9; j++) {
        uint32_t q;
        asm volatile("ld.shared.u8 %0, [%1];" : "=r"(q) : "r"(row + j));
        const int xi = x0 + c * S + j / 3;
        v[dr][j] = (row_in && xi >= 0 && xi < p.inW) ? lds32(lut + q * 4) : 0.f;
      }
    } else {
      const uint32_t row = raw + (uint32_t)(((r * S + dr) * R::ROW_FLOATS + p.rgb_off + c * S * 3) * 4);
#pragma unroll
      for (int j = 0; j < 9; j++)
        v[dr][j] = SPLIT3 ? lds32(row + j * 4) : round_tf32_for_mma(lds32(row + j * 4));  // the tensor core would truncate
    }
  }
  if (SPLIT3) {
    // 3xTF32: hi = tf32(x) goes to the slot's first tile, lo = tf32(x - hi) to its second (a
    // non-finite hi keeps lo at zero: inf - inf would poison the product with NaN)
    float lo[3][9];
#pragma unroll
    for (int dr = 0; dr < 3; dr++)
#pragma unroll
      for (int j = 0; j < 9; j++) {
        const float h = round_tf32(v[dr][j]);
        lo[dr][j] = (fabsf(h) <= 3.4028234e38f) ? round_tf32(v[dr][j] - h) : 0.f;
        v[dr][j] = h;
      }
    const uint32_t lo_tile = a_tile + A_TILE_BYTES;
    sts128(lo_tile + swz(t, 0), make_float4(lo[0][0], lo[0][1], lo[0][2], lo[0][3]));
    sts128(lo_tile + swz(t, 16), make_float4(lo[0][4], lo[0][5], lo[0][6], lo[0][7]));
    sts128(lo_tile + swz(t, 32), make_float4(lo[0][8], 0.f, lo[1][0], lo[1][1]));
    sts128(lo_tile + swz(t, 48), make_float4(lo[1][2], lo[1][3], lo[1][4], lo[1][5]));
    sts128(lo_tile + swz(t, 64), make_float4(lo[1][6], lo[1][7], lo[1][8], 0.f));
    sts128(lo_tile + swz(t, 80), make_float4(lo[2][0], lo[2][1], lo[2][2], lo[2][3]));
    sts128(lo_tile + swz(t, 96), make_float4(lo[2][4], lo[2][5], lo[2][6], lo[2][7]));
    sts128(lo_tile + swz(t, 112), make_float4(lo[2][8], 0.f, 0.f, 0.f));
  }
  sts128(a_tile + swz(t, 0), make_float4(v[0][0], v[0][1], v[0][2], v[0][3]));
  sts128(a_tile + swz(t, 16), make_float4(v[0][4], v[0][5], v[0][6], v[0][7]));
  sts128(a_tile + swz(t, 32), make_float4(v[0][8], 0.f, v[1][0], v[1][1]));
  sts128(a_tile + swz(t, 48), make_float4(v[1][2], v[1][3], v[1][4], v[1][5]));
  sts128(a_tile + swz(t, 64), make_float4(v[1][6], v[1][7], v[1][8], 0.f));
  sts128(a_tile + swz(t, 80), make_float4(v[2][0], v[2][1], v[2][2], v[2][3]));
  sts128(a_tile + swz(t, 96), make_float4(v[2][4], v[2][5], v[2][6], v[2][7]));
  sts128(a_tile + swz(t, 112), make_float4(v[2][8], 0.f, 0.f, 0.f));
}

// HALF: 16-bit activation storage.  The output is stored as IEEE half, and in MODE_DW the input
// is read as IEEE half; the stem (MODE_RGB) keeps its float32 input image.  The arithmetic does not
// change: float32 depthwise taps, tf32 tensor-core products, float32 accumulators and epilogue.
// IN8 (MODE_RGB): the input image is stored as bytes and decoded on chip as q * q_scale + q_min.
template <int BLOCK_N, int S, int MODE, bool HALF = false, bool IN8 = false>
__global__ void __launch_bounds__(THREADS, 1)
sepconv_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                       const __grid_constant__ CUtensorMap map_w_lo, const __grid_constant__ CUtensorMap map_y,
                       SepParams p) {
  static_assert(!IN8 || MODE == MODE_RGB, "byte input is the 3-channel stem's");
  constexpr bool SPLIT3 = is_split3(MODE);
  constexpr int A_SLOT_STRIDE = A_TILE_BYTES * (SPLIT3 ? 2 : 1);
  constexpr bool IN16 = HALF && MODE == MODE_DW;
  constexpr bool OUT16 = HALF;
  using R = Raw<S, MODE, IN16, IN8>;
  constexpr int W_STAGES = w_stages(BLOCK_N, S, MODE);
  constexpr int GROUPS = dw_groups(S, MODE);
  constexpr int GROUP_THREADS = DW_THREADS / GROUPS;
  constexpr int RAW_STAGES = raw_stages<S, MODE, IN16, IN8>(BLOCK_N);
  static_assert(RAW_STAGES >= 2 && RAW_STAGES % GROUPS == 0 && A_SLOTS % GROUPS == 0, "rings split evenly");
  constexpr bool IN_PLACE = a_in_place(BLOCK_N, S, MODE, IN16);
  // MODE_CONV: the stage the TMA load filled IS the A tile; the helper warps only round it to tf32
  // in place before the tensor core reads it
  constexpr bool STAGE_IS_A = IN_PLACE || is_conv(MODE);
  constexpr int NUM_A = STAGE_IS_A ? RAW_STAGES : A_SLOTS;  // A tiles (and their full barriers)
  static_assert(!IN_PLACE || (R::BYTES >= A_TILE_BYTES && R::STRIDE % 1024 == 0), "the tile fits its window's stage");
  static_assert(GROUPS == 1 || R::PARTS == 1, "two groups take whole k-blocks of one raw stage each");
  // Where k-block n of this CTA (counted over all its tiles) lives: with two groups, group n % 2
  // owns slots / stages [group * size / 2, (group + 1) * size / 2) and cycles through them.
  auto ring_pos = [](int seq, int size, int& index, uint32_t& phase) {
    const int per_group = size / GROUPS;
    const int group = seq % GROUPS, turn = seq / GROUPS;
    index = group * per_group + turn % per_group;
    phase = (uint32_t)(turn / per_group) & 1u;
  };
  constexpr int W_STAGE_BYTES = w_stage_bytes(BLOCK_N, MODE);
  constexpr int W_PLANE_BYTES = BLOCK_N * BLOCK_K * 4;
  // Accumulator buffers in tensor memory: two, or four when a tile is only 32 columns wide; then
  // each half of the epilogue warps drains every other tile, so two epilogues run at a time.
  constexpr int NUM_ACC = BLOCK_N == 32 ? 4 : 2;
  constexpr uint32_t TMEM_COLS = NUM_ACC * BLOCK_N;  // 128 .. 512
  // who frees a raw stage: the depthwise / im2col threads that read it, or (MODE_CONV, where the
  // stage is the A operand itself) the commit of the MMAs that read it
  // (one arrival per warp, by lane 0 after __syncwarp: 256 single-thread arrivals on one barrier
  // serialise in the shared-memory pipe, which is the busiest unit of this kernel)
  constexpr int RAW_READERS = is_conv(MODE) ? 1 : GROUP_THREADS / 32;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* a_tiles = smem;                                   // [A_SLOTS][16 KB], SWIZZLE_128B (none if in place)
  uint8_t* w_tiles = a_tiles + a_slot_bytes(BLOCK_N, S, MODE, IN16);  // [W_STAGES][BLOCK_N x 128 B]
  uint8_t* c_stage = w_tiles + W_STAGES * W_STAGE_BYTES;     // [8 warps][4 KB]
  uint8_t* raw = c_stage + C_STAGING_BYTES;                  // [RAW_STAGES][window]
  uint8_t* table = raw + RAW_STAGES * R::STRIDE;             // [10][C] floats
  uint8_t* bias_stage = table + DW_TABLE_BYTES;
  uint64_t* bars = (uint64_t*)(bias_stage + BIAS_STAGING_BYTES);
  uint64_t* raw_full = bars;                       // [RAW_STAGES] TMA -> depthwise warps
  uint64_t* raw_empty = raw_full + RAW_STAGES;     // [RAW_STAGES] depthwise warps -> TMA
  uint64_t* w_full = raw_empty + RAW_STAGES;       // [W_STAGES] TMA -> MMA
  uint64_t* w_empty = w_full + W_STAGES;           // [W_STAGES] MMA -> TMA
  uint64_t* a_full = w_empty + W_STAGES;           // [NUM_A] depthwise warps -> MMA
  uint64_t* a_empty = a_full + NUM_A;              // [NUM_A] MMA -> depthwise warps (unused if in place)
  uint64_t* tmem_full_bar = a_empty + NUM_A;             // [NUM_ACC] MMA -> epilogue
  uint64_t* tmem_empty_bar = tmem_full_bar + NUM_ACC;    // [NUM_ACC] epilogue -> MMA
  uint32_t* tmem_ptr_holder = (uint32_t*)(tmem_empty_bar + NUM_ACC);
  volatile int* abort_flag = (volatile int*)(tmem_ptr_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (threadIdx.x == 32 * 8) {  // the producer warp's first lane: descriptors on their way before the set-up below
    prefetch_tensormap(&map_x);
    prefetch_tensormap(&map_w);
    if (SPLIT3) prefetch_tensormap(&map_w_lo);
    prefetch_tensormap(&map_y);
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < RAW_STAGES; s++) {
      mbar_init(smem_u32(&raw_full[s]), 1);
      mbar_init(smem_u32(&raw_empty[s]), IN_PLACE ? 1 : RAW_READERS);  // in place: freed by the MMAs' commit
    }
    for (int s = 0; s < W_STAGES; s++) {
      mbar_init(smem_u32(&w_full[s]), 1);
      mbar_init(smem_u32(&w_empty[s]), 1);
    }
    for (int s = 0; s < NUM_A; s++) {
      mbar_init(smem_u32(&a_full[s]), GROUP_THREADS / 32);
      mbar_init(smem_u32(&a_empty[s]), 1);
    }
    for (int a = 0; a < NUM_ACC; a++) {
      mbar_init(smem_u32(&tmem_full_bar[a]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[a]), epi_arrivals(BLOCK_N));
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 9) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_ptr_holder)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // only shared and tensor memory was touched so far; global memory from here on
  pdl_wait();
  pdl_launch_dependents();
  // depthwise filter taps and bias of every channel: [tap][C], then the bias row
  if (MODE == MODE_DW) {
    float* tab = reinterpret_cast<float*>(table);
    for (int i = threadIdx.x; i < 9 * p.C; i += THREADS) tab[i] = __ldg(p.dw_filter + i);
    for (int i = threadIdx.x; i < p.C; i += THREADS)
      tab[9 * p.C + i] = p.dw_bias ? __ldg(p.dw_bias + (p.dw_bias_scalar ? 0 : i)) : 0.f;
  }
  if (IN8) {
    // the 256 byte values decoded once per CTA, q * scale + min in float64 as decodeWeights does
    // (io_utils.ts:139), already rounded for the tensor core
    float* lut = reinterpret_cast<float*>(table);
    for (int q = threadIdx.x; q < 256; q += THREADS)
      lut[q] = round_tf32_for_mma((float)((double)q * p.q_scale + p.q_min));
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_ptr_holder;
  const int tiles_per_image = p.tiles_y * p.tiles_x;

  if (warp == 8) {
    // ---------------- TMA producer ----------------
    // With two groups: two independent cursors, one over the weight tiles and one over the raw stages,
    // advanced by polling: a weight stage is only free once the MMAs three k-blocks back have retired, and an
    // in-order producer would hold the input loads back behind it although the raw ring has room.
    // The input loads carry the DRAM latency, so they must run as far ahead as their ring allows.
    // (Prefetching the windows into L2 a few k-blocks ahead as well measured slower on every block.)
    if (lane == 0 && GROUPS == 1) {
      // one group of consumers works through both rings at the same pace: plain in-order issue
      int rn = 0, ws = 0;
      uint32_t wphase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
        const int b = tile / tiles_per_image;
        const int rem = tile - b * tiles_per_image;
        const int ty = rem / p.tiles_x, tx = rem - ty * p.tiles_x;
        const int x0 = tx * PW * S - p.pad_c, y0 = ty * PH * S - p.pad_r;
        for (int kb = 0; kb < p.num_k_blocks && ok; kb++) {
          ok = mbar_wait(smem_u32(&w_empty[ws]), wphase ^ 1, abort_flag, p.status, 11);
          if (!ok) break;
          mbar_arrive_expect_tx(smem_u32(&w_full[ws]), W_STAGE_BYTES);
          tma_load_2d(smem_u32(w_tiles + ws * W_STAGE_BYTES), &map_w, smem_u32(&w_full[ws]), kb * BLOCK_K, 0);
          if (SPLIT3)
            tma_load_2d(smem_u32(w_tiles + ws * W_STAGE_BYTES + W_PLANE_BYTES), &map_w_lo, smem_u32(&w_full[ws]),
                        kb * BLOCK_K, 0);
          if (++ws == W_STAGES) { ws = 0; wphase ^= 1; }
          for (int part = 0; part < R::PARTS; part++, rn++) {
            int rs;
            uint32_t rphase;
            ring_pos(rn, RAW_STAGES, rs, rphase);
            ok = mbar_wait(smem_u32(&raw_empty[rs]), rphase ^ 1, abort_flag, p.status, 12);
            if (!ok) break;
            mbar_arrive_expect_tx(smem_u32(&raw_full[rs]), R::BYTES);
            if (is_conv(MODE)) {
              const int tap = kb / p.cin_groups, cg = kb - tap * p.cin_groups;
              const int wr = tap / p.fw, wc = tap - wr * p.fw;
              tma_load_4d(smem_u32(raw + rs * R::STRIDE), &map_x, smem_u32(&raw_full[rs]), cg * BLOCK_K,
                          x0 + wc * p.dil_w, y0 + wr * p.dil_h, b);
            } else {
              tma_load_4d(smem_u32(raw + rs * R::STRIDE), &map_x, smem_u32(&raw_full[rs]), kb * BLOCK_K, x0,
                          y0 + part * R::PART_ROWS * S, b);
            }
          }
        }
      }
    } else if (lane == 0) {
      int w_tile = blockIdx.x, w_kb = 0, ws = 0;
      uint32_t wphase = 0;
      int r_tile = blockIdx.x, r_kb = 0, r_part = 0, rn = 0;  // rn: raw stages requested so far
      long long t0 = clock64();
      uint32_t idle = 0;
      while (w_tile < p.num_tiles || r_tile < p.num_tiles) {
        bool progressed = false;
        if (r_tile < p.num_tiles) {
          int rs;
          uint32_t rphase;
          ring_pos(rn, RAW_STAGES, rs, rphase);
          if (mbar_test_wait(smem_u32(&raw_empty[rs]), rphase ^ 1)) {
            const int b = r_tile / tiles_per_image;
            const int rem = r_tile - b * tiles_per_image;
            const int ty = rem / p.tiles_x, tx = rem - ty * p.tiles_x;
            const int x0 = tx * PW * S - p.pad_c, y0 = ty * PH * S - p.pad_r;
            mbar_arrive_expect_tx(smem_u32(&raw_full[rs]), R::BYTES);
            if (MODE == MODE_DW)
              tma_load_4d(smem_u32(raw + rs * R::STRIDE), &map_x, smem_u32(&raw_full[rs]), r_kb * BLOCK_K, x0,
                          y0 + r_part * R::PART_ROWS * S, b);
            else  // image rows as runs of W*3 floats; the copy starts rgb_off floats before the window
              tma_load_3d(smem_u32(raw + rs * R::STRIDE), &map_x, smem_u32(&raw_full[rs]), x0 * 3 - p.rgb_off,
                          y0, b);
            rn++;
            if (++r_part == R::PARTS) {
              r_part = 0;
              if (++r_kb == p.num_k_blocks) { r_kb = 0; r_tile += gridDim.x; }
            }
            progressed = true;
          }
        }
        if (w_tile < p.num_tiles && mbar_test_wait(smem_u32(&w_empty[ws]), wphase ^ 1)) {
          mbar_arrive_expect_tx(smem_u32(&w_full[ws]), W_STAGE_BYTES);
          tma_load_2d(smem_u32(w_tiles + ws * W_STAGE_BYTES), &map_w, smem_u32(&w_full[ws]), w_kb * BLOCK_K, 0);
          if (SPLIT3)
            tma_load_2d(smem_u32(w_tiles + ws * W_STAGE_BYTES + W_PLANE_BYTES), &map_w_lo, smem_u32(&w_full[ws]),
                        w_kb * BLOCK_K, 0);
          if (++ws == W_STAGES) { ws = 0; wphase ^= 1; }
          if (++w_kb == p.num_k_blocks) { w_kb = 0; w_tile += gridDim.x; }
          progressed = true;
        }
        if (progressed) {
          idle = 0;
          continue;
        }
        // bounded: give up when nothing moved for the wait limit, or another role already gave up
        __nanosleep(64);  // each poll is a shared-memory access: keep them rare
        if (++idle == 1) t0 = clock64();
        if ((idle & 63) == 63) {
          if (*abort_flag) break;
          if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
            *abort_flag = 1;
            atomicCAS(p.status, 0, 12);
            break;
          }
        }
      }
    }
  } else if (warp == 9) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(128, BLOCK_N);
      int ws = 0, local = 0, n = 0;  // n: k-blocks so far
      uint32_t wphase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, local++) {
        const int acc = local % NUM_ACC;
        const uint32_t acc_phase = (local / NUM_ACC) & 1;
        ok = mbar_wait(smem_u32(&tmem_empty_bar[acc]), acc_phase ^ 1, abort_flag, p.status, 13);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BLOCK_N;
        for (int kb = 0; kb < p.num_k_blocks; kb++, n++) {
          int slot, rs;
          uint32_t sphase, rphase;
          ring_pos(n, RAW_STAGES, rs, rphase);  // MODE_CONV and in place: one raw stage per k-block
          if (IN_PLACE) {
            slot = rs;
            sphase = rphase;
          } else {
            ring_pos(n, A_SLOTS, slot, sphase);
          }
          ok = mbar_wait(smem_u32(&w_full[ws]), wphase, abort_flag, p.status, 14);
          if (ok && is_conv(MODE)) ok = mbar_wait(smem_u32(&a_full[rs]), rphase, abort_flag, p.status, 15);
          if (ok && !is_conv(MODE)) ok = mbar_wait(smem_u32(&a_full[slot]), sphase, abort_flag, p.status, 15);
          if (!ok) break;
          tcgen05_fence_after();
          const uint32_t a_s = STAGE_IS_A ? smem_u32(raw + rs * R::STRIDE)
                                                               : smem_u32(a_tiles + slot * A_SLOT_STRIDE);
          const uint32_t w_s = smem_u32(w_tiles + ws * W_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BLOCK_K / 8; k++) {
            tcgen05_mma_tf32(tmem_d, make_smem_desc(a_s + k * 32), make_smem_desc(w_s + k * 32), idesc,
                             (kb > 0 || k > 0) ? 1u : 0u);
            if (SPLIT3) {  // lo * hi and hi * lo
              tcgen05_mma_tf32(tmem_d, make_smem_desc(a_s + A_TILE_BYTES + k * 32), make_smem_desc(w_s + k * 32), idesc, 1u);
              tcgen05_mma_tf32(tmem_d, make_smem_desc(a_s + k * 32), make_smem_desc(w_s + W_PLANE_BYTES + k * 32), idesc, 1u);
            }
          }
          tcgen05_commit(smem_u32(&w_empty[ws]));
          if (STAGE_IS_A)
            tcgen05_commit(smem_u32(&raw_empty[rs]));
          else
            tcgen05_commit(smem_u32(&a_empty[slot]));
          if (++ws == W_STAGES) { ws = 0; wphase ^= 1; }
        }
        if (ok) tcgen05_commit(smem_u32(&tmem_full_bar[acc]));
      }
    }
  } else if (warp >= 10 && is_conv(MODE)) {
    // ---------------- rounding warps ----------------
    // The A tile arrives from TMA in the layout the tensor core reads, as raw float32.  The tensor
    // core would truncate it to tf32; these 256 threads round it to nearest in place (element-wise,
    // so the swizzled placement is untouched) and hand the stage on.
    const int t = threadIdx.x - 320;
    int n = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
      for (int kb = 0; kb < p.num_k_blocks && ok; kb++, n++) {
        int rs;
        uint32_t rphase;
        ring_pos(n, RAW_STAGES, rs, rphase);
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&raw_full[rs]), rphase, abort_flag, p.status, 17));
        if (!ok) break;
        float4* tile4 = reinterpret_cast<float4*>(raw + rs * R::STRIDE);
#pragma unroll
        for (int i = 0; i < A_TILE_BYTES / 16 / DW_THREADS; i++) {
          float4 v = tile4[t + i * DW_THREADS];
          if (SPLIT3) {
            // 3xTF32: hi = tf32(a) in place, lo = tf32(a - hi) into the tile behind it (a non-finite
            // hi keeps lo at zero: inf - inf would poison the product with NaN)
            float4 h, l;
            h.x = round_tf32(v.x); h.y = round_tf32(v.y); h.z = round_tf32(v.z); h.w = round_tf32(v.w);
            l.x = (fabsf(h.x) <= 3.4028234e38f) ? round_tf32(v.x - h.x) : 0.f;
            l.y = (fabsf(h.y) <= 3.4028234e38f) ? round_tf32(v.y - h.y) : 0.f;
            l.z = (fabsf(h.z) <= 3.4028234e38f) ? round_tf32(v.z - h.z) : 0.f;
            l.w = (fabsf(h.w) <= 3.4028234e38f) ? round_tf32(v.w - h.w) : 0.f;
            tile4[t + i * DW_THREADS] = h;
            tile4[A_TILE_BYTES / 16 + t + i * DW_THREADS] = l;
            continue;
          }
          v.x = round_tf32_for_mma(v.x); v.y = round_tf32_for_mma(v.y);
          v.z = round_tf32_for_mma(v.z); v.w = round_tf32_for_mma(v.w);
          tile4[t + i * DW_THREADS] = v;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&a_full[rs]));
      }
    }
  } else if (warp >= 10) {
    // ---------------- depthwise warps ----------------
    // With two groups, each takes every other k-block (counted over all the tiles of this CTA), so
    // that two A tiles are in the making at any time.
    const int t = (threadIdx.x - 320) % GROUP_THREADS;
    const int group = (threadIdx.x - 320) / GROUP_THREADS;
    const uint32_t table_s = smem_u32(table);
    const bool has_bias = p.dw_bias != nullptr;
    int n = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
      for (int kb = 0; kb < p.num_k_blocks && ok; kb++, n++) {
        if (n % GROUPS != group) continue;
        int slot = 0;
        uint32_t sphase = 0;
        uint32_t a_s = 0;
        if (!IN_PLACE) {
          ring_pos(n, A_SLOTS, slot, sphase);
          ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&a_empty[slot]), sphase ^ 1, abort_flag, p.status, 16));
          if (!ok) break;
          a_s = smem_u32(a_tiles + slot * A_SLOT_STRIDE);
        }
        for (int part = 0; part < R::PARTS; part++) {
          int rs;
          uint32_t rphase;
          ring_pos(n * R::PARTS + part, RAW_STAGES, rs, rphase);
          ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&raw_full[rs]), rphase, abort_flag, p.status, 17));
          if (!ok) break;
          const uint32_t raw_s = smem_u32(raw + rs * R::STRIDE);
          if (IN_PLACE) {  // the tile replaces its own window; the stage's index is the tile's
            a_s = raw_s;
            slot = rs;
          }
          if (is_rgb(MODE)) {
            const int img = tile / tiles_per_image;
            const int rem = tile - img * tiles_per_image;
            const int ty = rem / p.tiles_x, tx = rem - ty * p.tiles_x;
            rgb_part<S, IN8, SPLIT3>(raw_s, a_s, t, p, table_s, ty * PH * S - p.pad_r, tx * PW * S - p.pad_c);
          } else {
            // in place: named barrier 1 + group over the group's threads, between reads and writes
            const int sync_id = IN_PLACE ? 1 + group : 0;
            switch (p.dw_act) {
              case TFJS_ACT_RELU: dw_part<S, TFJS_ACT_RELU, IN16>(raw_s, a_s, table_s, t, part, kb, p, has_bias, sync_id); break;
              case TFJS_ACT_CLIP: dw_part<S, TFJS_ACT_CLIP, IN16>(raw_s, a_s, table_s, t, part, kb, p, has_bias, sync_id); break;
              default: dw_part<S, TFJS_ACT_LINEAR, IN16>(raw_s, a_s, table_s, t, part, kb, p, has_bias, sync_id); break;
            }
          }
          if (!IN_PLACE) {
            __syncwarp();  // every lane has read all it needs of the window
            if (lane == 0) mbar_arrive(smem_u32(&raw_empty[rs]));
          }
        }
        if (!ok) break;
        fence_proxy_async_smem();  // generic-proxy writes of the A tile -> visible to the tensor core
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&a_full[slot]));
      }
    }
  } else {
    // ---------------- epilogue warps 0-7 ----------------
    // Warps w and w+4 share TMEM lane quarter w%4 (patch rows 2*(w%4), 2*(w%4)+1) and split the
    // 32-channel chunks of the tile between them.
    constexpr int CHUNKS = BLOCK_N / 32;
    constexpr int MY_CHUNKS = CHUNKS >= 2 ? CHUNKS / 2 : 1;
    const int quarter = warp & 3;
    const int half = warp >> 2;
    {
    uint8_t* stage_buf = c_stage + warp * C_CHUNK_BYTES;
    float* bias_s = reinterpret_cast<float*>(bias_stage + warp * 128);
    const bool has_bias = p.epi.bias != nullptr;
    int local = 0;
    int store_parity = 0;  // OUT16: which half of the staging buffer the next chunk uses
    bool ok = true;
    for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, local++) {
      const int b = tile / tiles_per_image;
      const int rem = tile - b * tiles_per_image;
      const int ty = rem / p.tiles_x, tx = rem - ty * p.tiles_x;
      if (CHUNKS == 1 && (local & 1) != half) continue;  // 32-wide tiles alternate between the halves
      const int acc = local % NUM_ACC;
      const uint32_t acc_phase = (local / NUM_ACC) & 1;
      float bias_l[MY_CHUNKS];
#pragma unroll
      for (int i = 0; i < MY_CHUNKS; i++) {
        const int cl = (CHUNKS >= 2 ? 2 * i + half : 0) * 32 + lane;
        bias_l[i] = 0.f;
        if (has_bias) bias_l[i] = p.epi.bias_scalar ? __ldg(p.epi.bias) : (cl < p.N ? __ldg(p.epi.bias + cl) : 0.f);
      }
      ok = mbar_wait(smem_u32(&tmem_full_bar[acc]), acc_phase, abort_flag, p.status, 18);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BLOCK_N;
      bool released = false;
#pragma unroll
      for (int i = 0; i < MY_CHUNKS; i++) {
        const int chunk = CHUNKS >= 2 ? 2 * i + half : 0;
        const int c0 = chunk * 32;
        if (c0 >= p.N) break;
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + chunk * 32, r);
        __syncwarp();
        bias_s[lane] = bias_l[i];
        tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int k = 0; k < 32; k++) v[k] = __uint_as_float(r[k]);
        __syncwarp();
        if (i == MY_CHUNKS - 1) {
          tcgen05_fence_before();
          if (lane == 0) mbar_arrive(smem_u32(&tmem_empty_bar[acc]));
          released = true;
        }
        switch (p.epi.activation) {
          case TFJS_ACT_RELU: finish_chunk<TFJS_ACT_RELU>(v, has_bias, bias_s, bias_s, p.epi); break;
          case TFJS_ACT_CLIP: finish_chunk<TFJS_ACT_CLIP>(v, has_bias, bias_s, bias_s, p.epi); break;
          default: finish_chunk<TFJS_ACT_LINEAR>(v, has_bias, bias_s, bias_s, p.epi); break;
        }
        // A half chunk is 2 KB of the warp's 4 KB staging buffer: the two halves alternate, so one
        // store may still be reading its half while the next chunk is written (stores in flight
        // are what bounds the write rate of the narrow layers).
        if (lane == 0) {
          if (OUT16) tma_store_wait_read<1>(); else tma_store_wait_read<0>();
        }
        __syncwarp();
        if (OUT16) {
          // half output: a pixel's 32 channels are 64 bytes, stored unswizzled
          store_parity ^= 1;
          uint8_t* dst = stage_buf + store_parity * 2048 + lane * 64;
#pragma unroll
          for (int j = 0; j < 4; j++)
            *reinterpret_cast<uint4*>(dst + (j << 4)) =
                make_uint4(pack_half2(v[j * 8 + 0], v[j * 8 + 1]), pack_half2(v[j * 8 + 2], v[j * 8 + 3]),
                           pack_half2(v[j * 8 + 4], v[j * 8 + 5]), pack_half2(v[j * 8 + 6], v[j * 8 + 7]));
        } else {
          uint8_t* dst = stage_buf + lane * 128;
#pragma unroll
          for (int j = 0; j < 8; j++)
            *reinterpret_cast<float4*>(dst + ((j ^ (lane & 7)) << 4)) =
                make_float4(v[j * 4 + 0], v[j * 4 + 1], v[j * 4 + 2], v[j * 4 + 3]);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          // lanes 0-15 hold patch row 2*quarter, lanes 16-31 the next one: a [2 x 16 x 32] box
          tma_store_4d(&map_y, smem_u32(stage_buf + (OUT16 ? store_parity * 2048 : 0)), c0, tx * PW,
                       ty * PH + quarter * 2, b);
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

template <int BLOCK_N, int S, int MODE, bool HALF = false, bool IN8 = false>
int launch_variant(tfjs_cuda_ctx* ctx, const CUtensorMap& mx, const CUtensorMap& mw, const CUtensorMap& my,
                   const SepParams& p, const CUtensorMap* mw_lo = nullptr) {
  constexpr bool IN16 = HALF && MODE == MODE_DW;
  constexpr int smem_bytes = 1024 + a_slot_bytes(BLOCK_N, S, MODE, IN16) + w_stages(BLOCK_N, S, MODE) * w_stage_bytes(BLOCK_N, MODE) +
                             C_STAGING_BYTES + raw_stages<S, MODE, IN16, IN8>(BLOCK_N) * Raw<S, MODE, IN16, IN8>::STRIDE +
                             DW_TABLE_BYTES + BIAS_STAGING_BYTES + BARRIER_BYTES;
  static_assert(smem_bytes <= SMEM_LIMIT, "shared memory budget exceeded");
  auto kernel = sepconv_tcgen05_kernel<BLOCK_N, S, MODE, HALF, IN8>;
  // per device and per kernel; atomic because contexts of several devices may call from several
  // host threads (setting the attribute twice is harmless)
  static std::atomic<bool> configured[64];
  if (!configured[ctx->device & 63].load(std::memory_order_acquire)) {
    TFJS_CHECK_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    configured[ctx->device & 63].store(true, std::memory_order_release);
  }
  const int grid = p.num_tiles < ctx->sm_count ? p.num_tiles : ctx->sm_count;
  launch_ex(ctx, kernel, dim3(grid), dim3(THREADS), smem_bytes, mx, mw, mw_lo ? *mw_lo : mw, my, p);
  if (MODE == MODE_RGB3) return post_launch(ctx, "conv2d_tcgen05 (3-channel 3x3, window TMA, 3xTF32)");
  if (MODE == MODE_RGB && IN8)
    return post_launch(ctx, HALF ? "conv2d_tcgen05 (3-channel 3x3, window TMA, TF32, uint8 in, float16 out)"
                                 : "conv2d_tcgen05 (3-channel 3x3, window TMA, TF32, uint8 in)");
  if (MODE == MODE_RGB)
    return post_launch(ctx, HALF ? "conv2d_tcgen05 (3-channel 3x3, window TMA, TF32, float16 out)"
                                 : "conv2d_tcgen05 (3-channel 3x3, window TMA, TF32)");
  if (MODE == MODE_CONV3) return post_launch(ctx, "conv2d_tcgen05 (shifted-patch TMA, 3xTF32)");
  if (MODE == MODE_CONV) return post_launch(ctx, "conv2d_tcgen05 (shifted-patch TMA, TF32)");
  if (HALF)
    return post_launch(ctx, S == 1 ? "separableConv2d (fused dw3x3 s1 + pw, TF32, float16)"
                                   : "separableConv2d (fused dw3x3 s2 + pw, TF32, float16)");
  return post_launch(ctx, S == 1 ? "separableConv2d (fused dw3x3 s1 + pw, TF32)"
                                 : "separableConv2d (fused dw3x3 s2 + pw, TF32)");
}

template <int S, int MODE, bool HALF = false, bool IN8 = false>
int launch_stride(tfjs_cuda_ctx* ctx, int block_n, const CUtensorMap& mx, const CUtensorMap& mw,
                  const CUtensorMap& my, const SepParams& p, const CUtensorMap* mw_lo = nullptr) {
  switch (block_n) {
    case 32:
      if (MODE != MODE_DW)
        return launch_variant<32, S, MODE == MODE_DW ? MODE_RGB : MODE, HALF, IN8>(ctx, mx, mw, my, p, mw_lo);
      // depthwise mode has no 32-wide variant: falls through
    case 64: return launch_variant<64, S, MODE, HALF, IN8>(ctx, mx, mw, my, p, mw_lo);
    case 128: return launch_variant<128, S, MODE, HALF, IN8>(ctx, mx, mw, my, p, mw_lo);
    default:
      // (no 256-column 3xTF32 stem: two 64 KB weight stages and the hi / lo A slots leave no room for windows)
      if constexpr (is_split3(MODE)) return set_error(ctx, TFJS_CUDA_ERR_INVALID_ARG, "the 3xTF32 variants take at most 128 output channels");
      else return launch_variant<256, S, MODE, HALF, IN8>(ctx, mx, mw, my, p, mw_lo);
  }
}

}  // namespace

int set_wait_limit_sepconv(long long cycles) { return set_wait_limit_here(cycles); }

// Depthwise 3x3 (stride 1 or 2, dilation 1, channel multiplier 1, C a multiple of 32 up to 256)
// feeding a pointwise convolution with 8..256 output channels, in TF32.
bool sepconv_tcgen05_supported(const tfjs_conv2d_info& dw, int64_t N, int dw_activation, int pw_activation,
                               int math_mode) {
  const int64_t out_px = (int64_t)dw.batchSize * dw.outHeight * dw.outWidth;
  return math_mode == TFJS_MATH_TF32 && dw.filterHeight == 3 && dw.filterWidth == 3 && dw.dilationHeight == 1 &&
         dw.dilationWidth == 1 && dw.strideHeight == dw.strideWidth && (dw.strideHeight == 1 || dw.strideHeight == 2) &&
         dw.outChannels == dw.inChannels && dw.inChannels % 32 == 0 && dw.inChannels >= 32 &&
         dw.inChannels <= MAX_C && N >= 8 && N <= 256 && N % 4 == 0 && out_px >= 1 && dw.batchSize < 65536 &&
         (int64_t)dw.batchSize * dw.inHeight * dw.inWidth * dw.inChannels < (1ll << 40) &&
         dw_activation != TFJS_ACT_PRELU && pw_activation != TFJS_ACT_PRELU &&
         tcgen05_gemm_supported(128, N, dw.inChannels);
}

int launch_sepconv_tcgen05(tfjs_cuda_ctx* ctx, const void* x, const tfjs_conv2d_info& dw, const float* dw_filter,
                           const EpilogueArgs& dw_epi, const float* w_hi, int64_t kp, void* y, int64_t N,
                           const EpilogueArgs& pw_epi, bool half) {
  const int S = dw.strideHeight;
  const int C = dw.inChannels;
  const int block_n = N <= 64 ? 64 : (N <= 128 ? 128 : 256);
  const uint64_t el = half ? 2 : 4;  // bytes per stored activation
  const CUtensorMapDataType act_type = half ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUtensorMap mx, mw, my;
  const uint64_t xd[4] = {(uint64_t)C, (uint64_t)dw.inWidth, (uint64_t)dw.inHeight, (uint64_t)dw.batchSize};
  const uint64_t xs[3] = {(uint64_t)C * el, (uint64_t)dw.inWidth * C * el, (uint64_t)dw.inHeight * dw.inWidth * C * el};
  const uint32_t xb1[4] = {BLOCK_K, (uint32_t)Raw<1, MODE_DW>::COLS, (uint32_t)Raw<1, MODE_DW>::ROWS, 1};
  const uint32_t xb2[4] = {BLOCK_K, (uint32_t)Raw<2, MODE_DW>::COLS, (uint32_t)Raw<2, MODE_DW>::ROWS, 1};
  const uint64_t wd[2] = {(uint64_t)kp, (uint64_t)N};
  const uint64_t ws[1] = {(uint64_t)kp * 4};
  const uint32_t wb[2] = {BLOCK_K, (uint32_t)block_n};
  const uint64_t yd[4] = {(uint64_t)N, (uint64_t)dw.outWidth, (uint64_t)dw.outHeight, (uint64_t)dw.batchSize};
  const uint64_t ys[3] = {(uint64_t)N * el, (uint64_t)dw.outWidth * N * el, (uint64_t)dw.outHeight * dw.outWidth * N * el};
  const uint32_t yb[4] = {32, PW, 2, 1};
  const bool ok =
      tma_encode_tiled(&mx, act_type, 4, x, xd, xs, S == 1 ? xb1 : xb2, CU_TENSOR_MAP_SWIZZLE_NONE) &&
      tma_encode_tiled(&mw, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, w_hi, wd, ws, wb, CU_TENSOR_MAP_SWIZZLE_128B) &&
      tma_encode_tiled(&my, act_type, 4, y, yd, ys, yb, half ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B);
  if (!ok) return set_error(ctx, TFJS_CUDA_ERR_CUDA, "cuTensorMapEncodeTiled failed");
  SepParams p;
  p.B = dw.batchSize;
  p.inH = dw.inHeight;
  p.inW = dw.inWidth;
  p.C = C;
  p.outH = dw.outHeight;
  p.outW = dw.outWidth;
  p.N = (int)N;
  p.pad_r = dw.padLeft;  // (sic) the reference's depthwise uses padLeft for rows and padTop for
  p.pad_c = dw.padTop;   // columns (backend_cpu.ts:2000, 2010)
  p.tiles_y = (dw.outHeight + PH - 1) / PH;
  p.tiles_x = (dw.outWidth + PW - 1) / PW;
  p.num_tiles = dw.batchSize * p.tiles_y * p.tiles_x;
  p.num_k_blocks = C / BLOCK_K;
  p.dw_filter = dw_filter;
  p.dw_bias = dw_epi.bias;
  p.dw_bias_scalar = dw_epi.bias_scalar;
  p.dw_act = dw_epi.activation;
  p.dw_lo = dw_epi.clip_lo;
  p.dw_hi = dw_epi.clip_hi;
  p.epi = pw_epi;
  p.status = ctx->d_status;
  p.rgb_off = 0;
  p.q_scale = p.q_min = 0.0;
  if (half)
    return S == 1 ? launch_stride<1, MODE_DW, true>(ctx, block_n, mx, mw, my, p)
                  : launch_stride<2, MODE_DW, true>(ctx, block_n, mx, mw, my, p);
  return S == 1 ? launch_stride<1, MODE_DW>(ctx, block_n, mx, mw, my, p)
                : launch_stride<2, MODE_DW>(ctx, block_n, mx, mw, my, p);
}

// Dense 3x3 convolution of a 3-channel NHWC image (the network's stem), stride 1 or 2, in TF32:
// same kernel skeleton, the window arrives by TMA and is rearranged into im2col rows on chip.
// `w_hi` is the filter repacked with each filter row padded to 10 floats ([N, 32]).
bool conv_rgb_tcgen05_supported(const tfjs_conv2d_info& ci, int activation, int math_mode) {
  return (math_mode == TFJS_MATH_TF32 || (math_mode == TFJS_MATH_TF32X3 && ci.outChannels <= 128)) && ci.inChannels == 3 && ci.filterHeight == 3 && ci.filterWidth == 3 &&
         ci.dilationHeight == 1 && ci.dilationWidth == 1 && ci.strideHeight == ci.strideWidth &&
         (ci.strideHeight == 1 || ci.strideHeight == 2) && ci.inWidth % 4 == 0 && ci.outChannels >= 8 &&
         ci.outChannels <= 256 && ci.outChannels % 4 == 0 && ci.batchSize >= 1 && ci.batchSize < 65536 &&
         ci.outHeight >= 1 && ci.outWidth >= 1 && activation != TFJS_ACT_PRELU &&
         tcgen05_gemm_supported(128, ci.outChannels, 32);
}

// Byte input also needs image rows of a multiple of 16 bytes (the row stride of the tensor map).
bool conv_rgb_u8_tcgen05_supported(const tfjs_conv2d_info& ci, int activation, int math_mode) {
  return math_mode == TFJS_MATH_TF32 && conv_rgb_tcgen05_supported(ci, activation, math_mode) && (ci.inWidth * 3) % 16 == 0;
}

int launch_conv_rgb_tcgen05(tfjs_cuda_ctx* ctx, const void* x, const tfjs_conv2d_info& ci, const float* w_hi,
                            int64_t kp, void* y, const EpilogueArgs& epi, bool out_half, bool in_u8, double q_scale,
                            double q_min, const float* w_lo) {  // w_lo: 3xTF32 (float32 in and out only)
  const int S = ci.strideHeight;
  const int64_t N = ci.outChannels;
  const uint64_t el = out_half ? 2 : 4;
  const int block_n = N <= 32 ? 32 : (N <= 64 ? 64 : (N <= 128 ? 128 : 256));
  CUtensorMap mx, mw, my;
  const uint64_t xel = in_u8 ? 1 : 4;
  const uint64_t xd[3] = {(uint64_t)ci.inWidth * 3, (uint64_t)ci.inHeight, (uint64_t)ci.batchSize};
  const uint64_t xs[2] = {(uint64_t)ci.inWidth * 3 * xel, (uint64_t)ci.inHeight * ci.inWidth * 3 * xel};
  const uint32_t xb1[3] = {(uint32_t)(in_u8 ? Raw<1, MODE_RGB, false, true>::ROW_FLOATS : Raw<1, MODE_RGB>::ROW_FLOATS),
                           (uint32_t)Raw<1, MODE_RGB>::ROWS, 1};
  const uint32_t xb2[3] = {(uint32_t)(in_u8 ? Raw<2, MODE_RGB, false, true>::ROW_FLOATS : Raw<2, MODE_RGB>::ROW_FLOATS),
                           (uint32_t)Raw<2, MODE_RGB>::ROWS, 1};
  const uint64_t wd[2] = {(uint64_t)kp, (uint64_t)N};
  const uint64_t ws[1] = {(uint64_t)kp * 4};
  const uint32_t wb[2] = {BLOCK_K, (uint32_t)block_n};
  const uint64_t yd[4] = {(uint64_t)N, (uint64_t)ci.outWidth, (uint64_t)ci.outHeight, (uint64_t)ci.batchSize};
  const uint64_t ys[3] = {(uint64_t)N * el, (uint64_t)ci.outWidth * N * el, (uint64_t)ci.outHeight * ci.outWidth * N * el};
  const uint32_t yb[4] = {32, PW, 2, 1};
  const bool ok =
      tma_encode_tiled(&mx, in_u8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, x, xd, xs,
                       S == 1 ? xb1 : xb2, CU_TENSOR_MAP_SWIZZLE_NONE) &&
      tma_encode_tiled(&mw, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, w_hi, wd, ws, wb, CU_TENSOR_MAP_SWIZZLE_128B) &&
      tma_encode_tiled(&my, out_half ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, y, yd, ys, yb,
                       out_half ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B);
  if (!ok) return set_error(ctx, TFJS_CUDA_ERR_CUDA, "cuTensorMapEncodeTiled failed");
  CUtensorMap mwl;
  if (w_lo) {
    TFJS_REQUIRE(ctx, !out_half && !in_u8, "the 3xTF32 stem computes on float32 storage");
    if (!tma_encode_tiled(&mwl, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, w_lo, wd, ws, wb, CU_TENSOR_MAP_SWIZZLE_128B))
      return set_error(ctx, TFJS_CUDA_ERR_CUDA, "cuTensorMapEncodeTiled failed");
  }
  SepParams p;
  memset(&p, 0, sizeof(p));
  p.B = ci.batchSize;
  p.inH = ci.inHeight;
  p.inW = ci.inWidth;
  p.C = 3;
  p.outH = ci.outHeight;
  p.outW = ci.outWidth;
  p.N = (int)N;
  p.pad_r = ci.padTop;
  p.pad_c = ci.padLeft;
  p.tiles_y = (ci.outHeight + PH - 1) / PH;
  p.tiles_x = (ci.outWidth + PW - 1) / PW;
  p.num_tiles = ci.batchSize * p.tiles_y * p.tiles_x;
  p.num_k_blocks = 1;
  p.epi = epi;
  // the window of a patch starts at float (tx*16*S - padLeft)*3 of its image row; 16*S*3 is a
  // multiple of 4, so the distance to the 16-byte boundary below it is the same for every patch
  // (bytes: the distance to the 16-byte boundary counts bytes, and 16*S*3 bytes is a multiple of 16 too)
  p.rgb_off = in_u8 ? ((-3 * ci.padLeft) % 16 + 16) % 16 : ((-3 * ci.padLeft) % 4 + 4) % 4;
  p.q_scale = q_scale;
  p.q_min = q_min;
  p.status = ctx->d_status;
  if (in_u8) {
    if (out_half)
      return S == 1 ? launch_stride<1, MODE_RGB, true, true>(ctx, block_n, mx, mw, my, p)
                    : launch_stride<2, MODE_RGB, true, true>(ctx, block_n, mx, mw, my, p);
    return S == 1 ? launch_stride<1, MODE_RGB, false, true>(ctx, block_n, mx, mw, my, p)
                  : launch_stride<2, MODE_RGB, false, true>(ctx, block_n, mx, mw, my, p);
  }
  if (w_lo)
    return S == 1 ? launch_stride<1, MODE_RGB3>(ctx, block_n, mx, mw, my, p, &mwl)
                  : launch_stride<2, MODE_RGB3>(ctx, block_n, mx, mw, my, p, &mwl);
  if (out_half)
    return S == 1 ? launch_stride<1, MODE_RGB, true>(ctx, block_n, mx, mw, my, p)
                  : launch_stride<2, MODE_RGB, true>(ctx, block_n, mx, mw, my, p);
  return S == 1 ? launch_stride<1, MODE_RGB>(ctx, block_n, mx, mw, my, p)
                : launch_stride<2, MODE_RGB>(ctx, block_n, mx, mw, my, p);
}

// Dense convolution with Cin a multiple of 32 and stride 1 (any filter size and dilation), TF32:
// every k-block's A tile is the output patch shifted by one filter tap, fetched by one TMA load.
bool conv_tma_tcgen05_supported(const tfjs_conv2d_info& ci, int activation, int math_mode) {
  return (math_mode == TFJS_MATH_TF32 || (math_mode == TFJS_MATH_TF32X3 && ci.outChannels <= 128)) && ci.inChannels >= 32 && ci.inChannels % 32 == 0 && ci.strideHeight == 1 &&
         ci.strideWidth == 1 && ci.outChannels >= 8 && ci.outChannels <= 256 && ci.outChannels % 4 == 0 &&
         ci.batchSize >= 1 && ci.batchSize < 65536 && ci.outHeight >= 1 && ci.outWidth >= 1 &&
         (int64_t)ci.filterHeight * ci.filterWidth * ci.inChannels < (1ll << 24) && activation != TFJS_ACT_PRELU &&
         tcgen05_gemm_supported(128, ci.outChannels, ci.inChannels);
}

int launch_conv_tma_tcgen05(tfjs_cuda_ctx* ctx, const float* x, const tfjs_conv2d_info& ci, const float* w_hi,
                            int64_t kp, float* y, const EpilogueArgs& epi, const float* w_lo) {  // w_lo: 3xTF32
  const int64_t N = ci.outChannels;
  const int C = ci.inChannels;
  const int block_n = N <= 32 ? 32 : (N <= 64 ? 64 : (N <= 128 ? 128 : 256));
  CUtensorMap mx, mw, my;
  const uint64_t xd[4] = {(uint64_t)C, (uint64_t)ci.inWidth, (uint64_t)ci.inHeight, (uint64_t)ci.batchSize};
  const uint64_t xs[3] = {(uint64_t)C * 4, (uint64_t)ci.inWidth * C * 4, (uint64_t)ci.inHeight * ci.inWidth * C * 4};
  const uint32_t xb[4] = {BLOCK_K, PW, PH, 1};
  const uint64_t wd[2] = {(uint64_t)kp, (uint64_t)N};
  const uint64_t ws[1] = {(uint64_t)kp * 4};
  const uint32_t wb[2] = {BLOCK_K, (uint32_t)block_n};
  const uint64_t yd[4] = {(uint64_t)N, (uint64_t)ci.outWidth, (uint64_t)ci.outHeight, (uint64_t)ci.batchSize};
  const uint64_t ys[3] = {(uint64_t)N * 4, (uint64_t)ci.outWidth * N * 4, (uint64_t)ci.outHeight * ci.outWidth * N * 4};
  const uint32_t yb[4] = {32, PW, 2, 1};
  const bool ok =
      tma_encode_tiled(&mx, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, x, xd, xs, xb, CU_TENSOR_MAP_SWIZZLE_128B) &&
      tma_encode_tiled(&mw, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, w_hi, wd, ws, wb, CU_TENSOR_MAP_SWIZZLE_128B) &&
      tma_encode_tiled(&my, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, y, yd, ys, yb, CU_TENSOR_MAP_SWIZZLE_128B);
  if (!ok) return set_error(ctx, TFJS_CUDA_ERR_CUDA, "cuTensorMapEncodeTiled failed");
  SepParams p;
  memset(&p, 0, sizeof(p));
  p.B = ci.batchSize;
  p.inH = ci.inHeight;
  p.inW = ci.inWidth;
  p.C = C;
  p.outH = ci.outHeight;
  p.outW = ci.outWidth;
  p.N = (int)N;
  p.pad_r = ci.padTop;
  p.pad_c = ci.padLeft;
  p.tiles_y = (ci.outHeight + PH - 1) / PH;
  p.tiles_x = (ci.outWidth + PW - 1) / PW;
  p.num_tiles = ci.batchSize * p.tiles_y * p.tiles_x;
  p.fh = ci.filterHeight;
  p.fw = ci.filterWidth;
  p.dil_h = ci.dilationHeight;
  p.dil_w = ci.dilationWidth;
  p.cin_groups = C / BLOCK_K;
  p.num_k_blocks = ci.filterHeight * ci.filterWidth * p.cin_groups;
  p.epi = epi;
  p.status = ctx->d_status;
  if (w_lo) {
    CUtensorMap mwl;
    if (!tma_encode_tiled(&mwl, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, w_lo, wd, ws, wb, CU_TENSOR_MAP_SWIZZLE_128B))
      return set_error(ctx, TFJS_CUDA_ERR_CUDA, "cuTensorMapEncodeTiled failed");
    return launch_stride<1, MODE_CONV3>(ctx, block_n, mx, mw, my, p, &mwl);
  }
  return launch_stride<1, MODE_CONV>(ctx, block_n, mx, mw, my, p);
}
