// Definitions shared by the 1-CTA and 2-CTA rowwise FP8 GEMM kernels: launch
// parameters, the device-side tile scheduler over per-group row counts, and the
// scale/bias/convert/store step of the epilogue.
#pragma once

#include "../../include/mslk_b200.h"
#include "common.cuh"
#include "host.h"

namespace mslk_b200 {
namespace gemm_f8 {

constexpr int kBM = 128;          // rows of the output tile (UMMA M)
constexpr int kBK = 128;          // bytes (= fp8 elements) of K per pipeline stage
constexpr int kUmmaK = 32;        // K per tcgen05.mma for 8-bit operands
constexpr int kMaxGroups = 1024;
constexpr int kNumThreads = 192;
constexpr int kNumEpilogueThreads = 128;
constexpr int kBandM = 16;        // row blocks per scheduling band

struct GemmParams {
  const float *x_scale;
  const float *w_scale;
  const void *bias;
  __nv_bfloat16 *y;
  const int64_t *m_sizes;  // device, [G]; nullptr = G groups of group_m rows each (dense: G = 1)
  int *status;
  int bias_kind;
  int G;
  int total_m;
  int group_m;  // rows of every group when m_sizes is null (batched GEMM); total_m for the dense case
  // Alternative to m_sizes: int32 END offsets of the groups in the stacked rows (device, [G]);
  // group g owns rows [end_offsets[g-1], end_offsets[g]).  Takes precedence when set.
  const int32_t *end_offsets = nullptr;
  // Rows of the A (token) box of the one-CTA kernel's tensor map: 128, or fewer for a dense problem with
  // fewer rows, so that TMA neither fetches nor zero-fills rows that do not exist (the instruction still
  // reads 128 rows of shared memory; what the extra rows hold only reaches masked output rows).
  int a_box_rows = 128;
  // Scatter-add epilogue (MoE combine fused into the grouped GEMM): when set, stacked row r of the
  // product is ADDED atomically (bf16 vector reductions) to row scatter_idx[r] of y, which then has
  // scatter_rows rows; indices are 32- or 64-bit integers on the device.
  const void *scatter_idx = nullptr;
  int scatter_bits = 32;
  int scatter_rows = 0;
  int N;
  int K;
  // Output placement: y (and y_extra[0..n_extra)) are row-major with a pitch of ldy elements; the
  // N columns of this problem start at column col0.  Defaults: ldy = N, col0 = 0, n_extra = 0.
  // The extra destinations may be buffers of peer GPUs (plain stores over NVLink): that is how the
  // N-sharded GEMM delivers its column block to every rank without a separate all-gather.
  __nv_bfloat16 *y_extra[7];
  int n_extra;
  int ldy;
  int col0;
  int tma_store;  // pair kernel: full 32-row slabs leave through shared memory and TMA stores
  // Row-scatter mode (K-sharded GEMM feeding a reduce-scatter): rs_rows > 0 sends every 32-row slab
  // to ONE destination, the owner of its rows (owner = row / rs_rows; destinations are y, y_extra[0..]
  // in rank order), at row rs_slot * rs_rows + row % rs_rows of that destination's
  // [world * rs_rows, N] staging buffer; the owner sums the slots afterwards.
  int rs_rows;
  int rs_slot;
  // Tile order of the CTA-pair kernel (set by its launcher).  band_m > 0: bands of band_m row blocks, inside a
  // band the tiles run column by column, so the band's rows of X stay in L2 while W streams through once per
  // band.  band_n > 0 (dense problems only, takes precedence): bands of band_n column blocks, inside a band row
  // by row, so the band's rows of W stay and X streams.
  int band_m = 0;
  int band_n = 0;
};

inline void default_placement(GemmParams &p) {
  p.n_extra = 0;
  p.ldy = p.N;
  p.col0 = 0;
  p.tma_store = 0;
  p.rs_rows = 0;
  p.rs_slot = 0;
  for (auto &e : p.y_extra) e = nullptr;
}

// Builds the per-group prefix tables (first stacked row and first linear tile of every
// group) in shared memory; executed by one full warp.  Row counts come from device memory
// (m_sizes) and are clamped so that the stacked rows never run past total_m.  `tile_rows`
// is the row extent of one scheduled tile (128 for the 1-CTA kernel, 256 for a CTA pair).
__device__ __forceinline__ void build_group_tables(const GemmParams &p, int n_tiles, int tile_rows, int lane,
                                                   int *row_start, int *tile_start) {
  int row_carry = 0, tile_carry = 0;
  for (int base = 0; base < p.G; base += 32) {
    const int g = base + lane;
    long long mg = 0;
    if (g < p.G) {
      if (p.end_offsets) mg = static_cast<long long>(p.end_offsets[g]) - (g > 0 ? p.end_offsets[g - 1] : 0);
      else mg = p.m_sizes ? p.m_sizes[g] : p.group_m;
    }
    if (mg < 0) mg = 0;
    if (mg > p.total_m) mg = p.total_m;
    int rows = static_cast<int>(mg);
    int rsum = rows;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, rsum, o);
      if (lane >= o) rsum += v;
    }
    int start = row_carry + rsum - rows;
    if (start > p.total_m) start = p.total_m;
    if (start + rows > p.total_m) rows = p.total_m - start;
    int tiles = ((rows + tile_rows - 1) / tile_rows) * n_tiles;
    int tsum = tiles;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, tsum, o);
      if (lane >= o) tsum += v;
    }
    if (g < p.G) {
      row_start[g] = start;
      tile_start[g] = tile_carry + tsum - tiles;
    }
    row_carry = min(p.total_m, row_carry + __shfl_sync(0xffffffffu, rsum, 31));
    tile_carry += __shfl_sync(0xffffffffu, tsum, 31);
  }
  if (lane == 0) {
    row_start[p.G] = row_carry;
    tile_start[p.G] = tile_carry;
  }
}

struct Tile {
  int row0;   // first row of the tile in the stacked X / Y
  int rows;   // valid rows of the scheduled tile (1..tile_rows)
  int n0;     // first output column
  int wrow0;  // first row in WQ viewed as [G*N, K]
  int ws0;    // first index into w_scale
};

struct Scheduler {
  const int *tile_start;
  const int *row_start;
  int G, N, n_tiles, bn;
  int tile_rows;  // rows of one scheduled tile: 128 (single CTA) or 256 (CTA pair)
  int band_m;     // row blocks per band
  int g;
  int band_n = 0; // > 0 (one group only): bands of band_n column blocks, rows fastest-varying outside

  __device__ __forceinline__ bool get(int tile, Tile &t) {
    if (tile >= tile_start[G]) return false;
    while (tile >= tile_start[g + 1]) ++g;
    const int local = tile - tile_start[g];
    const int mg = row_start[g + 1] - row_start[g];
    const int m_tiles = (mg + tile_rows - 1) / tile_rows;
    int n_tile, m_tile;
    if (band_n > 0) {
      const int per_band = band_n * m_tiles;
      const int band = local / per_band;
      const int in_band = local - band * per_band;
      const int first_n = band * band_n;
      const int this_band_n = min(n_tiles - first_n, band_n);
      m_tile = in_band / this_band_n;
      n_tile = first_n + (in_band - m_tile * this_band_n);
    } else {
      const int per_band = band_m * n_tiles;
      const int band = local / per_band;
      const int in_band = local - band * per_band;
      const int first_m = band * band_m;
      const int this_band_m = min(m_tiles - first_m, band_m);
      n_tile = in_band / this_band_m;
      m_tile = first_m + (in_band - n_tile * this_band_m);
    }
    t.row0 = row_start[g] + m_tile * tile_rows;
    t.rows = min(tile_rows, mg - m_tile * tile_rows);
    t.n0 = n_tile * bn;
    t.wrow0 = g * N + t.n0;
    t.ws0 = g * N + t.n0;
    return true;
  }
};

// 32 accumulator columns of one row -> 16 packed bf16 pairs: (acc * xs) * ws (+ bias)
template <int BIAS>
__device__ __forceinline__ void epilogue_pack(const uint32_t (&acc)[32], float xs, const float *ws, const float *bs,
                                              uint32_t (&packed)[16]) {
#pragma unroll
  for (int j = 0; j < 32; j += 2) {
    float v0 = (__uint_as_float(acc[j]) * xs) * ws[j];
    float v1 = (__uint_as_float(acc[j + 1]) * xs) * ws[j + 1];
    if constexpr (BIAS == MSLK_B200_BIAS_F32) {
      v0 += bs[j];
      v1 += bs[j + 1];
    } else if constexpr (BIAS == MSLK_B200_BIAS_BF16) {
      // the scaled product is rounded to bf16 first and the add is done in bf16
      v0 = __bfloat162float(__float2bfloat16_rn(v0)) + bs[j];
      v1 = __bfloat162float(__float2bfloat16_rn(v1)) + bs[j + 1];
    }
    packed[j / 2] = pack_bf16x2(v0, v1);
  }
}

__device__ __forceinline__ void epilogue_pack_any(int bias_kind, const uint32_t (&acc)[32], float xs, const float *ws,
                                                  const float *bs, uint32_t (&packed)[16]) {
  if (bias_kind == MSLK_B200_BIAS_NONE) epilogue_pack<MSLK_B200_BIAS_NONE>(acc, xs, ws, bs, packed);
  else if (bias_kind == MSLK_B200_BIAS_F32) epilogue_pack<MSLK_B200_BIAS_F32>(acc, xs, ws, bs, packed);
  else epilogue_pack<MSLK_B200_BIAS_BF16>(acc, xs, ws, bs, packed);
}

template <int BN, int BIAS>
__device__ __forceinline__ void epilogue_chunk(const uint32_t (&acc)[32], float xs, const float *ws, const float *bs,
                                               const GemmParams &p, size_t elem_off, bool row_ok, int cols_left,
                                               bool vec_ok) {
  uint32_t packed[16];
  epilogue_pack<BIAS>(acc, xs, ws, bs, packed);
  if (!row_ok) return;
  if (p.scatter_idx) {   // elem_off already addresses the destination row
    __nv_bfloat16 *dst = p.y + elem_off;
    if (vec_ok && cols_left >= 32) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        asm volatile("red.relaxed.gpu.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(dst + 8 * j),
                     "r"(packed[4 * j]), "r"(packed[4 * j + 1]), "r"(packed[4 * j + 2]), "r"(packed[4 * j + 3])
                     : "memory");
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < cols_left)
          atomicAdd(dst + j, __ushort_as_bfloat16(static_cast<unsigned short>(packed[j / 2] >> ((j & 1) * 16))));
    }
    return;
  }
  for (int dsti = -1; dsti < p.n_extra; ++dsti) {
    __nv_bfloat16 *dst = (dsti < 0 ? p.y : p.y_extra[dsti]) + elem_off;
    if (vec_ok && cols_left >= 32) {
      uint4 *d4 = reinterpret_cast<uint4 *>(dst);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        d4[j] = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
    } else {
      uint16_t *d = reinterpret_cast<uint16_t *>(dst);
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < cols_left) d[j] = static_cast<uint16_t>(packed[j / 2] >> ((j & 1) * 16));
    }
  }
}

// Host side: the 2-CTA (cta_group::2) launcher lives in gemm_f8_rowwise_2cta.cu.
// Returns 0 on success, a non-zero code after recording an error, or -1 when the shape or
// the device cannot use CTA pairs (the caller then takes the 1-CTA kernel).
int launch_pair_kernel(const void *xq, const void *wq, const GemmParams &p, cudaStream_t st);

// Host side: the few-token (M <= 32) weight-streaming kernel lives in gemm_f8_rowwise_decode.cu.
// (The kernel itself handles up to 128 tokens, but beyond 32 the split-K traffic and its serial
// tail cost more than the small-BN tiles of the general kernel; measured on the Llama-3-8B shapes.)
// `scratch` (may be null) enables K splitting; its required size comes from decode_scratch_bytes().
// `scratch_is_clean`: the ticket words are known to be zero (skips the memset).
constexpr int kDecodeMaxTokens = 32;
size_t decode_scratch_bytes(int64_t M, int64_t N, int64_t K, int sms);
int launch_decode_kernel(const void *xq, const void *wq, const GemmParams &p, void *scratch, size_t scratch_bytes,
                         bool scratch_is_clean, cudaStream_t st);

}  // namespace gemm_f8
}  // namespace mslk_b200
