// NVFP4 quantization for sm_100a: bf16 -> packed e2m1 with one e4m3 scale per 16
// elements (stored in the 128x4-tile swizzled layout the block-scaled MMA reads)
// and an optional fp32 per-tensor global scale.
//
// Arithmetic (bit-exact with the reference's kernel,
// mslk/quantize/triton/quantize_kernels/nvfp4.py:213-296, precise-math branch):
//     s    = e4m3_rn(clamp((bamax / 6) * gs, 2^-9, 448))     per 16-element block
//     x^   = e2m1_rn_satfinite(x * (gs / float(s)))
// with IEEE fp32 divisions.  One thread owns one 16-element block: two 16-byte
// loads and one 8-byte store of packed nibbles; lanes are assigned so that a warp's
// 32 scale bytes are contiguous in the atom (one 32-byte store per warp).
// The tiles span the padded scale matrix, so padding rows / columns are written as zero.
#include "../../include/mslk_b200.h"
#include "common.cuh"
#include "host.h"

namespace mslk_b200 {
namespace {

__device__ __forceinline__ uint32_t cvt_e2m1x8(const float (&v)[8]) {
  uint32_t r;
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
      : "=r"(r)
      : "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]));
  return r;
}

__device__ __forceinline__ uint8_t f32_to_e4m3(float v) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.f), "f"(v));
  return static_cast<uint8_t>(r & 0xffu);
}

__device__ __forceinline__ float e4m3_to_f32(uint8_t c) {
  uint32_t h2;
  const uint16_t in = c;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(in));
  return __half2float(__ushort_as_half(static_cast<unsigned short>(h2 & 0xffffu)));
}

constexpr int kTileRows = 128;     // rows of one scale atom
constexpr int kTileBlocks = 4;     // 16-element blocks (scale columns) of one scale atom
constexpr int kWarpsPerTile = 16;  // one warp quantizes 8 rows x 4 blocks of a tile
constexpr int kThreads = 256;

struct BlockIn {
  uint4 a, b;   // 16 bf16 = one scale block
};

// a / b rounded to nearest, from b and its correctly rounded reciprocal rb: q0 = a * rb is within one
// unit of the quotient, the remainder a - b * q0 is exact in an fma, and one more fma lands on the
// correctly rounded quotient (Markstein) -- as long as nothing is subnormal on the way, which the
// magnitude guard ensures; outside it, and for a zero numerator, the IEEE division itself runs.
__device__ __forceinline__ float div_rn_via_rcp(float a, float b, float rb) {
  const float aa = fabsf(a);
  if (aa > 0x1p-80f && aa < 0x1p80f) {   // b in [2^-9, 448] or 6: quotient and remainder stay normal
    const float q0 = __fmul_rn(a, rb);
    const float rem = __fmaf_rn(-b, q0, a);
    return __fmaf_rn(rem, rb, q0);
  }
  return __fdiv_rn(a, b);
}

// The two 16-bit input types differ only in how a 32-bit word of two elements yields its maximum magnitude and its
// two fp32 values; everything after that is fp32 arithmetic.
template <bool kHalf>
__device__ __forceinline__ float pair_amax8(const uint32_t (&w)[8]) {
  if constexpr (kHalf) {
    __half2 mx = __habs2(*reinterpret_cast<const __half2 *>(&w[0]));
#pragma unroll
    for (int i = 1; i < 8; ++i) mx = __hmax2(mx, __habs2(*reinterpret_cast<const __half2 *>(&w[i])));
    return fmaxf(__low2float(mx), __high2float(mx));
  } else {
    __nv_bfloat162 mx = __habs2(*reinterpret_cast<const __nv_bfloat162 *>(&w[0]));
#pragma unroll
    for (int i = 1; i < 8; ++i) mx = __hmax2(mx, __habs2(*reinterpret_cast<const __nv_bfloat162 *>(&w[i])));
    return fmaxf(__bfloat162float(mx.x), __bfloat162float(mx.y));
  }
}

template <bool kHalf>
__device__ __forceinline__ float word_lo(uint32_t w) {
  if constexpr (kHalf) return __half2float(__ushort_as_half(static_cast<unsigned short>(w & 0xffffu)));
  else return __uint_as_float(w << 16);
}
template <bool kHalf>
__device__ __forceinline__ float word_hi(uint32_t w) {
  if constexpr (kHalf) return __half2float(__ushort_as_half(static_cast<unsigned short>(w >> 16)));
  else return __uint_as_float(w & 0xffff0000u);
}

template <int kVec>
__device__ __forceinline__ BlockIn load_block(const __nv_bfloat16 *src) {
  BlockIn v;
  if (kVec == 1) {
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.a.x), "=r"(v.a.y), "=r"(v.a.z), "=r"(v.a.w) : "l"(src));
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.b.x), "=r"(v.b.y), "=r"(v.b.z), "=r"(v.b.w) : "l"(src + 8));
  } else {
    const uint16_t *h = reinterpret_cast<const uint16_t *>(src);
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = static_cast<uint32_t>(h[2 * i]) | (static_cast<uint32_t>(h[2 * i + 1]) << 16);
    v.a = make_uint4(w[0], w[1], w[2], w[3]);
    v.b = make_uint4(w[4], w[5], w[6], w[7]);
  }
  return v;
}

// Work unit = one warp's share of a 128-row x 64-column tile (one 512-byte scale atom): warp w of
// the tile takes rows {2w, 2w+1} + {0, 32, 64, 96} and the 4 blocks of each, one 16-element block
// per lane.  With lane = (row & 1) * 16 + (row / 32) * 4 + block, the 32 scale bytes of a unit are
// the contiguous bytes [32w, 32w + 32) of the atom: one sector per warp store, no shared memory
// and no barrier between warps.  Units are walked grid-stride with the next unit's block prefetched
// into registers.  total = gs / float(s) comes from a 127-entry table of IEEE quotients built
// once per CTA.
template <int kVec, bool kHalf>
__global__ void __launch_bounds__(kThreads, 6)
    quant_nvfp4_kernel(const __nv_bfloat16 *__restrict__ x, int M, int nblk, int64_t row_stride,
                       const float *__restrict__ gs_ptr, uint8_t *__restrict__ q, uint8_t *__restrict__ scales,
                       int n_col_tiles, int total_units) {
  __shared__ float s_total[128];
  const int tid = threadIdx.x;
  const float gs = gs_ptr ? *gs_ptr : 1.0f;
  if (tid < 128) s_total[tid] = tid == 127 ? 0.f : __fdiv_rn(gs, e4m3_to_f32(static_cast<uint8_t>(tid)));
  __syncthreads();
  const int lane = tid & 31;
  const int c = lane & 3, row_in_tile = ((lane >> 2) & 3) * 32 + (lane >> 4);
  const int64_t q_pitch = static_cast<int64_t>(nblk) * 8;
  const int stride = gridDim.x * (kThreads / 32);

  int unit = blockIdx.x * (kThreads / 32) + (tid >> 5);
  if (unit >= total_units) return;
  // unit -> (row block tr, column tile tc, warp slot w), carried along digit by digit: the kernel is
  // close to its instruction-issue limit and two divisions per unit were a fifth of its instructions
  int tile = unit / kWarpsPerTile, w = unit - tile * kWarpsPerTile;
  int tr = tile / n_col_tiles, tc = tile - tr * n_col_tiles;
  const int d_tile = stride / kWarpsPerTile, d_w = stride - d_tile * kWarpsPerTile;
  const int d_tr = d_tile / n_col_tiles, d_tc = d_tile - d_tr * n_col_tiles;
  int m, j;
  auto locate_here = [&](int &mm, int &jj) {
    mm = tr * kTileRows + row_in_tile + 2 * w;
    jj = tc * kTileBlocks + c;
    return mm < M && jj < nblk;
  };
  auto advance = [&]() {
    w += d_w;
    const int carry = w >= kWarpsPerTile ? 1 : 0;
    w -= carry * kWarpsPerTile;
    tc += d_tc + carry;
    tr += d_tr;
    if (tc >= n_col_tiles) {
      tc -= n_col_tiles;
      ++tr;
    }
  };
  bool live = locate_here(m, j);
  BlockIn cur{};
  if (live) cur = load_block<kVec>(x + m * row_stride + j * 16);
  while (unit < total_units) {
    // prefetch the next unit's block
    const int nunit = unit + stride;
    int nm = 0, nj = 0;
    bool nlive = false;
    BlockIn nxt{};
    if (nunit < total_units) {
      advance();
      nlive = locate_here(nm, nj);
      if (nlive) nxt = load_block<kVec>(x + nm * row_stride + nj * 16);
    }
    uint8_t s8 = 0;
    if (live) {
      const uint32_t w[8] = {cur.a.x, cur.a.y, cur.a.z, cur.a.w, cur.b.x, cur.b.y, cur.b.z, cur.b.w};
      // block amax on the packed pairs (exact: max and abs do not round)
      const float bamax = pair_amax8<kHalf>(w);
      float s = __fmul_rn(div_rn_via_rcp(bamax, 6.0f, 0x1.555556p-3f), gs);
      s = fminf(fmaxf(s, 0.001953125f), 448.0f);
      s8 = f32_to_e4m3(s);
      const float total = s_total[s8 & 127];
      float lo[8], hi[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        lo[2 * i] = __fmul_rn(word_lo<kHalf>(w[i]), total);
        lo[2 * i + 1] = __fmul_rn(word_hi<kHalf>(w[i]), total);
        hi[2 * i] = __fmul_rn(word_lo<kHalf>(w[4 + i]), total);
        hi[2 * i + 1] = __fmul_rn(word_hi<kHalf>(w[4 + i]), total);
      }
      *reinterpret_cast<uint2 *>(q + m * q_pitch + j * 8) = make_uint2(cvt_e2m1x8(lo), cvt_e2m1x8(hi));
    }
    scales[static_cast<int64_t>(unit) * 32 + lane] = s8;   // zero for padding rows / columns
    unit = nunit;
    m = nm;
    j = nj;
    live = nlive;
    cur = nxt;
  }
}


// ---------------------------------------------------------------- stacked (grouped) variant
// Rows of several groups stacked in one [M, K] tensor, group g owning m_sizes[g] consecutive rows and
// its own global scale gs[g].  The scale rows of every group start on a 128-row boundary of the
// padded scale matrix (group g at sum_{i<g} roundup(m_i, 128)), which is the layout the grouped
// GEMM reads (mslk/quantize/triton/legacy/quantize_stacked.py:22-178,315-400).  A 128-row padded
// tile therefore belongs to one group: the unit's group, source rows and scale are uniform per warp.
constexpr int kMaxStackedGroups = 1024;

// Inclusive prefix sums of the group sizes (rows) and of their 128-row blocks; one warp.
__device__ __forceinline__ void build_stacked_tables(const int64_t *m_sizes, int G, int M, int lane, int *row_end,
                                                     int *blk_end) {
  int row_carry = 0, blk_carry = 0;
  for (int base = 0; base < G; base += 32) {
    const int g = base + lane;
    long long mg = g < G ? m_sizes[g] : 0;
    mg = mg < 0 ? 0 : (mg > M ? M : mg);
    int rows = static_cast<int>(mg), blks = (rows + kTileRows - 1) / kTileRows;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int r = __shfl_up_sync(0xffffffffu, rows, o), b = __shfl_up_sync(0xffffffffu, blks, o);
      if (lane >= o) {
        rows += r;
        blks += b;
      }
    }
    if (g < G) {
      row_end[g] = min(M, row_carry + rows);
      blk_end[g] = blk_carry + blks;
    }
    row_carry = min(M, row_carry + __shfl_sync(0xffffffffu, rows, 31));
    blk_carry += __shfl_sync(0xffffffffu, blks, 31);
  }
}

template <int kVec, bool kHalf>
__global__ void __launch_bounds__(kThreads, 6)
    quant_nvfp4_stacked_kernel(const __nv_bfloat16 *__restrict__ x, int M, int nblk, int64_t row_stride,
                               const float *__restrict__ gs_ptr, const int64_t *__restrict__ m_sizes, int G,
                               uint8_t *__restrict__ q, uint8_t *__restrict__ scales, int n_col_tiles) {
  __shared__ int s_row_end[kMaxStackedGroups];
  __shared__ int s_blk_end[kMaxStackedGroups];
  __shared__ float2 s_e4m3[128];   // value of every positive e4m3 code and its correctly rounded reciprocal
  const int tid = threadIdx.x, lane = tid & 31;
  if (tid < 32) build_stacked_tables(m_sizes, G, M, lane, s_row_end, s_blk_end);
  if (tid >= 128) {
    const float v = e4m3_to_f32(static_cast<uint8_t>(tid - 128));
    s_e4m3[tid - 128] = make_float2(v, __frcp_rn(v));
  }
  __syncthreads();
  const int c = lane & 3, row_in_tile = ((lane >> 2) & 3) * 32 + (lane >> 4);
  const int64_t q_pitch = static_cast<int64_t>(nblk) * 8;
  const int stride = gridDim.x * (kThreads / 32);
  const int total_units = s_blk_end[G - 1] * n_col_tiles * kWarpsPerTile;

  // The kernel is bound by instruction issue (ncu: issue slots 71 % busy, ~240 warp instructions per
  // unit), so the unit -> (row block, column tile, warp slot) split is carried along incrementally
  // instead of by two divisions per unit, and the group is a running index (row blocks only grow).
  struct Loc {
    int m, j, g;
    bool live;
  };
  auto emit = [&](int unit, const Loc &l, const BlockIn &cur, float gs) {
    uint8_t s8 = 0;
    if (l.live) {
      const uint32_t wd[8] = {cur.a.x, cur.a.y, cur.a.z, cur.a.w, cur.b.x, cur.b.y, cur.b.z, cur.b.w};
      const float bamax = pair_amax8<kHalf>(wd);
      float sc = __fmul_rn(div_rn_via_rcp(bamax, 6.0f, 0x1.555556p-3f), gs);
      sc = fminf(fmaxf(sc, 0.001953125f), 448.0f);
      s8 = f32_to_e4m3(sc);
      const float2 vr = s_e4m3[s8 & 127];   // s8 is a code in [2^-9, 448]: never zero, never NaN
      const float total = div_rn_via_rcp(gs, vr.x, vr.y);
      float lo8[8], hi8[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        lo8[2 * i] = __fmul_rn(word_lo<kHalf>(wd[i]), total);
        lo8[2 * i + 1] = __fmul_rn(word_hi<kHalf>(wd[i]), total);
        hi8[2 * i] = __fmul_rn(word_lo<kHalf>(wd[4 + i]), total);
        hi8[2 * i + 1] = __fmul_rn(word_hi<kHalf>(wd[4 + i]), total);
      }
      *reinterpret_cast<uint2 *>(q + l.m * q_pitch + l.j * 8) = make_uint2(cvt_e2m1x8(lo8), cvt_e2m1x8(hi8));
    }
    scales[static_cast<int64_t>(unit) * 32 + lane] = s8;   // zero for the padding rows / columns of the group
  };
  int unit = blockIdx.x * (kThreads / 32) + (tid >> 5);
  int tile = unit / kWarpsPerTile, w = unit - tile * kWarpsPerTile;
  int tr = tile / n_col_tiles, tc = tile - tr * n_col_tiles;
  const int d_tile = stride / kWarpsPerTile, d_w = stride - d_tile * kWarpsPerTile;
  const int d_tr = d_tile / n_col_tiles, d_tc = d_tile - d_tr * n_col_tiles;
  int g = 0;
  for (; unit < total_units; unit += stride) {
    while (g < G - 1 && s_blk_end[g] <= tr) ++g;   // group of padded row block tr: first g with blk_end[g] > tr
    const int blk0 = g ? s_blk_end[g - 1] : 0, row0 = g ? s_row_end[g - 1] : 0;
    Loc l;
    l.g = g;
    l.m = row0 + (tr - blk0) * kTileRows + row_in_tile + 2 * w;
    l.j = tc * kTileBlocks + c;
    l.live = l.m < s_row_end[g] && l.j < nblk;
    BlockIn blk = {};
    float gs = 0.f;
    if (l.live) {
      blk = load_block<kVec>(x + l.m * row_stride + l.j * 16);
      gs = gs_ptr[g];
    }
    emit(unit, l, blk, gs);
    // next unit of this warp: unit + stride, digit by digit
    w += d_w;
    const int carry = w >= kWarpsPerTile ? 1 : 0;
    w -= carry * kWarpsPerTile;
    tc += d_tc + carry;
    tr += d_tr;
    if (tc >= n_col_tiles) {
      tc -= n_col_tiles;
      ++tr;
    }
  }
}

// Per-group global scale 2688 / max|x| (mslk/quantize/triton/legacy/global_scale.py:40-152): phase 1
// reduces |x| per group into an integer maximum (bf16 magnitudes order like their bit patterns).
__global__ void __launch_bounds__(256) group_amax_kernel(const __nv_bfloat16 *__restrict__ x, int M, int K,
                                                         int64_t row_stride, const int64_t *__restrict__ m_sizes, int G,
                                                         unsigned int *__restrict__ amax_bits,
                                                         int64_t *__restrict__ tensor_idx, unsigned int inf_bits) {
  __shared__ int s_row_end[kMaxStackedGroups];
  __shared__ int s_blk_end[kMaxStackedGroups];
  __shared__ unsigned int s_max[8];
  if (threadIdx.x < 32) build_stacked_tables(m_sizes, G, M, threadIdx.x, s_row_end, s_blk_end);
  __syncthreads();
  const int total_rows = s_row_end[G - 1];
  for (int row = blockIdx.x; row < total_rows; row += gridDim.x) {
    int lo = 0, hi = G - 1;   // first g with row_end[g] > row
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (s_row_end[mid] > row) hi = mid; else lo = mid + 1;
    }
    const uint16_t *src = reinterpret_cast<const uint16_t *>(x + row * row_stride);
    unsigned int mx = 0;
    const bool vec = (reinterpret_cast<uintptr_t>(src) & 15u) == 0;
    if (vec) {
      for (int v = threadIdx.x; v < K / 8; v += blockDim.x) {
        const uint4 d = *reinterpret_cast<const uint4 *>(src + v * 8);
        const uint32_t wd[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const unsigned int a = wd[i] & 0x7fff7fffu;
          const unsigned int l = a & 0xffffu, h = a >> 16;
          // NaN patterns (above the infinity pattern: 0x7f80 for bf16, 0x7c00 for fp16) are ignored, like max() does
          if (l <= inf_bits) mx = max(mx, l);
          if (h <= inf_bits) mx = max(mx, h);
        }
      }
      for (int k = (K / 8) * 8 + threadIdx.x; k < K; k += blockDim.x) {
        const unsigned int a = src[k] & 0x7fffu;
        if (a <= inf_bits) mx = max(mx, a);
      }
    } else {
      for (int k = threadIdx.x; k < K; k += blockDim.x) {
        const unsigned int a = src[k] & 0x7fffu;
        if (a <= inf_bits) mx = max(mx, a);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if ((threadIdx.x & 31) == 0) s_max[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned int m8 = 0;
      for (int i = 0; i < static_cast<int>(blockDim.x >> 5); ++i) m8 = max(m8, s_max[i]);
      atomicMax(amax_bits + lo, m8);
      if (tensor_idx) tensor_idx[row] = lo;
    }
    __syncthreads();
  }
}

// Phase 2: out[g] = 2688 / amax_g with the approximate division the reference's kernel lowers to
// (div.full), 1e-8 standing in for an all-zero group; groups without rows keep FLT_MAX.
__global__ void group_scale_finish_kernel(const unsigned int *__restrict__ amax_bits, const int64_t *__restrict__ m_sizes,
                                          int G, float *__restrict__ out, int is_half) {
  const int g = blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= G) return;
  if (m_sizes[g] <= 0) {
    out[g] = 3.4028234663852886e38f;
    return;
  }
  const float amax = is_half ? __half2float(__ushort_as_half(static_cast<unsigned short>(amax_bits[g])))
                             : __uint_as_float(amax_bits[g] << 16);
  float r;
  const float d = amax == 0.f ? 1e-8f : amax;
  asm("div.full.f32 %0, %1, %2;" : "=f"(r) : "f"(2688.0f), "f"(d));
  out[g] = r;
}

}  // namespace
}  // namespace mslk_b200

MSLK_API int mslk_b200_quantize_nvfp4_dt(const void *x, int dtype, int64_t M, int64_t K, int64_t row_stride,
                                         const float *global_scale, void *q, void *scales, void *stream) {
  using namespace mslk_b200;
  clear_error();
  if (dtype != MSLK_B200_BF16 && dtype != MSLK_B200_F16) return fail(1, "quantize_nvfp4: input must be bf16 or fp16");
  const bool half = dtype == MSLK_B200_F16;
  if (M < 0 || K < 0 || K % 16 != 0) return fail(1, "quantize_nvfp4: K must be a non-negative multiple of 16");
  if (M == 0 || K == 0) return 0;
  if (!x || !q || !scales) return fail(1, "quantize_nvfp4: null pointer argument");
  if (reinterpret_cast<uintptr_t>(q) & 7u) return fail(1, "quantize_nvfp4: output must be 8-byte aligned");
  if (M > 0x7fffff00LL || K > 0x7fffff00LL) return fail(1, "quantize_nvfp4: dimension too large");
  const int64_t n_row_tiles = (M + kTileRows - 1) / kTileRows;
  const int64_t n_col_tiles = (K / 16 + kTileBlocks - 1) / kTileBlocks;
  const int64_t total = n_row_tiles * n_col_tiles;
  if (total > 0x07ff0000LL) return fail(1, "quantize_nvfp4: tensor too large");
  const bool vec_ok = (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && row_stride % 8 == 0;
  const int64_t units = total * kWarpsPerTile;
  // persistent: the 6 CTAs that fit on an SM walk the units grid-stride, prefetching one unit ahead
  const int64_t cap = static_cast<int64_t>(sm_count()) * 6;
  const int64_t want = (units + kThreads / 32 - 1) / (kThreads / 32);
  const unsigned blocks = static_cast<unsigned>(want < cap ? want : cap);
  auto *xb = static_cast<const __nv_bfloat16 *>(x);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto go = [&](auto kernel) {
    kernel<<<blocks, kThreads, 0, st>>>(xb, static_cast<int>(M), static_cast<int>(K / 16), row_stride, global_scale,
                                        static_cast<uint8_t *>(q), static_cast<uint8_t *>(scales),
                                        static_cast<int>(n_col_tiles), static_cast<int>(units));
  };
  if (vec_ok) half ? go(quant_nvfp4_kernel<1, true>) : go(quant_nvfp4_kernel<1, false>);
  else half ? go(quant_nvfp4_kernel<0, true>) : go(quant_nvfp4_kernel<0, false>);
  return check_cuda(cudaGetLastError(), "quantize_nvfp4 launch");
}

MSLK_API int mslk_b200_quantize_nvfp4(const void *x, int64_t M, int64_t K, int64_t row_stride,
                                      const float *global_scale, void *q, void *scales, void *stream) {
  return mslk_b200_quantize_nvfp4_dt(x, MSLK_B200_BF16, M, K, row_stride, global_scale, q, scales, stream);
}

MSLK_API int mslk_b200_quantize_nvfp4_stacked_dt(const void *x, int dtype, int64_t M, int64_t K, int64_t row_stride,
                                                 const int64_t *m_sizes, int64_t G, const float *global_scale, void *q,
                                                 void *scales, void *stream) {
  using namespace mslk_b200;
  clear_error();
  const char *name = "quantize_nvfp4_stacked";
  if (dtype != MSLK_B200_BF16 && dtype != MSLK_B200_F16) return fail(1, "%s: input must be bf16 or fp16", name);
  const bool half = dtype == MSLK_B200_F16;
  if (M < 0 || K < 0 || K % 16 != 0) return fail(1, "%s: K must be a non-negative multiple of 16", name);
  if (G < 1 || G > kMaxStackedGroups) return fail(1, "%s: between 1 and %d groups are supported", name, kMaxStackedGroups);
  if (M == 0 || K == 0) return 0;
  if (!x || !q || !scales || !m_sizes || !global_scale) return fail(1, "%s: null pointer argument", name);
  if (reinterpret_cast<uintptr_t>(q) & 7u) return fail(1, "%s: output must be 8-byte aligned", name);
  if (M > 0x7fffff00LL || K > 0x7fffff00LL) return fail(1, "%s: dimension too large", name);
  const int64_t n_col_tiles = (K / 16 + kTileBlocks - 1) / kTileBlocks;
  const int64_t units_ub = ((M + kTileRows - 1) / kTileRows + G) * n_col_tiles * kWarpsPerTile;
  if (units_ub > 0x7fff0000LL) return fail(1, "%s: tensor too large", name);
  const bool vec_ok = (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && row_stride % 8 == 0;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 6;
  const int64_t want = (units_ub + kThreads / 32 - 1) / (kThreads / 32);
  const unsigned blocks = static_cast<unsigned>(want < cap ? want : cap);
  auto *xb = static_cast<const __nv_bfloat16 *>(x);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto go = [&](auto kernel) {
    kernel<<<blocks, kThreads, 0, st>>>(xb, static_cast<int>(M), static_cast<int>(K / 16), row_stride, global_scale, m_sizes,
                                        static_cast<int>(G), static_cast<uint8_t *>(q), static_cast<uint8_t *>(scales),
                                        static_cast<int>(n_col_tiles));
  };
  if (vec_ok) half ? go(quant_nvfp4_stacked_kernel<1, true>) : go(quant_nvfp4_stacked_kernel<1, false>);
  else half ? go(quant_nvfp4_stacked_kernel<0, true>) : go(quant_nvfp4_stacked_kernel<0, false>);
  return check_cuda(cudaGetLastError(), "quantize_nvfp4_stacked launch");
}

MSLK_API int mslk_b200_quantize_nvfp4_stacked(const void *x, int64_t M, int64_t K, int64_t row_stride,
                                              const int64_t *m_sizes, int64_t G, const float *global_scale, void *q,
                                              void *scales, void *stream) {
  return mslk_b200_quantize_nvfp4_stacked_dt(x, MSLK_B200_BF16, M, K, row_stride, m_sizes, G, global_scale, q, scales,
                                             stream);
}

MSLK_API int mslk_b200_calculate_group_max_dt(const void *x, int dtype, int64_t M, int64_t K, int64_t row_stride,
                                              const int64_t *m_sizes, int64_t G, float *global_scale,
                                              int64_t *tensor_idx, void *stream) {
  using namespace mslk_b200;
  clear_error();
  const char *name = "calculate_group_max";
  if (dtype != MSLK_B200_BF16 && dtype != MSLK_B200_F16) return fail(1, "%s: input must be bf16 or fp16", name);
  const bool half = dtype == MSLK_B200_F16;
  if (M < 0 || K < 0) return fail(1, "%s: bad shape", name);
  if (G < 1 || G > kMaxStackedGroups) return fail(1, "%s: between 1 and %d groups are supported", name, kMaxStackedGroups);
  if (!m_sizes || !global_scale) return fail(1, "%s: null pointer argument", name);
  if (M > 0x7fffff00LL || K > 0x7fffff00LL) return fail(1, "%s: dimension too large", name);
  if ((M > 0 && K > 0) && !x) return fail(1, "%s: null input", name);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // the output doubles as the integer accumulator of phase 1 (bf16 magnitude bits), rewritten by phase 2
  unsigned int *bits = reinterpret_cast<unsigned int *>(global_scale);
  if (int rc = check_cuda(cudaMemsetAsync(bits, 0, sizeof(float) * static_cast<size_t>(G), st), "memset")) return rc;
  if (M > 0 && K > 0) {
    const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
    const unsigned blocks = static_cast<unsigned>(M < cap ? M : cap);
    group_amax_kernel<<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(x), static_cast<int>(M), static_cast<int>(K),
                                              row_stride, m_sizes, static_cast<int>(G), bits, tensor_idx,
                                              half ? 0x7c00u : 0x7f80u);
    if (int rc = check_cuda(cudaGetLastError(), "calculate_group_max launch")) return rc;
  }
  group_scale_finish_kernel<<<static_cast<unsigned>((G + 127) / 128), 128, 0, st>>>(bits, m_sizes, static_cast<int>(G),
                                                                                   global_scale, half ? 1 : 0);
  return check_cuda(cudaGetLastError(), "calculate_group_max launch");
}

MSLK_API int mslk_b200_calculate_group_max(const void *x, int64_t M, int64_t K, int64_t row_stride,
                                           const int64_t *m_sizes, int64_t G, float *global_scale, int64_t *tensor_idx,
                                           void *stream) {
  return mslk_b200_calculate_group_max_dt(x, MSLK_B200_BF16, M, K, row_stride, m_sizes, G, global_scale, tensor_idx, stream);
}
