// MXFP4 quantization for sm_100a: bf16 / fp16 -> packed e2m1 with one e8m0 (power-of-two) scale per group of
// 32 (OCP MX) or 16 elements, scales in the 128 x 4 swizzled layout the block-scaled tensor-core instructions read.
//
// Arithmetic of the reference's kernel (mslk/quantize/triton/quantize_kernels/mx4.py:28-214 with
// fp4_primitives/scale.py:96-265), all of it integer work on fp32 bit patterns, so it is reproduced bit for bit:
//     e      = exponent of the group's max |x| rounded as `rounding_mode` says (floor: the fp32 exponent field;
//              even: after adding 2^21 - 1 to the bits; ceil: after adding 2^23 - 1), minus 2 (e2m1 spans 2^2),
//              clamped to [-127, 125]
//     scale  = byte e + 127                         (e8m0)
//     x^     = e2m1_rn_satfinite(x * 2^-e)          (the factor built from its exponent bits)
// Padded scale slots (rows up to a multiple of 128, groups up to a multiple of 4 per row) are written as 0.
//
// Stochastic rounding (rounding mode 3, fp4_primitives/scale.py:213-261): two counter-based random streams, Philox-4x32
// with 7 rounds, key = the 64-bit seed (low word first), counter = (offset, 0, 0, 0), first output word:
//     group stream    seed,               offset = row * (K / group) + group index:
//                     e = exponent of bits(max |x|) + (rand & (2^22 - 1)), then as above
//     element stream  seed ^ 0x5A5A5A5A,  offset = row * K + column:
//                     bits(x * 2^-e) + (rand & (2^22 - 1)) - (2^21 - 1) before the round-to-nearest conversion
// with 32-bit wrapping offsets; `row` is the row of X (dense) or of the padded scale matrix (stacked).  Integer work
// again, so the same seed gives the reference's bytes.
//
// Work unit = one warp's share of a 128-row x 4-group tile (one 512-byte scale atom): warp w of the tile takes rows
// {2w, 2w+1} + {0, 32, 64, 96} and the 4 groups of each, one group (64 or 32 input bytes) per lane.  With
// lane = (row & 1) * 16 + (row / 32) * 4 + group, the 32 scale bytes of a unit are the contiguous bytes [32w, 32w + 32)
// of the atom: one sector per warp store.  Units are walked grid-stride, the (tile row, tile column, warp slot) digits
// carried along without divisions, the next unit's group prefetched into registers.  HBM-bound: 2.53 bytes per
// element at group size 32.
//
// Stacked form (mslk/quantize/triton/quantize_kernels/mx4_stacked.py:34-360): rows of G segments stacked in one
// [M, K] tensor, segment g owning m_sizes[g] rows (device int64); its scale rows start on a 128-row boundary of the
// padded scale matrix (at sum_{i<g} roundup(m_i, 128)), which is what the grouped MXFP4 GEMM reads.  The scale buffer
// has M + 127 G rows (an upper bound that needs no host read of the sizes); every byte of it that is not a scale of a
// live group is written as 0.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

#include "../../include/mslk_b200.h"
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

// Philox-4x32, `kRounds` rounds, counter (c0, 0, 0, 0), key (k0, k1); returns the first word of the output block.
template <int kRounds>
__device__ __forceinline__ uint32_t philox_first_word(uint32_t k0, uint32_t k1, uint32_t c0) {
  constexpr uint32_t kMulA = 0xD2511F53u, kMulB = 0xCD9E8D57u, kKeyA = 0x9E3779B9u, kKeyB = 0xBB67AE85u;
  uint32_t c1 = 0, c2 = 0, c3 = 0;
#pragma unroll
  for (int r = 0; r < kRounds; ++r) {
    const uint64_t pa = static_cast<uint64_t>(kMulA) * c0, pb = static_cast<uint64_t>(kMulB) * c2;   // one wide multiply each
    c0 = static_cast<uint32_t>(pb >> 32) ^ c1 ^ k0;
    c2 = static_cast<uint32_t>(pa >> 32) ^ c3 ^ k1;
    c1 = static_cast<uint32_t>(pb);
    c3 = static_cast<uint32_t>(pa);
    k0 += kKeyA;
    k1 += kKeyB;
  }
  return c0;
}

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

constexpr int kMaxSegments = 1024;

struct Mx4Params {
  const void *x;
  uint8_t *q;
  uint8_t *scales;
  int64_t M, K, row_stride;
  int64_t scale_rows;       // rows of the scale buffer (dense: a multiple of 128; stacked: M + 127 G)
  int padded_cols;          // scale slots per padded row, multiple of 4
  int scale_cols;           // K / group
  int round_add;            // added to the fp32 bits of the group maximum before its exponent is taken; -1: nearest
  uint32_t seed_lo, seed_hi;   // stochastic rounding only
  const int64_t *m_sizes;   // stacked form: rows per segment (device), else null
  int G;
};

// Inclusive prefix sums of the segment sizes (rows) and of their 128-row padded extents; one warp.
__device__ __forceinline__ void build_segment_tables(const int64_t *m_sizes, int G, int64_t M, int lane, int *row_end,
                                                     int *pad_end) {
  int row_carry = 0, pad_carry = 0;
  for (int base = 0; base < G; base += 32) {
    const int g = base + lane;
    long long mg = g < G ? m_sizes[g] : 0;
    mg = mg < 0 ? 0 : (mg > M ? M : mg);
    int rows = static_cast<int>(mg), pads = (rows + 127) / 128 * 128;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int r = __shfl_up_sync(0xffffffffu, rows, o), b = __shfl_up_sync(0xffffffffu, pads, o);
      if (lane >= o) {
        rows += r;
        pads += b;
      }
    }
    if (g < G) {
      row_end[g] = static_cast<int>(min(M, static_cast<int64_t>(row_carry) + rows));
      pad_end[g] = pad_carry + pads;
    }
    row_carry = static_cast<int>(min(M, static_cast<int64_t>(row_carry) + __shfl_sync(0xffffffffu, rows, 31)));
    pad_carry += __shfl_sync(0xffffffffu, pads, 31);
  }
}

constexpr int kWarpsPerTile = 16;   // one warp quantizes 8 rows x 4 groups of a 128 x 4 tile
constexpr int kThreadsMx = 256;

template <int kGroup>
struct GroupIn {
  uint4 v[kGroup / 8];   // 32 or 16 two-byte elements
};

template <typename T, int kGroup, bool kStacked, bool kSr>
__global__ void __launch_bounds__(kThreadsMx, kSr ? 2 : 4) quant_mx4_kernel(const Mx4Params p) {
  __shared__ int s_row_end[kStacked ? kMaxSegments : 1];
  __shared__ int s_pad_end[kStacked ? kMaxSegments : 1];
  const int tid = threadIdx.x, lane = tid & 31;
  if constexpr (kStacked) {
    if (tid < 32) build_segment_tables(p.m_sizes, p.G, p.M, lane, s_row_end, s_pad_end);
    __syncthreads();
  }
  const int n_col_tiles = p.padded_cols / 4;
  const int n_row_tiles = static_cast<int>((p.scale_rows + 127) / 128);
  const int total_units = n_row_tiles * n_col_tiles * kWarpsPerTile;
  const int64_t scale_bytes = p.scale_rows * p.padded_cols;
  const int c = lane & 3, row_in_tile = ((lane >> 2) & 3) * 32 + (lane >> 4);
  const int stride = gridDim.x * (kThreadsMx / 32);
  int unit = blockIdx.x * (kThreadsMx / 32) + (tid >> 5);
  if (unit >= total_units) return;
  int tile = unit / kWarpsPerTile, w = unit - tile * kWarpsPerTile;
  int tr = tile / n_col_tiles, tc = tile - tr * n_col_tiles;
  const int d_tile = stride / kWarpsPerTile, d_w = stride - d_tile * kWarpsPerTile;
  const int d_tr = d_tile / n_col_tiles, d_tc = d_tile - d_tr * n_col_tiles;
  int g = 0;
  auto padded_row = [&]() { return tr * 128 + row_in_tile + 2 * w; };   // row of the padded scale matrix
  auto locate_here = [&](int64_t &row, int &col) {
    const int pr = padded_row();
    col = tc * 4 + c;
    bool live = pr < p.M;
    row = pr;
    if constexpr (kStacked) {
      while (g < p.G - 1 && s_pad_end[g] <= tr * 128) ++g;   // tile rows only grow along a warp's units
      const int pad0 = g ? s_pad_end[g - 1] : 0, row0 = g ? s_row_end[g - 1] : 0;
      row = row0 + (pr - pad0);
      live = pr < s_pad_end[g] && row < s_row_end[g];
    }
    return live && col < p.scale_cols;
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
  auto load = [&](int64_t row, int col, GroupIn<kGroup> &gi) {
    const uint4 *src = reinterpret_cast<const uint4 *>(static_cast<const T *>(p.x) + row * p.row_stride +
                                                       static_cast<int64_t>(col) * kGroup);
#pragma unroll
    for (int j = 0; j < kGroup / 8; ++j)
      asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                   : "=r"(gi.v[j].x), "=r"(gi.v[j].y), "=r"(gi.v[j].z), "=r"(gi.v[j].w) : "l"(src + j));
  };
  int64_t row;
  int col;
  bool live = locate_here(row, col);
  int prow = padded_row();
  GroupIn<kGroup> cur{};
  if (live) load(row, col, cur);
  while (unit < total_units) {
    const int nunit = unit + stride;
    int64_t nrow = 0;
    int ncol = 0, nprow = 0;
    bool nlive = false;
    GroupIn<kGroup> nxt{};
    if (nunit < total_units) {
      advance();
      nlive = locate_here(nrow, ncol);
      nprow = padded_row();
      if (nlive) load(nrow, ncol, nxt);
    }
    uint8_t s8 = 0;
    if (live) {
      float v[kGroup];
      float amax = 0.f;
#pragma unroll
      for (int j = 0; j < kGroup / 8; ++j) {
        const T *h = reinterpret_cast<const T *>(&cur.v[j]);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          v[8 * j + e] = to_f32<T>(h[e]);
          amax = fmaxf(amax, fabsf(v[8 * j + e]));
        }
      }
      int e;
      // row of the random streams' offsets: the row of X, or of the padded scale matrix for stacked segments
      const uint32_t sr_row = kStacked ? static_cast<uint32_t>(prow) : static_cast<uint32_t>(row);
      if constexpr (kSr) {
        const uint32_t off = sr_row * static_cast<uint32_t>(p.scale_cols) + static_cast<uint32_t>(col);
        const uint32_t rnd = philox_first_word<7>(p.seed_lo, p.seed_hi, off) & 0x3fffffu;
        e = static_cast<int>(((__float_as_uint(amax) + rnd) & 0x7f800000u) >> 23) - 127 - 2;
      } else if (p.round_add < 0) {
        // nearest: floor(log2(max) + 0.5), a zero maximum standing in as the smallest normal bf16 (2^-126)
        e = static_cast<int>(floorf(log2f(amax == 0.f ? 1.17549435e-38f : amax) + 0.5f)) - 2;
      } else {
        e = static_cast<int>(((__float_as_uint(amax) + static_cast<uint32_t>(p.round_add)) & 0x7f800000u) >> 23) - 127 - 2;
      }
      e = max(-127, min(125, e));
      const float inv = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);
      uint8_t *dst = p.q + row * (p.K / 2) + static_cast<int64_t>(col) * (kGroup / 2);
#pragma unroll
      for (int j = 0; j < kGroup / 16; ++j) {
        uint32_t wd[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float y[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            y[k] = v[16 * j + 8 * h + k] * inv;
            if constexpr (kSr) {
              const uint32_t off = sr_row * static_cast<uint32_t>(p.K) +
                                   static_cast<uint32_t>(col * kGroup + 16 * j + 8 * h + k);
              const uint32_t rnd = philox_first_word<7>(p.seed_lo ^ 0x5A5A5A5Au, p.seed_hi, off) & 0x3fffffu;
              y[k] = __uint_as_float(__float_as_uint(y[k]) + rnd - 0x1fffffu);
            }
          }
          wd[h] = cvt_e2m1x8(y);
        }
        *reinterpret_cast<uint2 *>(dst + 8 * j) = make_uint2(wd[0], wd[1]);
      }
      s8 = static_cast<uint8_t>(e + 127);
    }
    const int64_t soff = static_cast<int64_t>(unit) * 32 + lane;   // zero for padding rows / columns / slack
    if (soff < scale_bytes) p.scales[soff] = s8;
    unit = nunit;
    row = nrow;
    col = ncol;
    prow = nprow;
    live = nlive;
    cur = nxt;
  }
}

int run_mx4(const char *name, const void *x, int dtype, int64_t M, int64_t K, int64_t row_stride, const int64_t *m_sizes,
            int64_t G, int group_size, int rounding_mode, uint64_t seed, void *q, void *scales, cudaStream_t st) {
  const bool stacked = m_sizes != nullptr;
  if (M < 0 || K < 0) return fail(1, "%s: bad shape", name);
  if (group_size != 32 && group_size != 16) return fail(1, "%s: group_size must be 32 or 16 (got %d)", name, group_size);
  if (K % group_size != 0) return fail(1, "%s: K (%lld) must be a multiple of the group size %d", name, (long long)K, group_size);
  if (dtype != MSLK_B200_BF16 && dtype != MSLK_B200_F16) return fail(1, "%s: input must be bf16 or fp16", name);
  if (stacked && (G < 1 || G > kMaxSegments)) return fail(1, "%s: between 1 and %d segments are supported", name, kMaxSegments);
  int round_add;
  switch (rounding_mode) {
    case 0: round_add = -1; break;                // nearest: floor(log2(max) + 0.5)
    case 1: round_add = 0; break;                 // floor
    case 2: round_add = (1 << 21) - 1; break;     // even: pre-round at the e2m1 mantissa
    case 3: round_add = 0; break;                 // stochastic: random bits take its place
    case 4: round_add = (1 << 23) - 1; break;     // ceil (the reference's default)
    default:
      return fail(1, "%s: rounding mode %d does not exist (nearest = 0, floor = 1, even = 2, stochastic = 3, ceil = 4)",
                  name, rounding_mode);
  }
  if (K == 0 || (M == 0 && !stacked)) return 0;
  if (!scales || (M > 0 && (!x || !q))) return fail(1, "%s: null pointer argument", name);
  if (M > 0x7fff0000LL - 127 * G) return fail(1, "%s: too many rows", name);
  if ((reinterpret_cast<uintptr_t>(x) & 15u) || (row_stride * 2) % 16 != 0)
    return fail(1, "%s: input rows must be 16-byte aligned", name);
  if (reinterpret_cast<uintptr_t>(q) & 7u) return fail(1, "%s: output must be 8-byte aligned", name);
  Mx4Params p;
  p.x = x;
  p.q = static_cast<uint8_t *>(q);
  p.scales = static_cast<uint8_t *>(scales);
  p.M = M;
  p.K = K;
  p.row_stride = row_stride;
  p.scale_rows = stacked ? M + 127 * G : (M + 127) / 128 * 128;
  p.scale_cols = static_cast<int>(K / group_size);
  p.padded_cols = (p.scale_cols + 3) / 4 * 4;
  p.round_add = round_add;
  p.seed_lo = static_cast<uint32_t>(seed);
  p.seed_hi = static_cast<uint32_t>(seed >> 32);
  p.m_sizes = m_sizes;
  p.G = static_cast<int>(G);
  const int64_t units = ((p.scale_rows + 127) / 128) * (p.padded_cols / 4) * kWarpsPerTile;
  if (units > 0x7fff0000LL) return fail(1, "%s: tensor too large", name);
  const int64_t want = (units + 7) / 8;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 4;
  const unsigned blocks = static_cast<unsigned>(want < cap ? want : cap);
  auto go = [&](auto kernel) { kernel<<<blocks, kThreadsMx, 0, st>>>(p); };
  auto pick = [&](auto type_tag, auto group_tag) {
    using T = decltype(type_tag);
    constexpr int kG = decltype(group_tag)::value;
    if (rounding_mode == 3) stacked ? go(quant_mx4_kernel<T, kG, true, true>) : go(quant_mx4_kernel<T, kG, false, true>);
    else stacked ? go(quant_mx4_kernel<T, kG, true, false>) : go(quant_mx4_kernel<T, kG, false, false>);
  };
  if (dtype == MSLK_B200_BF16) {
    if (group_size == 32) pick(__nv_bfloat16{}, std::integral_constant<int, 32>{});
    else pick(__nv_bfloat16{}, std::integral_constant<int, 16>{});
  } else {
    if (group_size == 32) pick(__half{}, std::integral_constant<int, 32>{});
    else pick(__half{}, std::integral_constant<int, 16>{});
  }
  return check_cuda(cudaGetLastError(), name);
}

}  // namespace
}  // namespace mslk_b200

MSLK_API int mslk_b200_quantize_mx4(const void *x, int dtype, int64_t M, int64_t K, int64_t row_stride, int group_size,
                                    int rounding_mode, void *q, void *scales, void *stream) {
  using namespace mslk_b200;
  clear_error();
  if (rounding_mode == 3) return fail(1, "quantize_mx4: stochastic rounding takes a seed: call mslk_b200_quantize_mx4_seeded");
  return run_mx4("quantize_mx4", x, dtype, M, K, row_stride, nullptr, 1, group_size, rounding_mode, 0, q, scales,
                 static_cast<cudaStream_t>(stream));
}

MSLK_API int mslk_b200_quantize_mx4_seeded(const void *x, int dtype, int64_t M, int64_t K, int64_t row_stride,
                                           int group_size, int rounding_mode, uint64_t seed, void *q, void *scales,
                                           void *stream) {
  using namespace mslk_b200;
  clear_error();
  return run_mx4("quantize_mx4", x, dtype, M, K, row_stride, nullptr, 1, group_size, rounding_mode, seed, q, scales,
                 static_cast<cudaStream_t>(stream));
}

MSLK_API int mslk_b200_quantize_mx4_stacked(const void *x, int dtype, int64_t M, int64_t K, int64_t row_stride,
                                            const int64_t *m_sizes, int64_t G, int group_size, int rounding_mode, void *q,
                                            void *scales, void *stream) {
  using namespace mslk_b200;
  clear_error();
  if (!m_sizes) return fail(1, "quantize_mx4_stacked: m_sizes is null");
  if (rounding_mode == 3)
    return fail(1, "quantize_mx4_stacked: stochastic rounding takes a seed: call mslk_b200_quantize_mx4_stacked_seeded");
  return run_mx4("quantize_mx4_stacked", x, dtype, M, K, row_stride, m_sizes, G, group_size, rounding_mode, 0, q, scales,
                 static_cast<cudaStream_t>(stream));
}

MSLK_API int mslk_b200_quantize_mx4_stacked_seeded(const void *x, int dtype, int64_t M, int64_t K, int64_t row_stride,
                                                   const int64_t *m_sizes, int64_t G, int group_size, int rounding_mode,
                                                   uint64_t seed, void *q, void *scales, void *stream) {
  using namespace mslk_b200;
  clear_error();
  if (!m_sizes) return fail(1, "quantize_mx4_stacked: m_sizes is null");
  return run_mx4("quantize_mx4_stacked", x, dtype, M, K, row_stride, m_sizes, G, group_size, rounding_mode, seed, q,
                 scales, static_cast<cudaStream_t>(stream));
}
