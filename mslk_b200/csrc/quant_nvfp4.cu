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
template <int kVec>
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
  int m, j;
  auto locate = [&](int u, int &mm, int &jj) {
    const int tile = u / kWarpsPerTile, w = u - tile * kWarpsPerTile;
    const int tr = tile / n_col_tiles, tc = tile - tr * n_col_tiles;
    mm = tr * kTileRows + row_in_tile + 2 * w;
    jj = tc * kTileBlocks + c;
    return mm < M && jj < nblk;
  };
  bool live = locate(unit, m, j);
  BlockIn cur{};
  if (live) cur = load_block<kVec>(x + m * row_stride + j * 16);
  while (unit < total_units) {
    // prefetch the next unit's block
    const int nunit = unit + stride;
    int nm = 0, nj = 0;
    bool nlive = false;
    BlockIn nxt{};
    if (nunit < total_units) {
      nlive = locate(nunit, nm, nj);
      if (nlive) nxt = load_block<kVec>(x + nm * row_stride + nj * 16);
    }
    uint8_t s8 = 0;
    if (live) {
      const uint32_t w[8] = {cur.a.x, cur.a.y, cur.a.z, cur.a.w, cur.b.x, cur.b.y, cur.b.z, cur.b.w};
      // block amax on the packed pairs (exact: max and abs do not round)
      __nv_bfloat162 mx = __habs2(*reinterpret_cast<const __nv_bfloat162 *>(&w[0]));
#pragma unroll
      for (int i = 1; i < 8; ++i) mx = __hmax2(mx, __habs2(*reinterpret_cast<const __nv_bfloat162 *>(&w[i])));
      const float bamax = fmaxf(__bfloat162float(mx.x), __bfloat162float(mx.y));
      float s = __fmul_rn(__fdiv_rn(bamax, 6.0f), gs);
      s = fminf(fmaxf(s, 0.001953125f), 448.0f);
      s8 = f32_to_e4m3(s);
      const float total = s_total[s8 & 127];
      float lo[8], hi[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        lo[2 * i] = __fmul_rn(__uint_as_float(w[i] << 16), total);
        lo[2 * i + 1] = __fmul_rn(__uint_as_float(w[i] & 0xffff0000u), total);
        hi[2 * i] = __fmul_rn(__uint_as_float(w[4 + i] << 16), total);
        hi[2 * i + 1] = __fmul_rn(__uint_as_float(w[4 + i] & 0xffff0000u), total);
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

}  // namespace
}  // namespace mslk_b200

MSLK_API int mslk_b200_quantize_nvfp4(const void *x, int64_t M, int64_t K, int64_t row_stride,
                                      const float *global_scale, void *q, void *scales, void *stream) {
  using namespace mslk_b200;
  clear_error();
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
  if (vec_ok)
    quant_nvfp4_kernel<1><<<blocks, kThreads, 0, st>>>(xb, static_cast<int>(M), static_cast<int>(K / 16), row_stride,
                                                          global_scale, static_cast<uint8_t *>(q),
                                                          static_cast<uint8_t *>(scales), static_cast<int>(n_col_tiles),
                                                          static_cast<int>(units));
  else
    quant_nvfp4_kernel<0><<<blocks, kThreads, 0, st>>>(xb, static_cast<int>(M), static_cast<int>(K / 16), row_stride,
                                                           global_scale, static_cast<uint8_t *>(q),
                                                           static_cast<uint8_t *>(scales), static_cast<int>(n_col_tiles),
                                                           static_cast<int>(units));
  return check_cuda(cudaGetLastError(), "quantize_nvfp4 launch");
}
