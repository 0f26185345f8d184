// Device helpers shared by the row-oriented elementwise kernels (SwiGLU + quantize, token gather /
// scatter): 16-byte streaming loads, bf16 / fp16 unpacking and packing, the approximate division the
// reference's Triton kernels lower to, e4m3 conversion and a block-wide maximum.
#pragma once

#include "common.cuh"

#include <cuda_fp16.h>

namespace mslk_b200 {
namespace rowwise {

// Full-range approximate division (not IEEE): what `a / b` on fp32 values becomes in a Triton kernel.
__device__ __forceinline__ float div_full(float a, float b) {
  float r;
  asm("div.full.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
// two fp32 -> two e4m3 bytes (round to nearest even, saturating), `lo` in the low byte
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}
// 16-byte read-only load that does not allocate in L1 (data used once)
__device__ __forceinline__ uint4 ld_stream_v4(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

template <typename T>
struct Elem;
template <>
struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ void unpack8(const uint4 &v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  // max |element| of the 8 packed values (exact: abs and max do not round)
  static __device__ __forceinline__ float absmax8(const uint4 &v) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    __nv_bfloat162 m = __habs2(*reinterpret_cast<const __nv_bfloat162 *>(&w[0]));
#pragma unroll
    for (int i = 1; i < 4; ++i) m = __hmax2(m, __habs2(*reinterpret_cast<const __nv_bfloat162 *>(&w[i])));
    return fmaxf(__bfloat162float(m.x), __bfloat162float(m.y));
  }
  static __device__ __forceinline__ uint32_t pack2(float lo, float hi) { return pack_bf16x2(lo, hi); }
  static __device__ __forceinline__ float load(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ __nv_bfloat16 make(float v) { return __float2bfloat16_rn(v); }
};
template <>
struct Elem<__half> {
  static __device__ __forceinline__ void unpack8(const uint4 &v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 p = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
      f[2 * i] = p.x;
      f[2 * i + 1] = p.y;
    }
  }
  static __device__ __forceinline__ float absmax8(const uint4 &v) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    __half2 m = __habs2(*reinterpret_cast<const __half2 *>(&w[0]));
#pragma unroll
    for (int i = 1; i < 4; ++i) m = __hmax2(m, __habs2(*reinterpret_cast<const __half2 *>(&w[i])));
    return fmaxf(__low2float(m), __high2float(m));
  }
  static __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&h);
  }
  static __device__ __forceinline__ float load(const __half *p) { return __half2float(*p); }
  static __device__ __forceinline__ __half make(float v) { return __float2half_rn(v); }
};

// Maximum over the block (blockDim.x a multiple of 32, at most 1024); s_part holds 32 floats.
__device__ __forceinline__ float block_max(float v, float *s_part) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x / 32] = v;
  __syncthreads();
  const int warps = blockDim.x / 32;
  float m = (threadIdx.x & 31) < warps ? s_part[threadIdx.x & 31] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  return m;
}

// One row quantized from registers: y[kVecs][8] scaled by `scale`, converted to e4m3 and stored as
// 8-byte pieces; vector i of this thread is vector threadIdx.x + i * nthreads of the row.
template <int kVecs>
__device__ __forceinline__ void store_row_e4m3(const float (&y)[kVecs][8], float scale, uint8_t *row, int nvec, int nthreads) {
#pragma unroll
  for (int i = 0; i < kVecs; ++i) {
    const int v = threadIdx.x + i * nthreads;
    if (v < nvec) {
      uint32_t o[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t lo = cvt_e4m3x2(__fmul_rn(y[i][4 * h], scale), __fmul_rn(y[i][4 * h + 1], scale));
        const uint32_t hi = cvt_e4m3x2(__fmul_rn(y[i][4 * h + 2], scale), __fmul_rn(y[i][4 * h + 3], scale));
        o[h] = lo | (hi << 16);
      }
      *reinterpret_cast<uint2 *>(row + static_cast<int64_t>(v) * 8) = make_uint2(o[0], o[1]);
    }
  }
}

}  // namespace rowwise
}  // namespace mslk_b200
