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
// One thread per scale slot of the padded scale matrix: it loads its group (64 or 32 bytes), reduces, converts and
// stores 16 or 8 packed bytes and one scale byte.  HBM-bound: 2.53 bytes per element at group size 32.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

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

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

struct Mx4Params {
  const void *x;
  uint8_t *q;
  uint8_t *scales;
  int64_t M, K, row_stride;
  int64_t padded_rows;      // multiple of 128
  int padded_cols;          // scale slots per padded row, multiple of 4
  int scale_cols;           // K / group
  int round_add;            // added to the fp32 bits of the group maximum before its exponent is taken
};

template <typename T, int kGroup>
__global__ void __launch_bounds__(256) quant_mx4_kernel(const Mx4Params p) {
  const int64_t slots = p.padded_rows * p.padded_cols;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < slots;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / p.padded_cols;
    const int c = static_cast<int>(i - r * p.padded_cols);
    // swizzled position of scale (r, c): 128-row block, 4-column block, then (r % 32) * 16 + (r / 32 % 4) * 4 + c % 4
    const int64_t soff = (r / 128) * (static_cast<int64_t>(p.padded_cols / 4) * 512) + (c / 4) * 512 + (r % 32) * 16 +
                         ((r % 128) / 32) * 4 + (c % 4);
    if (r >= p.M || c >= p.scale_cols) {
      p.scales[soff] = 0;
      continue;
    }
    const T *src = static_cast<const T *>(p.x) + r * p.row_stride + static_cast<int64_t>(c) * kGroup;
    float v[kGroup];
#pragma unroll
    for (int j = 0; j < kGroup / 8; ++j) {
      const uint4 raw = *reinterpret_cast<const uint4 *>(src + 8 * j);
      const T *h = reinterpret_cast<const T *>(&raw);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[8 * j + e] = to_f32<T>(h[e]);
    }
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < kGroup; ++j) amax = fmaxf(amax, fabsf(v[j]));
    int e = static_cast<int>(((__float_as_uint(amax) + static_cast<uint32_t>(p.round_add)) & 0x7f800000u) >> 23) - 127 - 2;
    e = max(-127, min(125, e));
    const float inv = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);
    uint8_t *dst = p.q + r * (p.K / 2) + static_cast<int64_t>(c) * (kGroup / 2);
#pragma unroll
    for (int j = 0; j < kGroup / 16; ++j) {
      uint32_t w[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float y[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) y[k] = v[16 * j + 8 * h + k] * inv;
        w[h] = cvt_e2m1x8(y);
      }
      *reinterpret_cast<uint2 *>(dst + 8 * j) = make_uint2(w[0], w[1]);
    }
    p.scales[soff] = static_cast<uint8_t>(e + 127);
  }
}

}  // namespace
}  // namespace mslk_b200

MSLK_API int mslk_b200_quantize_mx4(const void *x, int dtype, int64_t M, int64_t K, int64_t row_stride, int group_size,
                                    int rounding_mode, void *q, void *scales, void *stream) {
  using namespace mslk_b200;
  clear_error();
  const char *name = "quantize_mx4";
  if (M < 0 || K < 0) return fail(1, "%s: bad shape", name);
  if (group_size != 32 && group_size != 16) return fail(1, "%s: group_size must be 32 or 16 (got %d)", name, group_size);
  if (K % group_size != 0) return fail(1, "%s: K (%lld) must be a multiple of the group size %d", name, (long long)K, group_size);
  if (dtype != MSLK_B200_BF16 && dtype != MSLK_B200_F16) return fail(1, "%s: input must be bf16 or fp16", name);
  int round_add;
  switch (rounding_mode) {
    case 1: round_add = 0; break;                 // floor
    case 2: round_add = (1 << 21) - 1; break;     // even: pre-round at the e2m1 mantissa
    case 4: round_add = (1 << 23) - 1; break;     // ceil (the reference's default)
    default:
      return fail(1, "%s: rounding mode %d is not implemented (floor = 1, even = 2, ceil = 4 are; nearest and stochastic "
                     "depend on the GPU's approximate log2 / a Philox stream)", name, rounding_mode);
  }
  if (M == 0 || K == 0) return 0;
  if (!x || !q || !scales) return fail(1, "%s: null pointer argument", name);
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
  p.padded_rows = (M + 127) / 128 * 128;
  p.scale_cols = static_cast<int>(K / group_size);
  p.padded_cols = (p.scale_cols + 3) / 4 * 4;
  p.round_add = round_add;
  const int64_t slots = p.padded_rows * p.padded_cols;
  const int64_t want = (slots + 255) / 256;
  const unsigned blocks = static_cast<unsigned>(want < 148 * 32 ? want : 148 * 32);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == MSLK_B200_BF16) {
    if (group_size == 32) quant_mx4_kernel<__nv_bfloat16, 32><<<blocks, 256, 0, st>>>(p);
    else quant_mx4_kernel<__nv_bfloat16, 16><<<blocks, 256, 0, st>>>(p);
  } else {
    if (group_size == 32) quant_mx4_kernel<__half, 32><<<blocks, 256, 0, st>>>(p);
    else quant_mx4_kernel<__half, 16><<<blocks, 256, 0, st>>>(p);
  }
  return check_cuda(cudaGetLastError(), "quantize_mx4 launch");
}
