// NVFP4 quantization for sm_100a: bf16 -> packed e2m1 with one e4m3 scale per 16
// elements (stored in the 128x4-tile swizzled layout the block-scaled MMA reads)
// and an optional fp32 per-tensor global scale.
//
// Arithmetic (bit-exact with the reference's kernel,
// mslk/quantize/triton/quantize_kernels/nvfp4.py:213-296, precise-math branch):
//     s    = e4m3_rn(clamp((bamax / 6) * gs, 2^-9, 448))     per 16-element block
//     x^   = e2m1_rn_satfinite(x * (gs / float(s)))
// with IEEE fp32 divisions.  One thread owns one 16-element block: two 16-byte
// loads, one 8-byte store of packed nibbles and one scale byte.  The grid spans
// the padded scale matrix so that padding rows / columns are written as zero.
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

__global__ void __launch_bounds__(256) quant_nvfp4_kernel(const __nv_bfloat16 *__restrict__ x, int64_t M, int64_t K,
                                                          int64_t row_stride, const float *__restrict__ gs_ptr,
                                                          uint8_t *__restrict__ q, uint8_t *__restrict__ scales,
                                                          int64_t pad_rows, int64_t pad_cols) {
  const int64_t nblk = K / 16;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= pad_rows * pad_cols) return;
  const int64_t m = idx / pad_cols, j = idx - m * pad_cols;
  const int64_t ncb = pad_cols / 4;
  const int64_t ri = m % 128;
  const int64_t soff = ((m / 128) * ncb + j / 4) * 512 + (ri % 32) * 16 + (ri / 32) * 4 + (j % 4);
  if (m >= M || j >= nblk) {
    scales[soff] = 0;
    return;
  }
  const float gs = gs_ptr ? *gs_ptr : 1.0f;
  const __nv_bfloat16 *src = x + m * row_stride + j * 16;
  float f[16];
  if ((reinterpret_cast<uintptr_t>(src) & 15u) == 0) {
    const uint4 a = reinterpret_cast<const uint4 *>(src)[0];
    const uint4 b = reinterpret_cast<const uint4 *>(src)[1];
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) f[i] = __bfloat162float(src[i]);
  }
  float bamax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) bamax = fmaxf(bamax, fabsf(f[i]));
  float s = __fmul_rn(__fdiv_rn(bamax, 6.0f), gs);
  s = fminf(fmaxf(s, 0.001953125f), 448.0f);
  const uint8_t s8 = f32_to_e4m3(s);
  scales[soff] = s8;
  const float total = __fdiv_rn(gs, e4m3_to_f32(s8));
  float lo[8], hi[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    lo[i] = __fmul_rn(f[i], total);
    hi[i] = __fmul_rn(f[8 + i], total);
  }
  uint2 out = make_uint2(cvt_e2m1x8(lo), cvt_e2m1x8(hi));
  *reinterpret_cast<uint2 *>(q + m * (K / 2) + j * 8) = out;
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
  const int64_t pad_rows = (M + 127) / 128 * 128;
  const int64_t pad_cols = (K / 16 + 3) / 4 * 4;
  const int64_t total = pad_rows * pad_cols;
  const int64_t blocks = (total + 255) / 256;
  if (blocks > 0x7fffffffLL) return fail(1, "quantize_nvfp4: tensor too large");
  quant_nvfp4_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16 *>(x), M, K, row_stride, global_scale, static_cast<uint8_t *>(q),
      static_cast<uint8_t *>(scales), pad_rows, pad_cols);
  return check_cuda(cudaGetLastError(), "quantize_nvfp4 launch");
}
