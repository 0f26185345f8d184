// Fused SwiGLU + per-row FP8 quantization for sm_100a:  y = x0 * sigmoid(x0) * x1, then
// (q, inv_scale) = rowwise e4m3 quantization of y.  This is the step between the gate+up and
// the down projection of an FFN (the reference's Triton kernel: mslk/moe/activation.py:220-294).
//
// Arithmetic, operation for operation as the reference's kernel lowers on NVIDIA GPUs:
//     e      = ex2.approx(-x0 * log2(e))             sigmoid(x0) = 1 / (1 + e), division = div.full
//                                                     (evaluated by an equivalent shorter sequence, see silu_mul)
//     y      = (x0 * sigmoid) * x1                    fp32
//     rmax   = min(max(max_k |y|, 1e-12), *scale_ub)
//     yscale = 448 / rmax                             div.full;  inv_scale = 1 / yscale (div.full)
//     q      = e4m3_rn_satfinite(y * yscale)
// (Note the differences from quantize_fp8_row: reciprocal scale applied by multiplication,
// floor 1e-12, the INVERSE scale is what is stored.)
//
// HBM-bound: 4 bytes read + 1 byte written per element (bf16 inputs).  One block per row; each
// thread keeps its share of y in registers (fp32) across the row-max reduction, so x0/x1 are read
// once.  Rows at or beyond *valid_token_count are left untouched.
#include "../../include/mslk_b200.h"
#include "common.cuh"
#include "host.h"
#include "rowwise_elem.cuh"

#include <algorithm>

namespace mslk_b200 {
namespace {

using namespace rowwise;

__device__ __forceinline__ float ex2_approx_ftz(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float rcp_approx_ftz(float x) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
// The reference's kernel lowers sigmoid(x) to  div.full(1, 1 + ex2.approx(-x * log2(e))).  Two
// substitutions keep every result bit identical while shortening the instruction sequence (both
// were checked exhaustively on a B200, over all 2^32 inputs of the first and every divisor in
// [1, +inf] of the second):
//   * 1 + ex2.approx(t) == 1 + ex2.approx.ftz(t): the variants differ only where the exponential is
//     subnormal, which the addition to 1 absorbs;
//   * div.full(1, d) == rcp.approx.ftz(d) for 1 <= d <= 2^126; larger d (x below about -87.3)
//     need the range scaling of div.full.
// kFast = true asserts x >= -87 (so that d < 2^126); callers test that per vector of inputs.
template <bool kFast>
__device__ __forceinline__ float silu_mul(float x0, float x1) {
  const float e = ex2_approx_ftz(__fmul_rn(-x0, 1.4426950408889634f));
  const float d = __fadd_rn(1.0f, e);
  const float sig = kFast ? rcp_approx_ftz(d) : div_full(1.0f, d);
  return __fmul_rn(__fmul_rn(x0, sig), x1);
}
constexpr float kFastSigmoidMinX = -87.0f;

// y[j] = silu_mul(f0[j], f1[j]) for 8 elements; one range test for the whole vector
__device__ __forceinline__ void silu_mul8(const float (&f0)[8], const float (&f1)[8], float (&y)[8]) {
  const float lo = fminf(fminf(fminf(f0[0], f0[1]), fminf(f0[2], f0[3])), fminf(fminf(f0[4], f0[5]), fminf(f0[6], f0[7])));
  if (lo >= kFastSigmoidMinX) {   // false for NaN as well: the general form handles it
#pragma unroll
    for (int j = 0; j < 8; ++j) y[j] = silu_mul<true>(f0[j], f1[j]);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) y[j] = silu_mul<false>(f0[j], f1[j]);
  }
}

struct SiluParams {
  const void *x0;
  const void *x1;
  uint8_t *q;
  float *inv_scale;
  const float *scale_ub;
  const int *valid_token_count;
  int64_t T, D, stride0, stride1;
};

// Vector path: D % 8 == 0, 16-byte aligned rows; kVecs 8-element vectors per thread, the block size
// chosen by the host so that kVecs * blockDim.x covers the row with less than one warp of slack.
template <typename T, int kVecs, int kMaxThreads>
__global__ void __launch_bounds__(kMaxThreads) silu_mul_quant_vec_kernel(const SiluParams p) {
  __shared__ float s_part[32];
  const int kBlock = blockDim.x;
  const int64_t row = blockIdx.x;
  if (p.valid_token_count && row >= *p.valid_token_count) return;
  const T *r0 = static_cast<const T *>(p.x0) + row * p.stride0;
  const T *r1 = static_cast<const T *>(p.x1) + row * p.stride1;
  const int nvec = static_cast<int>(p.D / 8);
  uint4 a[kVecs], b[kVecs];
#pragma unroll
  for (int i = 0; i < kVecs; ++i) {
    const int v = threadIdx.x + i * kBlock;
    if (v < nvec) {
      a[i] = ld_stream_v4(r0 + static_cast<int64_t>(v) * 8);
      b[i] = ld_stream_v4(r1 + static_cast<int64_t>(v) * 8);
    } else {
      a[i] = make_uint4(0, 0, 0, 0);
      b[i] = make_uint4(0, 0, 0, 0);
    }
  }
  float y[kVecs][8];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < kVecs; ++i) {
    float f0[8], f1[8];
    Elem<T>::unpack8(a[i], f0);
    Elem<T>::unpack8(b[i], f1);
    silu_mul8(f0, f1, y[i]);
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(y[i][j]));
  }
  amax = block_max(amax, s_part);
  float rmax = fmaxf(amax, 1e-12f);
  if (p.scale_ub) rmax = fminf(rmax, *p.scale_ub);
  const float y_scale = div_full(448.0f, rmax);
  if (threadIdx.x == 0) p.inv_scale[row] = div_full(1.0f, y_scale);
  store_row_e4m3<kVecs>(y, y_scale, p.q + row * p.D, nvec, kBlock);
}

// General path (any D / alignment): two passes, y recomputed in the second.
template <typename T, int kBlock>
__global__ void __launch_bounds__(kBlock) silu_mul_quant_generic_kernel(const SiluParams p) {
  __shared__ float s_part[32];
  const int64_t row = blockIdx.x;
  if (p.valid_token_count && row >= *p.valid_token_count) return;
  const T *r0 = static_cast<const T *>(p.x0) + row * p.stride0;
  const T *r1 = static_cast<const T *>(p.x1) + row * p.stride1;
  float amax = 0.f;
  for (int64_t k = threadIdx.x; k < p.D; k += kBlock) amax = fmaxf(amax, fabsf(silu_mul<false>(Elem<T>::load(r0 + k), Elem<T>::load(r1 + k))));
  amax = block_max(amax, s_part);
  float rmax = fmaxf(amax, 1e-12f);
  if (p.scale_ub) rmax = fminf(rmax, *p.scale_ub);
  const float y_scale = div_full(448.0f, rmax);
  if (threadIdx.x == 0) p.inv_scale[row] = div_full(1.0f, y_scale);
  uint8_t *qr = p.q + row * p.D;
  for (int64_t k = threadIdx.x; k < p.D; k += kBlock) {
    const float y = silu_mul<false>(Elem<T>::load(r0 + k), Elem<T>::load(r1 + k));
    qr[k] = static_cast<uint8_t>(cvt_e4m3x2(__fmul_rn(y, y_scale), 0.f) & 0xffu);
  }
}

template <typename T, int kVecs>
int launch_vec(const SiluParams &p, int64_t nvec, cudaStream_t st) {
  const int threads = static_cast<int>((nvec + kVecs - 1) / kVecs + 31) / 32 * 32;
  if (threads <= 512)
    silu_mul_quant_vec_kernel<T, kVecs, 512><<<static_cast<unsigned>(p.T), threads, 0, st>>>(p);
  else
    silu_mul_quant_vec_kernel<T, kVecs, 1024><<<static_cast<unsigned>(p.T), threads, 0, st>>>(p);
  return check_cuda(cudaGetLastError(), "silu_mul_quant launch");
}

template <typename T>
int launch_typed(const SiluParams &p, bool vec_ok, cudaStream_t st) {
  const int64_t nvec = p.D / 8;
  if (vec_ok && nvec <= 4 * 1024) {
    // four vectors per thread once that still gives a block of 128 threads; fewer for short rows
    if (nvec >= 4 * 128) return launch_vec<T, 4>(p, nvec, st);
    if (nvec >= 2 * 64) return launch_vec<T, 2>(p, nvec, st);
    return launch_vec<T, 1>(p, nvec, st);
  }
  silu_mul_quant_generic_kernel<T, 256><<<static_cast<unsigned>(p.T), 256, 0, st>>>(p);
  return check_cuda(cudaGetLastError(), "silu_mul_quant launch");
}

// y = x0 * sigmoid(x0) * x1 without quantization (the reference's _mslk_silu_mul,
// mslk/moe/activation.py:181-217): elementwise, output in the input dtype, contiguous [T, D].
template <typename T, bool kVec>
__global__ void __launch_bounds__(256) silu_mul_kernel(const SiluParams p, T *__restrict__ y) {
  const int64_t valid = p.valid_token_count ? min(static_cast<int64_t>(*p.valid_token_count), p.T) : p.T;
  const T *x0 = static_cast<const T *>(p.x0);
  const T *x1 = static_cast<const T *>(p.x1);
  const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
  if (kVec) {
    const int64_t per_row = p.D / 8, total = valid * per_row;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += step) {
      const int64_t row = i / per_row, v = i - row * per_row;
      float f0[8], f1[8];
      Elem<T>::unpack8(ld_stream_v4(x0 + row * p.stride0 + v * 8), f0);
      Elem<T>::unpack8(ld_stream_v4(x1 + row * p.stride1 + v * 8), f1);
      float r[8];
      silu_mul8(f0, f1, r);
      uint4 o;
      o.x = Elem<T>::pack2(r[0], r[1]);
      o.y = Elem<T>::pack2(r[2], r[3]);
      o.z = Elem<T>::pack2(r[4], r[5]);
      o.w = Elem<T>::pack2(r[6], r[7]);
      *reinterpret_cast<uint4 *>(y + row * p.D + v * 8) = o;
    }
  } else {
    const int64_t total = valid * p.D;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += step) {
      const int64_t row = i / p.D, k = i - row * p.D;
      y[i] = Elem<T>::make(silu_mul<false>(Elem<T>::load(x0 + row * p.stride0 + k), Elem<T>::load(x1 + row * p.stride1 + k)));
    }
  }
}

template <typename T>
int launch_silu_mul(const SiluParams &p, bool vec_ok, void *y, cudaStream_t st) {
  const int64_t work = vec_ok ? p.T * (p.D / 8) : p.T * p.D;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 32;
  const unsigned blocks = static_cast<unsigned>(std::max<int64_t>(1, std::min<int64_t>((work + 255) / 256, cap)));
  if (vec_ok)
    silu_mul_kernel<T, true><<<blocks, 256, 0, st>>>(p, static_cast<T *>(y));
  else
    silu_mul_kernel<T, false><<<blocks, 256, 0, st>>>(p, static_cast<T *>(y));
  return check_cuda(cudaGetLastError(), "silu_mul launch");
}

}  // namespace
}  // namespace mslk_b200

MSLK_API int mslk_b200_silu_mul_quant(const void *x0, const void *x1, int dtype, int64_t T, int64_t D, int64_t stride0,
                                      int64_t stride1, const float *scale_ub, const int *valid_token_count, void *q,
                                      float *inv_scale, void *stream) {
  using namespace mslk_b200;
  clear_error();
  if (T < 0 || D < 0) return fail(1, "silu_mul_quant: bad shape");
  if (T == 0 || D == 0) return 0;
  if (T > 0x7fffffffLL) return fail(1, "silu_mul_quant: too many rows");
  if (!x0 || !x1 || !q || !inv_scale) return fail(1, "silu_mul_quant: null pointer argument");
  if (dtype != MSLK_B200_BF16 && dtype != MSLK_B200_F16) return fail(1, "silu_mul_quant: inputs must be bf16 or fp16");
  SiluParams p{x0, x1, static_cast<uint8_t *>(q), inv_scale, scale_ub, valid_token_count, T, D, stride0, stride1};
  const bool vec_ok = D % 8 == 0 && stride0 % 8 == 0 && stride1 % 8 == 0 &&
                      ((reinterpret_cast<uintptr_t>(x0) | reinterpret_cast<uintptr_t>(x1)) & 15u) == 0 &&
                      (reinterpret_cast<uintptr_t>(q) & 7u) == 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return dtype == MSLK_B200_BF16 ? launch_typed<__nv_bfloat16>(p, vec_ok, st) : launch_typed<__half>(p, vec_ok, st);
}

MSLK_API int mslk_b200_silu_mul(const void *x0, const void *x1, int dtype, int64_t T, int64_t D, int64_t stride0,
                                int64_t stride1, const int *valid_token_count, void *y, void *stream) {
  using namespace mslk_b200;
  clear_error();
  if (T < 0 || D < 0) return fail(1, "silu_mul: bad shape");
  if (T == 0 || D == 0) return 0;
  if (!x0 || !x1 || !y) return fail(1, "silu_mul: null pointer argument");
  if (dtype != MSLK_B200_BF16 && dtype != MSLK_B200_F16) return fail(1, "silu_mul: inputs must be bf16 or fp16");
  SiluParams p{x0, x1, nullptr, nullptr, nullptr, valid_token_count, T, D, stride0, stride1};
  const bool vec_ok = D % 8 == 0 && stride0 % 8 == 0 && stride1 % 8 == 0 &&
                      ((reinterpret_cast<uintptr_t>(x0) | reinterpret_cast<uintptr_t>(x1) | reinterpret_cast<uintptr_t>(y)) & 15u) == 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return dtype == MSLK_B200_BF16 ? launch_silu_mul<__nv_bfloat16>(p, vec_ok, y, st) : launch_silu_mul<__half>(p, vec_ok, y, st);
}
