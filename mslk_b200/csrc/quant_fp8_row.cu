// Per-row FP8 (e4m3fn) quantization for sm_100a.
//
// Arithmetic (bit-exact with the reference's GPU kernel,
// mslk/quantize/triton/fp8_quantize.py:131-207):
//     cur   = min(max(amax_row, eps), *scale_ub)
//     scale = cur / 448                      IEEE fp32 division
//     q     = e4m3_rn_satfinite(x / scale)   IEEE fp32 division
// The clamp to +-448 of the reference is the saturation of the conversion.
//
// HBM-bound: 2 bytes read + 1 byte written per bf16 element, so the fast path
// reads every row exactly once with 16-byte loads, keeps it in registers across
// the amax reduction, and writes 8-byte (bf16/fp16 input) or 4-byte (fp32 input)
// packed results.  At most four (eight for very long rows) vectors per thread
// keep the kernel near 40 registers, so an SM holds 1536+ threads and ~96 KB of
// loads in flight; the per-element instruction count (about 11, mostly on the
// integer/logic pipe: unpack, packed |max|, e4m3 conversion) is what bounds it
// once the loads are covered.  x/scale is evaluated as q0 = x*r, q = fma(fma(-q0, scale, x), r, q0)
// with r = 1/scale correctly rounded; for operands in the guarded range this is
// the correctly rounded quotient (three FMA-pipe operations instead of a
// division sequence).  Rows whose scale falls outside the guarded range use a
// true division.
#include "../../include/mslk_b200.h"
#include "common.cuh"
#include "host.h"

namespace mslk_b200 {
namespace {

constexpr float kFp8Max = 448.0f;

template <typename T>
struct Elem;
template <>
struct Elem<float> {
  static constexpr int kPerVec = 4;
};
template <>
struct Elem<__nv_bfloat16> {
  static constexpr int kPerVec = 8;
};
template <>
struct Elem<__half> {
  static constexpr int kPerVec = 8;
};

__device__ __forceinline__ uint4 ld_stream_v4(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

template <typename T>
__device__ __forceinline__ void unpack(const uint4 &v, float (&f)[Elem<T>::kPerVec]);
template <>
__device__ __forceinline__ void unpack<float>(const uint4 &v, float (&f)[4]) {
  f[0] = __uint_as_float(v.x);
  f[1] = __uint_as_float(v.y);
  f[2] = __uint_as_float(v.z);
  f[3] = __uint_as_float(v.w);
}
template <>
__device__ __forceinline__ void unpack<__nv_bfloat16>(const uint4 &v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <>
__device__ __forceinline__ void unpack<__half>(const uint4 &v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 p = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
    f[2 * i] = p.x;
    f[2 * i + 1] = p.y;
  }
}

// two fp32 -> two e4m3 bytes (lo in bits 0..7), round-to-nearest-even, saturating
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}

struct RowScale {
  float scale;  // what is stored
  float rcp;    // 1/scale correctly rounded
  bool fast;    // scale inside the range where the FMA form equals IEEE division
};

__device__ __forceinline__ RowScale make_row_scale(float amax, float eps, const float *scale_ub) {
  float cur = fmaxf(amax, eps);
  if (scale_ub) cur = fminf(cur, *scale_ub);
  RowScale rs;
  rs.scale = __fdiv_rn(cur, kFp8Max);
  rs.rcp = __frcp_rn(rs.scale);
  // 2^-40 .. 2^40 and a bounded largest quotient (scale_ub can make |x|/scale
  // huge): no intermediate of the FMA form can overflow or lose bits to underflow
  // for any quotient that does not round to zero in e4m3.
  rs.fast = (rs.scale > 9.0949470e-13f) && (rs.scale < 1.0995116e12f) && (amax * rs.rcp < 1.0e30f);
  return rs;
}

// x / scale, correctly rounded.  Fast form: q0 = x*r; d = q0*scale - x (exact in an FMA);
// q = q0 - d*r.  Written with d = -(residual) so that x = -0 yields -0 like a division does.
template <bool kFast>
__device__ __forceinline__ float divide(float x, const RowScale &rs) {
  if constexpr (kFast) {
    const float q0 = __fmul_rn(x, rs.rcp);
    const float d = __fmaf_rn(q0, rs.scale, -x);
    return __fmaf_rn(-d, rs.rcp, q0);
  } else {
    return __fdiv_rn(x, rs.scale);
  }
}

// One 16-byte vector of inputs -> packed e4m3 bytes (2 words for 16-bit inputs, 1 for fp32).
template <typename T, bool kFast>
__device__ __forceinline__ void quantize_vec(const uint4 &v, const RowScale &rs, uint32_t (&o)[Elem<T>::kPerVec / 4]) {
  constexpr int kE = Elem<T>::kPerVec;
  float f[kE];
  unpack<T>(v, f);
#pragma unroll
  for (int j = 0; j < kE / 4; ++j) {
    const uint32_t lo = cvt_e4m3x2(divide<kFast>(f[4 * j], rs), divide<kFast>(f[4 * j + 1], rs));
    const uint32_t hi = cvt_e4m3x2(divide<kFast>(f[4 * j + 2], rs), divide<kFast>(f[4 * j + 3], rs));
    o[j] = lo | (hi << 16);
  }
}

template <typename T>
__device__ __forceinline__ void store_quantized(uint8_t *row, int v, const uint32_t (&o)[Elem<T>::kPerVec / 4]) {
  if constexpr (Elem<T>::kPerVec == 8) {
    *reinterpret_cast<uint2 *>(row + static_cast<int64_t>(v) * 8) = make_uint2(o[0], o[1]);
  } else {
    *reinterpret_cast<uint32_t *>(row + static_cast<int64_t>(v) * 4) = o[0];
  }
}

// Running |max| over 16-byte vectors.  16-bit inputs stay packed (sign bits masked off,
// then one two-lane max per word); the pair is only widened once at the end.
template <typename T>
struct AmaxAcc;
template <>
struct AmaxAcc<float> {
  float m = 0.f;
  __device__ __forceinline__ void add(const uint4 &v) {
    m = fmaxf(fmaxf(m, fabsf(__uint_as_float(v.x))), fabsf(__uint_as_float(v.y)));
    m = fmaxf(fmaxf(m, fabsf(__uint_as_float(v.z))), fabsf(__uint_as_float(v.w)));
  }
  __device__ __forceinline__ float get() const { return m; }
};
template <>
struct AmaxAcc<__nv_bfloat16> {
  uint32_t a = 0, b = 0;
  static __device__ __forceinline__ uint32_t mx(uint32_t acc, uint32_t w) {
    const __nv_bfloat162 r = __hmax2(*reinterpret_cast<const __nv_bfloat162 *>(&acc),
                                     __habs2(*reinterpret_cast<const __nv_bfloat162 *>(&w)));
    return *reinterpret_cast<const uint32_t *>(&r);
  }
  __device__ __forceinline__ void add(const uint4 &v) {
    a = mx(mx(a, v.x), v.z);
    b = mx(mx(b, v.y), v.w);
  }
  __device__ __forceinline__ float get() const {
    const uint32_t m = mx(a, b);
    return fmaxf(__uint_as_float(m << 16), __uint_as_float(m & 0xffff0000u));
  }
};
template <>
struct AmaxAcc<__half> {
  uint32_t a = 0, b = 0;
  static __device__ __forceinline__ uint32_t mx(uint32_t acc, uint32_t w) {
    const __half2 r = __hmax2(*reinterpret_cast<const __half2 *>(&acc), __habs2(*reinterpret_cast<const __half2 *>(&w)));
    return *reinterpret_cast<const uint32_t *>(&r);
  }
  __device__ __forceinline__ void add(const uint4 &v) {
    a = mx(mx(a, v.x), v.z);
    b = mx(mx(b, v.y), v.w);
  }
  __device__ __forceinline__ float get() const {
    const uint32_t m = mx(a, b);
    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&m));
    return fmaxf(f.x, f.y);
  }
};

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

struct QuantParams {
  const void *x;
  uint8_t *q;
  float *scale;
  const float *scale_ub;
  const int64_t *zero_start;  // [B*M] or nullptr
  int64_t rows;               // B*M*N
  int64_t M, N, K, K_out;
  int64_t sb, sm, sn, sk;     // element strides of x
  float eps;
  int uniform_pitch;          // rows are sn elements apart throughout: base = r * sn, no index split needed
};

__device__ __forceinline__ int64_t row_base(const QuantParams &p, int64_t r, bool &empty) {
  if (p.uniform_pitch && p.zero_start == nullptr) {
    empty = false;
    return r * p.sn;
  }
  const int64_t mn = p.M * p.N;
  const int64_t b = r / mn, rem = r - b * mn;
  const int64_t m = rem / p.N, n = rem - m * p.N;
  empty = p.zero_start != nullptr && n >= p.zero_start[b * p.M + m];
  return b * p.sb + m * p.sm + n * p.sn;
}

// ---------------------------------------------------------------------------
// Fast path: unit inner stride, 16-byte aligned rows, K and K_out multiples of
// the vector length.  kThreadsPerRow threads own one row; each holds kVecs
// 16-byte vectors in registers.  kThreadsPerRow == 32: one warp per row, several
// rows per block.  kThreadsPerRow == blockDim.x: one block per row.
// ---------------------------------------------------------------------------
template <typename T, int kVecs, int kThreadsPerRow, int kBlock>
__global__ void __launch_bounds__(kBlock) quant_fp8_row_vec_kernel(const QuantParams p) {
  constexpr int kE = Elem<T>::kPerVec;
  constexpr int kRowsPerBlock = kBlock / kThreadsPerRow;
  constexpr int kWarpsPerRow = kThreadsPerRow / 32;
  __shared__ float s_part[kBlock / 32];
  griddep_launch_dependents();   // the next kernel of the stream may start its prologue
  griddep_wait();                // ... and this one touches memory only after the previous kernel has finished

  const int tid = threadIdx.x;
  const int t_in_row = tid % kThreadsPerRow;
  const int64_t r = static_cast<int64_t>(blockIdx.x) * kRowsPerBlock + tid / kThreadsPerRow;
  const bool row_ok = r < p.rows;

  const int nvec_in = static_cast<int>(p.K / kE);
  const int nvec_out = static_cast<int>(p.K_out / kE);

  bool empty = true;
  int64_t base = 0;
  if (row_ok) base = row_base(p, r, empty);
  const T *xr = static_cast<const T *>(p.x) + base;

  uint4 v[kVecs];
#pragma unroll
  for (int i = 0; i < kVecs; ++i) {
    const int vi = t_in_row + i * kThreadsPerRow;
    if (row_ok && !empty && vi < nvec_in) {
      v[i] = ld_stream_v4(xr + static_cast<int64_t>(vi) * kE);
    } else {
      v[i] = make_uint4(0, 0, 0, 0);
    }
  }
  AmaxAcc<T> acc;
#pragma unroll
  for (int i = 0; i < kVecs; ++i) acc.add(v[i]);
  float amax = warp_max(acc.get());
  if constexpr (kWarpsPerRow > 1) {
    const int warp = tid / 32;
    if ((tid & 31) == 0) s_part[warp] = amax;
    __syncthreads();
    const int w0 = (tid / kThreadsPerRow) * kWarpsPerRow;
    float m = 0.f;
#pragma unroll
    for (int w = 0; w < kWarpsPerRow; ++w) m = fmaxf(m, s_part[w0 + w]);
    amax = m;
  }
  if (!row_ok) return;

  const RowScale rs = make_row_scale(amax, p.eps, p.scale_ub);
  if (t_in_row == 0) p.scale[r] = rs.scale;

  uint8_t *qr = p.q + r * p.K_out;
  if (rs.fast) {
#pragma unroll
    for (int i = 0; i < kVecs; ++i) {
      const int vi = t_in_row + i * kThreadsPerRow;
      if (vi < nvec_out) {
        uint32_t o[kE / 4];
        quantize_vec<T, true>(v[i], rs, o);
        store_quantized<T>(qr, vi, o);
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < kVecs; ++i) {
      const int vi = t_in_row + i * kThreadsPerRow;
      if (vi < nvec_out) {
        uint32_t o[kE / 4];
        quantize_vec<T, false>(v[i], rs, o);
        store_quantized<T>(qr, vi, o);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// General path: any strides, any K / K_out, any alignment.  One block per row,
// two passes (the second pass re-reads the row from L2).
// ---------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float load_as_float(const T *p);
template <>
__device__ __forceinline__ float load_as_float<float>(const float *p) {
  return *p;
}
template <>
__device__ __forceinline__ float load_as_float<__nv_bfloat16>(const __nv_bfloat16 *p) {
  return __bfloat162float(*p);
}
template <>
__device__ __forceinline__ float load_as_float<__half>(const __half *p) {
  return __half2float(*p);
}

template <typename T, int kBlock>
__global__ void __launch_bounds__(kBlock) quant_fp8_row_generic_kernel(const QuantParams p) {
  __shared__ float s_part[kBlock / 32];
  for (int64_t r = blockIdx.x; r < p.rows; r += gridDim.x) {
    bool empty;
    const int64_t base = row_base(p, r, empty);
    const T *xr = static_cast<const T *>(p.x) + base;
    const int64_t k_in = empty ? 0 : p.K;
    float amax = 0.f;
    for (int64_t k = threadIdx.x; k < k_in; k += kBlock) amax = fmaxf(amax, fabsf(load_as_float<T>(xr + k * p.sk)));
    amax = warp_max(amax);
    __syncthreads();  // s_part reuse across rows
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x / 32] = amax;
    __syncthreads();
    amax = 0.f;
#pragma unroll
    for (int w = 0; w < kBlock / 32; ++w) amax = fmaxf(amax, s_part[w]);
    const RowScale rs = make_row_scale(amax, p.eps, p.scale_ub);
    if (threadIdx.x == 0) p.scale[r] = rs.scale;
    uint8_t *qr = p.q + r * p.K_out;
    for (int64_t k = threadIdx.x; k < p.K_out; k += kBlock) {
      const float x = k < k_in ? load_as_float<T>(xr + k * p.sk) : 0.f;
      qr[k] = static_cast<uint8_t>(cvt_e4m3x2(divide<false>(x, rs), 0.f) & 0xffu);
    }
  }
}

template <typename T, int kVecs, int kThreadsPerRow, int kBlock>
int launch_vec(const QuantParams &p, cudaStream_t st) {
  constexpr int kRowsPerBlock = kBlock / kThreadsPerRow;
  const int64_t blocks = (p.rows + kRowsPerBlock - 1) / kRowsPerBlock;
  if (blocks > 0x7fffffffLL) return fail(1, "quantize_fp8_row: too many rows (%lld)", (long long)p.rows);
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  cfg.gridDim = dim3(static_cast<unsigned>(blocks), 1, 1);
  cfg.blockDim = dim3(kBlock, 1, 1);
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_attribute(&attr[0]);
  return check_cuda(cudaLaunchKernelEx(&cfg, quant_fp8_row_vec_kernel<T, kVecs, kThreadsPerRow, kBlock>, p),
                    "quantize_fp8_row launch");
}

template <typename T>
int launch_typed(const QuantParams &p, bool vec_ok, cudaStream_t st) {
  constexpr int kE = Elem<T>::kPerVec;
  if (vec_ok) {
    const int64_t nvec = p.K_out / kE;
    // Threads per row and vectors per thread are fitted to the row so that few load slots idle
    // (K = 5120 on <4,256> left 37 % of them empty: 5.0 TB/s, on <5,128> 5.9 TB/s).  Rows longer
    // than 1024 vectors keep 256 threads and take more vectors per thread: blocks of 512 threads
    // quantise occupancy too coarsely (8192 x 28672: 5.98 TB/s with <7,512>, 6.64 with <14,256>).
    if (nvec <= 32 * 1) return launch_vec<T, 1, 32, 256>(p, st);
    if (nvec <= 32 * 2) return launch_vec<T, 2, 32, 256>(p, st);
    if (nvec <= 32 * 4) return launch_vec<T, 4, 32, 256>(p, st);
    if (nvec <= 64 * 4) return launch_vec<T, 4, 64, 256>(p, st);
    if (nvec <= 128 * 4) return launch_vec<T, 4, 128, 256>(p, st);
    if (nvec <= 128 * 5) return launch_vec<T, 5, 128, 256>(p, st);   // K = 5120 (MoE hidden size): no idle load slots
    if (nvec <= 256 * 3) return launch_vec<T, 3, 256, 256>(p, st);
    if (nvec <= 256 * 4) return launch_vec<T, 4, 256, 256>(p, st);
    if (nvec <= 256 * 5) return launch_vec<T, 5, 256, 256>(p, st);
    if (nvec <= 256 * 6) return launch_vec<T, 6, 256, 256>(p, st);
    if (nvec <= 256 * 7) return launch_vec<T, 7, 256, 256>(p, st);
    if (nvec <= 256 * 8) return launch_vec<T, 8, 256, 256>(p, st);
    if (nvec <= 256 * 10) return launch_vec<T, 10, 256, 256>(p, st);
    if (nvec <= 256 * 12) return launch_vec<T, 12, 256, 256>(p, st);
    if (nvec <= 256 * 14) return launch_vec<T, 14, 256, 256>(p, st);
    if (nvec <= 256 * 16) return launch_vec<T, 16, 256, 256>(p, st);
  }
  const int64_t blocks = p.rows < 148 * 16 ? p.rows : 148 * 16;
  quant_fp8_row_generic_kernel<T, 256><<<static_cast<unsigned>(blocks), 256, 0, st>>>(p);
  return check_cuda(cudaGetLastError(), "quantize_fp8_row launch");
}

}  // namespace
}  // namespace mslk_b200

MSLK_API int mslk_b200_quantize_fp8_row(const void *x, int dtype, int64_t B, int64_t M, int64_t N, int64_t K,
                                        int64_t K_out, int64_t sb, int64_t sm, int64_t sn, int64_t sk,
                                        const float *scale_ub, const int64_t *zero_start_index_M, float eps,
                                        void *q, float *scale, void *stream) {
  using namespace mslk_b200;
  clear_error();
  if (B < 0 || M < 0 || N < 0 || K < 0 || K_out < K) return fail(1, "quantize_fp8_row: bad shape");
  const int64_t rows = B * M * N;
  if (rows == 0) return 0;
  if (!x && K > 0) return fail(1, "quantize_fp8_row: null input");
  if (!q && K_out > 0) return fail(1, "quantize_fp8_row: null output");
  if (!scale) return fail(1, "quantize_fp8_row: null scale output");
  QuantParams p;
  p.x = x;
  p.q = static_cast<uint8_t *>(q);
  p.scale = scale;
  p.scale_ub = scale_ub;
  p.zero_start = zero_start_index_M;
  p.rows = rows;
  p.M = M;
  p.N = N;
  p.K = K;
  p.K_out = K_out;
  p.sb = sb;
  p.sm = sm;
  p.sn = sn;
  p.sk = sk;
  p.eps = eps;
  p.uniform_pitch = ((M == 1 || sm == N * sn) && (B == 1 || sb == M * N * sn)) ? 1 : 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int esz = dtype == MSLK_B200_F32 ? 4 : 2;
  const int per_vec = 16 / esz;
  const bool vec_ok = K > 0 && sk == 1 && (K % per_vec) == 0 && (K_out % per_vec) == 0 &&
                      (reinterpret_cast<uintptr_t>(x) % 16) == 0 && (sb * esz) % 16 == 0 && (sm * esz) % 16 == 0 &&
                      (sn * esz) % 16 == 0 && (reinterpret_cast<uintptr_t>(q) % 8) == 0;
  switch (dtype) {
    case MSLK_B200_F32: return launch_typed<float>(p, vec_ok, st);
    case MSLK_B200_BF16: return launch_typed<__nv_bfloat16>(p, vec_ok, st);
    case MSLK_B200_F16: return launch_typed<__half>(p, vec_ok, st);
    default: return fail(1, "quantize_fp8_row: unsupported dtype code %d", dtype);
  }
}
