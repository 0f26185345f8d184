// Token gather / scatter steps either side of the grouped GEMM of a mixture-of-experts layer
// (the reference's Triton kernels in mslk/moe/gather_scatter.py), for sm_100a.  All HBM-bound.
//
//   gather_scale_dense_tokens        out[i]  = dtype(f32(x[tok[i]]) * f32(scores[tok[i], exp[i]]))            :431-486
//   gather_scale_quant_dense_tokens  v = f32(x[tok[i]]) * score;  rmax = min(max(max|v|, 1e-12), *ub);
//                                    os = 448 / rmax;  inv_scale[i] = 1 / os;  q[i] = e4m3((v) * os)           :537-655
//   scatter_add_dense_tokens         out[tok[i]] += in[i]          (atomic, in the tensors' dtype)             :489-526
//   scatter_add_padded_tokens        out[tok[i]] += in[rank(i), i] for the first sum(counts) rows, rank(i) =
//                                    (expert owning stacked row i) / (E / EP)                                    :677-740
// Rows at or past *valid_token_count are skipped.  The two divisions of the quantizing gather are the
// approximate full-range division (div.full) the reference's kernel lowers to, so its bytes and scales
// agree bit for bit; everything else is exact fp32 arithmetic with one rounding.
#include "../../include/mslk_b200.h"
#include "common.cuh"
#include "host.h"
#include "rowwise_elem.cuh"

#include <algorithm>

namespace mslk_b200 {
namespace {

using namespace rowwise;

__device__ __forceinline__ int64_t load_index(const void *p, int bits, int64_t i) {
  return bits == 64 ? static_cast<const int64_t *>(p)[i] : static_cast<int64_t>(static_cast<const int32_t *>(p)[i]);
}
__device__ __forceinline__ float load_as_f32(const void *p, int dtype, int64_t i) {
  if (dtype == MSLK_B200_BF16) return __bfloat162float(static_cast<const __nv_bfloat16 *>(p)[i]);
  if (dtype == MSLK_B200_F16) return __half2float(static_cast<const __half *>(p)[i]);
  return static_cast<const float *>(p)[i];
}

struct GatherParams {
  const void *x;
  const void *token_indices;
  const void *expert_indices;
  const void *scores;
  const float *scale_ub;
  const int *valid_token_count;
  void *out;          // gather: [a, D] in the dtype of x; quantizing gather: [a, D] bytes
  float *inv_scale;   // quantizing gather only
  int64_t T, D, a, E, stride_t, stride_e;
  int token_bits, expert_bits, scores_dtype;
  int *status;
};

// Source row and score of output row `row`; false (and a status flag) when an index is out of range.
__device__ __forceinline__ bool locate_row(const GatherParams &p, int64_t row, int64_t &ti, float &score) {
  ti = load_index(p.token_indices, p.token_bits, row);
  const int64_t ei = load_index(p.expert_indices, p.expert_bits, row);
  if (ti < 0 || ti >= p.T || ei < 0 || ei >= p.E) {
    if (threadIdx.x == 0) atomicOr(p.status, kStatusBadGatherIndex);
    return false;
  }
  score = load_as_f32(p.scores, p.scores_dtype, ti * p.stride_t + ei * p.stride_e);
  return true;
}

// ---------------------------------------------------------------- gather + scale
template <typename T, bool kVec>
__global__ void __launch_bounds__(1024) gather_scale_kernel(const GatherParams p) {
  const int64_t row = blockIdx.x;
  if (p.valid_token_count && row >= *p.valid_token_count) return;
  int64_t ti;
  float score;
  if (!locate_row(p, row, ti, score)) return;
  const T *src = static_cast<const T *>(p.x) + ti * p.D;
  T *dst = static_cast<T *>(p.out) + row * p.D;
  if (kVec) {
    const int nvec = static_cast<int>(p.D / 8);
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float f[8];
      Elem<T>::unpack8(ld_stream_v4(src + static_cast<int64_t>(v) * 8), f);
      uint4 o;
      o.x = Elem<T>::pack2(__fmul_rn(f[0], score), __fmul_rn(f[1], score));
      o.y = Elem<T>::pack2(__fmul_rn(f[2], score), __fmul_rn(f[3], score));
      o.z = Elem<T>::pack2(__fmul_rn(f[4], score), __fmul_rn(f[5], score));
      o.w = Elem<T>::pack2(__fmul_rn(f[6], score), __fmul_rn(f[7], score));
      *reinterpret_cast<uint4 *>(dst + static_cast<int64_t>(v) * 8) = o;
    }
  } else {
    for (int64_t k = threadIdx.x; k < p.D; k += blockDim.x) dst[k] = Elem<T>::make(__fmul_rn(Elem<T>::load(src + k), score));
  }
}

// ---------------------------------------------------------------- gather + scale + per-row FP8 quantize
// One CTA per output row, the scaled row kept in registers (kVecs vectors of 8 per thread), so the
// source row is read once (the reference reads it twice, the second time from L2).
template <typename T, int kVecs, int kMaxThreads>
__global__ void __launch_bounds__(kMaxThreads) gather_scale_quant_vec_kernel(const GatherParams p) {
  __shared__ float s_part[32];
  const int64_t row = blockIdx.x;
  if (p.valid_token_count && row >= *p.valid_token_count) return;
  int64_t ti;
  float score;
  if (!locate_row(p, row, ti, score)) return;
  const T *src = static_cast<const T *>(p.x) + ti * p.D;
  const int nvec = static_cast<int>(p.D / 8);
  const int nthreads = blockDim.x;
  uint4 raw[kVecs];
#pragma unroll
  for (int i = 0; i < kVecs; ++i) {
    const int v = threadIdx.x + i * nthreads;
    raw[i] = v < nvec ? ld_stream_v4(src + static_cast<int64_t>(v) * 8) : make_uint4(0, 0, 0, 0);
  }
  // Row maximum of |x * score|: rounding is monotone, so it is |fl(max|x| * score)|; the packed inputs
  // stay in registers (16 instead of 32 per thread) and the products are formed again when they are stored.
  float xmax = 0.f;
#pragma unroll
  for (int i = 0; i < kVecs; ++i) xmax = fmaxf(xmax, Elem<T>::absmax8(raw[i]));
  const float amax = block_max(fabsf(__fmul_rn(xmax, score)), s_part);
  float rmax = fmaxf(amax, 1e-12f);
  if (p.scale_ub) rmax = fminf(rmax, *p.scale_ub);
  const float out_scale = div_full(448.0f, rmax);
  if (threadIdx.x == 0) p.inv_scale[row] = div_full(1.0f, out_scale);
  uint8_t *qr = static_cast<uint8_t *>(p.out) + row * p.D;
#pragma unroll
  for (int i = 0; i < kVecs; ++i) {
    const int v = threadIdx.x + i * nthreads;
    if (v < nvec) {
      float f[8];
      Elem<T>::unpack8(raw[i], f);
      uint32_t o[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t lo = cvt_e4m3x2(__fmul_rn(__fmul_rn(f[4 * h], score), out_scale),
                                       __fmul_rn(__fmul_rn(f[4 * h + 1], score), out_scale));
        const uint32_t hi = cvt_e4m3x2(__fmul_rn(__fmul_rn(f[4 * h + 2], score), out_scale),
                                       __fmul_rn(__fmul_rn(f[4 * h + 3], score), out_scale));
        o[h] = lo | (hi << 16);
      }
      *reinterpret_cast<uint2 *>(qr + static_cast<int64_t>(v) * 8) = make_uint2(o[0], o[1]);
    }
  }
}

// Any D / alignment: two passes over the source row.
template <typename T>
__global__ void __launch_bounds__(256) gather_scale_quant_generic_kernel(const GatherParams p) {
  __shared__ float s_part[32];
  const int64_t row = blockIdx.x;
  if (p.valid_token_count && row >= *p.valid_token_count) return;
  int64_t ti;
  float score;
  if (!locate_row(p, row, ti, score)) return;
  const T *src = static_cast<const T *>(p.x) + ti * p.D;
  float amax = 0.f;
  for (int64_t k = threadIdx.x; k < p.D; k += blockDim.x) amax = fmaxf(amax, fabsf(__fmul_rn(Elem<T>::load(src + k), score)));
  amax = block_max(amax, s_part);
  float rmax = fmaxf(amax, 1e-12f);
  if (p.scale_ub) rmax = fminf(rmax, *p.scale_ub);
  const float out_scale = div_full(448.0f, rmax);
  if (threadIdx.x == 0) p.inv_scale[row] = div_full(1.0f, out_scale);
  uint8_t *qr = static_cast<uint8_t *>(p.out) + row * p.D;
  for (int64_t k = threadIdx.x; k < p.D; k += blockDim.x)
    qr[k] = static_cast<uint8_t>(cvt_e4m3x2(__fmul_rn(__fmul_rn(Elem<T>::load(src + k), score), out_scale), 0.f) & 0xffu);
}

// ---------------------------------------------------------------- scatter-add
constexpr int kI32 = MSLK_B200_I32;

struct ScatterParams {
  void *out;
  const void *in;
  const void *token_indices;
  const int *valid_token_count;   // dense variant
  const void *token_counts;       // padded variant: [E]
  int64_t rows;                   // dense: a; padded: T_K (upper bound of the stacked rows)
  int64_t D, T;                   // T = rows of out
  int64_t E, EP;
  int token_bits, count_bits;
  int *status;
};

// 16 bytes of `in` added atomically to 16 bytes of `out` (relaxed, device scope), in the tensors' dtype
template <int kDtype>
__device__ __forceinline__ void red_add_16B(void *dst, const uint4 &v) {
  if constexpr (kDtype == MSLK_B200_BF16) {
    asm volatile("red.relaxed.gpu.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(v.x), "r"(v.y),
                 "r"(v.z), "r"(v.w)
                 : "memory");
  } else if constexpr (kDtype == MSLK_B200_F16) {
    asm volatile("red.relaxed.gpu.global.add.noftz.v4.f16x2 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(v.x), "r"(v.y),
                 "r"(v.z), "r"(v.w)
                 : "memory");
  } else if constexpr (kDtype == MSLK_B200_F32) {
    asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(__uint_as_float(v.x)),
                 "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
                 : "memory");
  } else {
    int *d = static_cast<int *>(dst);
    atomicAdd(d + 0, static_cast<int>(v.x));
    atomicAdd(d + 1, static_cast<int>(v.y));
    atomicAdd(d + 2, static_cast<int>(v.z));
    atomicAdd(d + 3, static_cast<int>(v.w));
  }
}

template <int kDtype>
__device__ __forceinline__ void red_add_elem(void *out, const void *in, int64_t o, int64_t i) {
  if constexpr (kDtype == MSLK_B200_BF16)
    atomicAdd(static_cast<__nv_bfloat16 *>(out) + o, static_cast<const __nv_bfloat16 *>(in)[i]);
  else if constexpr (kDtype == MSLK_B200_F16)
    atomicAdd(static_cast<__half *>(out) + o, static_cast<const __half *>(in)[i]);
  else if constexpr (kDtype == MSLK_B200_F32)
    atomicAdd(static_cast<float *>(out) + o, static_cast<const float *>(in)[i]);
  else
    atomicAdd(static_cast<int *>(out) + o, static_cast<const int *>(in)[i]);
}

template <int kDtype>
constexpr int elem_bytes() {
  return (kDtype == MSLK_B200_BF16 || kDtype == MSLK_B200_F16) ? 2 : 4;
}

// One 16-byte piece per thread and step, grid-stride over (input row, piece).  kPadded: the input row
// of stacked row i lives in plane rank(i) of in[EP, rows, D]; the stacked row count is the sum of the
// per-expert counts read from the device.
template <int kDtype, bool kVec, bool kPadded>
__global__ void __launch_bounds__(256) scatter_add_kernel(const ScatterParams p) {
  __shared__ int64_t s_end[kPadded ? 1025 : 1];   // inclusive prefix of the expert counts
  int64_t rows = p.rows;
  if (kPadded) {
    if (threadIdx.x < 32) {   // warp 0: inclusive prefix of the counts, 32 experts per step
      const int lane = threadIdx.x;
      int64_t carry = 0;
      for (int base = 0; base < p.E; base += 32) {
        const int e = base + lane;
        int64_t n = e < p.E ? load_index(p.token_counts, p.count_bits, e) : 0;
        if (n < 0) n = 0;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int64_t up = __shfl_up_sync(0xffffffffu, n, o);
          if (lane >= o) n += up;
        }
        if (e < p.E) s_end[e] = carry + n;
        carry += __shfl_sync(0xffffffffu, n, 31);
      }
      if (lane == 0) s_end[p.E] = carry;
    }
    __syncthreads();
    rows = min(rows, s_end[p.E]);
  } else if (p.valid_token_count) {
    rows = min(rows, static_cast<int64_t>(*p.valid_token_count));
  }
  constexpr int kPer = kVec ? 16 / elem_bytes<kDtype>() : 1;
  const int64_t per_row = p.D / kPer, total = rows * per_row;
  const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int experts_per_rank = kPadded ? static_cast<int>(p.E / p.EP) : 1;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += step) {
    const int64_t row = i / per_row, v = i - row * per_row;
    const int64_t to = load_index(p.token_indices, p.token_bits, row);
    if (to < 0 || to >= p.T) {
      atomicOr(p.status, kStatusBadScatterIndex);
      continue;
    }
    int64_t src_row = row;
    if (kPadded) {
      int lo = 0, hi = static_cast<int>(p.E) - 1;   // first expert whose prefix end exceeds row
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (s_end[mid] > row) hi = mid; else lo = mid + 1;
      }
      src_row = static_cast<int64_t>(lo / experts_per_rank) * p.rows + row;
    }
    if (kVec) {
      const char *src = static_cast<const char *>(p.in) + (src_row * p.D) * elem_bytes<kDtype>() + v * 16;
      char *dst = static_cast<char *>(p.out) + (to * p.D) * elem_bytes<kDtype>() + v * 16;
      red_add_16B<kDtype>(dst, ld_stream_v4(src));
    } else {
      red_add_elem<kDtype>(p.out, p.in, to * p.D + v, src_row * p.D + v);
    }
  }
}

template <typename T>
int launch_gather(const GatherParams &p, bool quant, bool vec_ok, cudaStream_t st) {
  const unsigned rows = static_cast<unsigned>(p.a);
  const int64_t nvec = p.D / 8;
  if (!quant) {
    int threads = static_cast<int>(std::min<int64_t>(1024, std::max<int64_t>(32, ((vec_ok ? (nvec + 1) / 2 : p.D) + 31) / 32 * 32)));
    if (vec_ok)
      gather_scale_kernel<T, true><<<rows, threads, 0, st>>>(p);
    else
      gather_scale_kernel<T, false><<<rows, threads, 0, st>>>(p);
  } else if (vec_ok && nvec <= 4 * 1024) {
    auto go = [&](auto kv) {
      constexpr int kVecs = decltype(kv)::value;
      const int threads = static_cast<int>((nvec + kVecs - 1) / kVecs + 31) / 32 * 32;
      if (threads <= 512)
        gather_scale_quant_vec_kernel<T, kVecs, 512><<<rows, threads, 0, st>>>(p);
      else
        gather_scale_quant_vec_kernel<T, kVecs, 1024><<<rows, threads, 0, st>>>(p);
    };
    if (nvec >= 4 * 128) go(std::integral_constant<int, 4>{});
    else if (nvec >= 2 * 64) go(std::integral_constant<int, 2>{});
    else go(std::integral_constant<int, 1>{});
  } else {
    gather_scale_quant_generic_kernel<T><<<rows, 256, 0, st>>>(p);
  }
  return check_cuda(cudaGetLastError(), "gather_scale launch");
}

int run_gather(bool quant, const void *x, int dtype, int64_t T, int64_t D, const void *token_indices, int token_bits,
               const void *expert_indices, int expert_bits, const void *scores, int scores_dtype, int64_t E,
               int64_t stride_t, int64_t stride_e, int64_t a, const float *scale_ub, const int *valid_token_count,
               void *out, float *inv_scale, cudaStream_t st, const char *name) {
  if (T < 0 || D < 0 || a < 0 || E < 0) return fail(1, "%s: bad shape", name);
  if (a == 0 || D == 0) return 0;
  if (a > 0x7fffffffLL) return fail(1, "%s: too many rows", name);
  if (!x || !token_indices || !expert_indices || !scores || !out || (quant && !inv_scale))
    return fail(1, "%s: null pointer argument", name);
  if (dtype != MSLK_B200_BF16 && dtype != MSLK_B200_F16) return fail(1, "%s: x must be bf16 or fp16", name);
  if (scores_dtype < 0 || scores_dtype > 2) return fail(1, "%s: bad scores dtype", name);
  if ((token_bits != 32 && token_bits != 64) || (expert_bits != 32 && expert_bits != 64))
    return fail(1, "%s: indices must be int32 or int64", name);
  int *status = device_status_ptr();
  if (!status) return 2;
  GatherParams p{x, token_indices, expert_indices, scores, scale_ub, valid_token_count, out, inv_scale,
                 T, D, a, E, stride_t, stride_e, token_bits, expert_bits, scores_dtype, status};
  const bool vec_ok = D % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0 &&
                      (reinterpret_cast<uintptr_t>(out) & (quant ? 7u : 15u)) == 0;
  return dtype == MSLK_B200_BF16 ? launch_gather<__nv_bfloat16>(p, quant, vec_ok, st)
                                 : launch_gather<__half>(p, quant, vec_ok, st);
}

template <bool kPadded>
int run_scatter(const ScatterParams &p, int dtype, cudaStream_t st, const char *name) {
  const int eb = (dtype == MSLK_B200_BF16 || dtype == MSLK_B200_F16) ? 2 : 4;
  const bool vec_ok = (p.D * eb) % 16 == 0 && ((reinterpret_cast<uintptr_t>(p.in) | reinterpret_cast<uintptr_t>(p.out)) & 15u) == 0;
  const int64_t work = p.rows * (vec_ok ? p.D * eb / 16 : p.D);
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  const unsigned blocks = static_cast<unsigned>(std::max<int64_t>(1, std::min<int64_t>((work + 255) / 256, cap)));
#define MSLK_LAUNCH(DT)                                                     \
  if (vec_ok)                                                               \
    scatter_add_kernel<DT, true, kPadded><<<blocks, 256, 0, st>>>(p);       \
  else                                                                      \
    scatter_add_kernel<DT, false, kPadded><<<blocks, 256, 0, st>>>(p);
  switch (dtype) {
    case MSLK_B200_BF16: MSLK_LAUNCH(MSLK_B200_BF16) break;
    case MSLK_B200_F16: MSLK_LAUNCH(MSLK_B200_F16) break;
    case MSLK_B200_F32: MSLK_LAUNCH(MSLK_B200_F32) break;
    case kI32: MSLK_LAUNCH(kI32) break;
    default: return fail(1, "%s: unsupported dtype code %d", name, dtype);
  }
#undef MSLK_LAUNCH
  return check_cuda(cudaGetLastError(), "scatter_add launch");
}

}  // namespace
}  // namespace mslk_b200

MSLK_API int mslk_b200_gather_scale_dense_tokens(const void *x, int dtype, int64_t T, int64_t D,
                                                 const void *token_indices, int token_index_bits,
                                                 const void *expert_indices, int expert_index_bits, const void *scores,
                                                 int scores_dtype, int64_t E, int64_t stride_t, int64_t stride_e,
                                                 int64_t a, const int *valid_token_count, void *out, void *stream) {
  using namespace mslk_b200;
  clear_error();
  return run_gather(false, x, dtype, T, D, token_indices, token_index_bits, expert_indices, expert_index_bits, scores,
                    scores_dtype, E, stride_t, stride_e, a, nullptr, valid_token_count, out, nullptr,
                    static_cast<cudaStream_t>(stream), "gather_scale_dense_tokens");
}

MSLK_API int mslk_b200_gather_scale_quant_dense_tokens(const void *x, int dtype, int64_t T, int64_t D,
                                                       const void *token_indices, int token_index_bits,
                                                       const void *expert_indices, int expert_index_bits,
                                                       const void *scores, int scores_dtype, int64_t E,
                                                       int64_t stride_t, int64_t stride_e, int64_t a,
                                                       const float *scale_ub, const int *valid_token_count, void *q,
                                                       float *inv_scale, void *stream) {
  using namespace mslk_b200;
  clear_error();
  return run_gather(true, x, dtype, T, D, token_indices, token_index_bits, expert_indices, expert_index_bits, scores,
                    scores_dtype, E, stride_t, stride_e, a, scale_ub, valid_token_count, q, inv_scale,
                    static_cast<cudaStream_t>(stream), "gather_scale_quant_dense_tokens");
}

MSLK_API int mslk_b200_scatter_add_dense_tokens(void *out_tokens, int64_t T, const void *in_tokens, int dtype, int64_t a,
                                                int64_t D, const void *token_indices, int token_index_bits,
                                                const int *valid_token_count, void *stream) {
  using namespace mslk_b200;
  clear_error();
  const char *name = "scatter_add_dense_tokens";
  if (T < 0 || a < 0 || D < 0) return fail(1, "%s: bad shape", name);
  if (a == 0 || D == 0) return 0;
  if (!out_tokens || !in_tokens || !token_indices) return fail(1, "%s: null pointer argument", name);
  if (token_index_bits != 32 && token_index_bits != 64) return fail(1, "%s: indices must be int32 or int64", name);
  int *status = device_status_ptr();
  if (!status) return 2;
  ScatterParams p{out_tokens, in_tokens, token_indices, valid_token_count, nullptr, a, D, T, 1, 1, token_index_bits, 32, status};
  return run_scatter<false>(p, dtype, static_cast<cudaStream_t>(stream), name);
}

MSLK_API int mslk_b200_scatter_add_padded_tokens(const void *in_tokens, int dtype, int64_t EP, int64_t T_K, int64_t D,
                                                 const void *token_counts, int count_bits, int64_t E,
                                                 const void *token_indices, int token_index_bits, void *out_tokens,
                                                 int64_t T, void *stream) {
  using namespace mslk_b200;
  clear_error();
  const char *name = "scatter_add_padded_tokens";
  if (EP <= 0 || E <= 0 || T_K < 0 || D < 0 || T < 0) return fail(1, "%s: bad shape", name);
  if (E % EP != 0) return fail(1, "%s: the expert count (%lld) must be a multiple of the rank count (%lld)", name,
                               (long long)E, (long long)EP);
  if (E > 1024) return fail(1, "%s: at most 1024 experts are supported", name);
  if (T_K == 0 || D == 0) return 0;
  if (!out_tokens || !in_tokens || !token_indices || !token_counts) return fail(1, "%s: null pointer argument", name);
  if ((token_index_bits != 32 && token_index_bits != 64) || (count_bits != 32 && count_bits != 64))
    return fail(1, "%s: indices and counts must be int32 or int64", name);
  int *status = device_status_ptr();
  if (!status) return 2;
  ScatterParams p{out_tokens, in_tokens, token_indices, nullptr, token_counts, T_K, D, T, E, EP, token_index_bits, count_bits, status};
  return run_scatter<true>(p, dtype, static_cast<cudaStream_t>(stream), name);
}
