/*
 * CPU oracle for the low-precision GEMM hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain scalar C, the arithmetic of the reference
 * (meta-pytorch/MSLK) for the functions on the hot path so that the CUDA
 * kernels can be checked bit for bit (quantizers) or within tolerance (GEMMs).
 * Nothing in the shipped package links, loads or calls this file; only the
 * test-suite, the smoke check and the CPU-baseline leg of the benchmark do.
 *
 * Each function names the reference file:line whose arithmetic it follows.
 * All float arithmetic is IEEE binary32 with round-to-nearest-even and no
 * contraction (compile with -ffp-contract=off, never -ffast-math).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------ */
/* scalar format helpers                                                     */
/* ------------------------------------------------------------------------ */

static inline float bits_to_f32(uint32_t b) {
  float f;
  memcpy(&f, &b, 4);
  return f;
}
static inline uint32_t f32_to_bits(float f) {
  uint32_t b;
  memcpy(&b, &f, 4);
  return b;
}

static inline float bf16_to_f32(uint16_t h) { return bits_to_f32((uint32_t)h << 16); }

/* fp32 -> bf16, round to nearest even (what torch .to(bfloat16) and
 * cvt.rn.bf16.f32 both do).  NaN stays NaN. */
ORACLE_API uint16_t oracle_f32_to_bf16(float f) {
  uint32_t b = f32_to_bits(f);
  if ((b & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((b >> 16) | 0x40u);
  uint32_t lsb = (b >> 16) & 1u;
  b += 0x7fffu + lsb;
  return (uint16_t)(b >> 16);
}

static inline float f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  if (exp == 0) {
    if (man == 0) return bits_to_f32(sign);
    float v = ldexpf((float)man, -24);
    return sign ? -v : v;
  }
  if (exp == 31) return bits_to_f32(sign | 0x7f800000u | (man << 13));
  return bits_to_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

/* dtype codes shared with the C-ABI of the product: 0 = fp32, 1 = bf16, 2 = fp16 */
static inline float load_elem(const void *base, int dtype, int64_t idx) {
  switch (dtype) {
    case 0: return ((const float *)base)[idx];
    case 1: return bf16_to_f32(((const uint16_t *)base)[idx]);
    default: return f16_to_f32(((const uint16_t *)base)[idx]);
  }
}

/* fp32 -> float8_e4m3fn, round to nearest even, saturate finite values to
 * +-448 ("satfinite"), NaN -> 0x7f | sign.  This is the conversion the
 * reference's Triton kernels get from `.to(tl.float8e4nv)` on NVIDIA
 * (cvt.rn.satfinite.e4m3x2.f32) and, for |v| <= 448, what
 * torch.Tensor.to(torch.float8_e4m3fn) does on CPU. */
ORACLE_API uint8_t oracle_f32_to_e4m3(float f) {
  uint32_t b = f32_to_bits(f);
  uint8_t sign = (uint8_t)((b >> 24) & 0x80u);
  uint32_t a = b & 0x7fffffffu;
  if (a > 0x7f800000u) return (uint8_t)(sign | 0x7fu); /* NaN */
  float av = bits_to_f32(a);
  if (av >= 448.0f) return (uint8_t)(sign | 0x7eu);    /* saturate (incl. inf) */
  if (av < 0.015625f) {
    /* subnormal target range: multiples of 2^-9; rintf is RNE in the default
     * rounding mode; 8 * 2^-9 = 2^-6 is the first normal and encodes as 0x08. */
    int q = (int)rintf(av * 512.0f);
    return (uint8_t)(sign | (uint8_t)q);
  }
  /* normal: keep 3 mantissa bits, RNE on the 20 dropped bits */
  uint32_t lsb = (a >> 20) & 1u;
  a += 0x7ffffu + lsb;
  uint32_t exp = (a >> 23) - 127u + 7u;
  uint32_t man = (a >> 20) & 7u;
  uint32_t code = (exp << 3) | man;
  if (code > 0x7eu) code = 0x7eu;
  return (uint8_t)(sign | code);
}

ORACLE_API float oracle_e4m3_to_f32(uint8_t c) {
  uint32_t exp = (c >> 3) & 0xfu;
  uint32_t man = c & 7u;
  float v;
  if (exp == 0xf && man == 7) return bits_to_f32(0x7fc00000u);
  if (exp == 0) v = ldexpf((float)man, -9);
  else v = ldexpf((float)(8 + man), (int)exp - 10);
  return (c & 0x80u) ? -v : v;
}

/* fp32 -> e2m1 nibble, round to nearest even, saturate to +-6.
 * (cvt.rn.satfinite.e2m1x2.f32 as issued by the reference at
 * mslk/quantize/triton/fp4_primitives/packing.py:112-133.)
 * Representable magnitudes {0,.5,1,1.5,2,3,4,6}; ties go to the even code. */
ORACLE_API uint8_t oracle_f32_to_e2m1(float f) {
  uint8_t sign = (f32_to_bits(f) >> 28) & 0x8u;
  float a = fabsf(f);
  uint8_t m;
  if (a != a) return 7u;       /* NaN of either sign: +6, what cvt.rn.satfinite.e2m1x2.f32 returns on sm_100a */
  if (a <= 0.25f) m = 0;       /* tie 0.25 -> 0   (code 0 even) */
  else if (a < 0.75f) m = 1;   /* tie 0.75 -> 1.0 (code 2 even) */
  else if (a <= 1.25f) m = 2;  /* tie 1.25 -> 1.0 (code 2 even) */
  else if (a < 1.75f) m = 3;   /* tie 1.75 -> 2.0 (code 4 even) */
  else if (a <= 2.5f) m = 4;   /* tie 2.5  -> 2.0 (code 4 even) */
  else if (a < 3.5f) m = 5;    /* tie 3.5  -> 4.0 (code 6 even) */
  else if (a <= 5.0f) m = 6;   /* tie 5.0  -> 4.0 (code 6 even) */
  else m = 7;
  return (uint8_t)(sign | m);
}

static const float kE2M1[16] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f,
                                -0.f, -.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};

ORACLE_API float oracle_e2m1_to_f32(uint8_t nib) { return kE2M1[nib & 15u]; }

/* ------------------------------------------------------------------------ */
/* per-row FP8 quantize, GPU (Triton) arithmetic                             */
/* mslk/quantize/triton/fp8_quantize.py:104-207                              */
/* ------------------------------------------------------------------------ */
/*
 * x is viewed as a 4-D tensor [B, M, N, K] with element strides sb, sm, sn, sk
 * (fp8_quantize.py:236-241); row index r = (b*M + m)*N + n.  Output q is
 * contiguous [B*M*N, K_out] with K_out >= K (align_rows_to padding, :250-259),
 * scale is [B*M*N].
 *   cur   = scale_ub ? min(max(amax, eps), *scale_ub) : max(amax, eps)   (:141-146)
 *   scale = cur / 448            (IEEE division, tl.div_rn)                (:149)
 *   q     = e4m3(clamp(x / scale, -448, 448))  (IEEE division)             (:152-153)
 * Rows with n >= zero_start_index_M[b*M+m] are treated as all-zero (:123-129).
 */
ORACLE_API void oracle_quantize_fp8_row(const void *x, int dtype, int64_t B, int64_t M,
                                        int64_t N, int64_t K, int64_t K_out, int64_t sb,
                                        int64_t sm, int64_t sn, int64_t sk,
                                        const float *scale_ub,
                                        const int64_t *zero_start_index_M, float eps,
                                        uint8_t *q, float *scale) {
  int64_t rows = B * M * N;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    int64_t b = r / (M * N), m = (r % (M * N)) / N, n = (r % (M * N)) % N;
    int64_t base = b * sb + m * sm + n * sn;
    int64_t k_in = K;
    if (zero_start_index_M && n >= zero_start_index_M[b * M + m]) k_in = 0;
    float amax = 0.f;
    for (int64_t k = 0; k < k_in; ++k) {
      float v = fabsf(load_elem(x, dtype, base + k * sk));
      if (v > amax) amax = v;
    }
    float cur = amax > eps ? amax : eps;
    if (scale_ub && cur > *scale_ub) cur = *scale_ub;
    volatile float s = cur / 448.0f;
    scale[r] = s;
    uint8_t *qr = q + r * K_out;
    for (int64_t k = 0; k < K_out; ++k) {
      float v = k < k_in ? load_elem(x, dtype, base + k * sk) : 0.f;
      volatile float t = v / s;
      float c = t;
      if (c > 448.f) c = 448.f;
      if (c < -448.f) c = -448.f;
      qr[k] = oracle_f32_to_e4m3(c);
    }
  }
}

/* ------------------------------------------------------------------------ */
/* per-row FP8 quantize, the reference's CPU (torch) arithmetic              */
/* mslk/quantize/triton/fp8_quantize.py:356-378                              */
/* ------------------------------------------------------------------------ */
/*
 * Contiguous [rows, K] bf16 input only (what the reference's CPU path is used
 * for here: the timed CPU baseline and the fixtures it generates).
 *   row_max = clamp(max|a| , min=eps[, max=ub])   computed in bf16   (:363-369)
 *   a_scale = 448 / float(row_max); inf -> 1                         (:371-372)
 *             (torch evaluates `scalar / tensor` as reciprocal(tensor) * scalar,
 *              so this is RN(RN(1/row_max) * 448), not one division)
 *   q       = e4m3(float(a) * a_scale)                               (:373-375)
 *   returns 1 / a_scale                                              (:378)
 * eps = 1e-12 (mslk/utils/triton/fp8_utils.py:37-40), rounded to bf16 by the
 * clamp on a bf16 tensor.
 */
ORACLE_API void oracle_quantize_fp8_row_cpu_path(const uint16_t *x_bf16, int64_t rows,
                                                 int64_t K, const float *scale_ub,
                                                 uint8_t *q, float *scale_out) {
  const float eps_bf16 = bf16_to_f32(oracle_f32_to_bf16(1e-12f));
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const uint16_t *xr = x_bf16 + r * K;
    float amax = 0.f;
    for (int64_t k = 0; k < K; ++k) {
      float v = fabsf(bf16_to_f32(xr[k]));
      if (v > amax) amax = v;
    }
    if (amax < eps_bf16) amax = eps_bf16;
    if (scale_ub) {
      float ub = bf16_to_f32(oracle_f32_to_bf16(*scale_ub));
      if (amax > ub) amax = ub;
    }
    volatile float rcp = 1.0f / amax;
    volatile float a_scale = rcp * 448.0f;
    if (isinf(a_scale)) a_scale = 1.0f;
    for (int64_t k = 0; k < K; ++k) {
      volatile float t = bf16_to_f32(xr[k]) * a_scale;
      /* torch's CPU cast does not saturate: anything that rounds past 448
       * (|t| > 464) becomes the NaN code, and the CPU path has no clamp. */
      uint8_t c = oracle_f32_to_e4m3(t);
      if (fabsf(t) > 464.0f) c = (uint8_t)((c & 0x80u) | 0x7fu);
      q[r * K + k] = c;
    }
    volatile float inv = 1.0f / a_scale;
    scale_out[r] = inv;
  }
}

/* ------------------------------------------------------------------------ */
/* rowwise-scaled FP8 GEMM                                                   */
/* ------------------------------------------------------------------------ */
/*
 * y[m,n] = bf16( (xs[m] * acc) * ws[n] (+ bias[n]) ),  acc = sum_k xq*wq in fp32.
 * Epilogue order follows the reference's EVT wiring
 * (csrc/gemm/cutlass/f8f8bf16_rowwise/f8f8bf16_rowwise_common.cuh:173-198,293-312):
 * fp32 bias is added in fp32; a bf16 bias makes the scaled product round to bf16
 * first and the add happen in bf16.  bias_kind: 0 none, 1 fp32, 2 bf16.
 * The accumulation order of the reference is unspecified; this one sums k
 * ascending in fp32 (the test oracle formula
 * test/gemm/triton/grouped_gemm_test.py:124-129 is a float matmul).
 */
ORACLE_API void oracle_gemm_f8_rowwise(const uint8_t *xq, const uint8_t *wq,
                                       const float *xs, const float *ws, const void *bias,
                                       int bias_kind, int64_t M, int64_t N, int64_t K,
                                       uint16_t *y_bf16) {
  float lut[256];
  for (int i = 0; i < 256; ++i) lut[i] = oracle_e4m3_to_f32((uint8_t)i);
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m) {
    float *xrow = (float *)malloc(sizeof(float) * (size_t)(K > 0 ? K : 1));
    for (int64_t k = 0; k < K; ++k) xrow[k] = lut[xq[m * K + k]];
    for (int64_t n = 0; n < N; ++n) {
      const uint8_t *wr = wq + n * K;
      float acc = 0.f;
      for (int64_t k = 0; k < K; ++k) acc += xrow[k] * lut[wr[k]];
      volatile float t0 = xs[m] * acc;
      volatile float t1 = t0 * ws[n];
      uint16_t out;
      if (bias_kind == 1) {
        volatile float t2 = t1 + ((const float *)bias)[n];
        out = oracle_f32_to_bf16(t2);
      } else if (bias_kind == 2) {
        float p = bf16_to_f32(oracle_f32_to_bf16(t1));
        volatile float t2 = p + bf16_to_f32(((const uint16_t *)bias)[n]);
        out = oracle_f32_to_bf16(t2);
      } else {
        out = oracle_f32_to_bf16(t1);
      }
      y_bf16[m * N + n] = out;
    }
    free(xrow);
  }
}

/* Stacked grouped variant: group g owns rows [off_g, off_g + M_sizes[g]) of xq / y
 * and weight slab wq[g] ([N,K]) with scales ws[g*N + n]; no bias
 * (csrc/gemm/cutlass/f8f8bf16_rowwise_grouped.cu:342-368,
 *  f8f8bf16_rowwise_grouped_sm100/f8f8bf16_rowwise_grouped_common.cuh:148-213,310-328). */
ORACLE_API void oracle_gemm_f8_rowwise_grouped_stacked(const uint8_t *xq, const uint8_t *wq,
                                                       const float *xs, const float *ws,
                                                       const int64_t *M_sizes, int64_t G,
                                                       int64_t N, int64_t K,
                                                       uint16_t *y_bf16) {
  int64_t off = 0;
  for (int64_t g = 0; g < G; ++g) {
    int64_t Mg = M_sizes[g];
    if (Mg > 0)
      oracle_gemm_f8_rowwise(xq + off * K, wq + g * N * K, xs + off, ws + g * N, 0, 0, Mg, N,
                             K, y_bf16 + off * N);
    off += Mg;
  }
}

/* ------------------------------------------------------------------------ */
/* NVFP4                                                                     */
/* ------------------------------------------------------------------------ */

/* byte offset of scale (row r, col c) in the 128x4-tile swizzled layout:
 * tiles of 512 bytes ordered row-block major then col-block; inside a tile
 * (r%32)*16 + (r%128/32)*4 + c%4
 * (mslk/quantize/triton/fp4_primitives/layout.py:21-60,
 *  mslk/quantize/triton/legacy/primitives.py:51-86). */
ORACLE_API int64_t oracle_nvfp4_scale_offset(int64_t r, int64_t c, int64_t n_col_blocks) {
  int64_t rb = r / 128, cb = c / 4, ri = r % 128, ci = c % 4;
  return (rb * n_col_blocks + cb) * 512 + (ri % 32) * 16 + (ri / 32) * 4 + ci;
}

/*
 * NVFP4 quantize, the reference's Triton arithmetic
 * (mslk/quantize/triton/quantize_kernels/nvfp4.py:213-296, USE_PRECISE_MATH):
 *   s   = e4m3( clamp( (bamax / 6) * gs , 2^-9, 448 ) )      per 16 elements
 *   x^  = e2m1( x * (gs / float(s)) )
 * q: [M, K/2] bytes, element 2j in the low nibble.  scales: swizzled, padded to
 * [ceil(M/128)*128, ceil(K/16/4)*4], padding zero.  gs may be NULL (= 1.0).
 */
ORACLE_API void oracle_quantize_nvfp4_dt(const uint16_t *x16, int dtype, int64_t M, int64_t K,
                                         const float *global_scale, uint8_t *q,
                                         uint8_t *scales_swizzled) {
  int64_t nblk = K / 16;
  int64_t ncb = (nblk + 3) / 4;
  int64_t nrb = (M + 127) / 128;
  memset(scales_swizzled, 0, (size_t)(nrb * ncb * 512));
  float gs = global_scale ? *global_scale : 1.0f;
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m) {
    for (int64_t j = 0; j < nblk; ++j) {
      const uint16_t *xb = x16 + m * K + j * 16;
      float bamax = 0.f;
      for (int i = 0; i < 16; ++i) {
        float v = fabsf(dtype == 2 ? f16_to_f32(xb[i]) : bf16_to_f32(xb[i]));
        if (v > bamax) bamax = v;
      }
      volatile float d = bamax / 6.0f;
      volatile float s = d * gs;
      float sc = s;
      if (sc < 0.001953125f) sc = 0.001953125f;
      if (sc > 448.f) sc = 448.f;
      uint8_t s8 = oracle_f32_to_e4m3(sc);
      scales_swizzled[oracle_nvfp4_scale_offset(m, j, ncb)] = s8;
      volatile float total = gs / oracle_e4m3_to_f32(s8);
      for (int i = 0; i < 16; i += 2) {
        volatile float a = (dtype == 2 ? f16_to_f32(xb[i]) : bf16_to_f32(xb[i])) * total;
        volatile float b = (dtype == 2 ? f16_to_f32(xb[i + 1]) : bf16_to_f32(xb[i + 1])) * total;
        q[m * (K / 2) + j * 8 + i / 2] =
            (uint8_t)(oracle_f32_to_e2m1(a) | (oracle_f32_to_e2m1(b) << 4));
      }
    }
  }
}

/*
 * MXFP4 quantize, the reference's arithmetic (mslk/quantize/triton/quantize_kernels/mx4.py:118-214 with
 * fp4_primitives/scale.py:96-265): per group of `group` elements (32 or 16)
 *   e     = ((bits(max|x|) + round_add) & 0x7F800000) >> 23) - 127 - 2, clamped to [-127, 125]
 *           round_add = 0 (floor), 2^21 - 1 (even), 2^23 - 1 (ceil); round_add < 0: nearest,
 *           e = floor(log2(max|x| or 2^-126 for 0) + 0.5) - 2 (the GPU's log2f may differ from libm's in the last
 *           place, so groups whose maximum sits on a rounding boundary can differ by one binade)
 *   scale = byte e + 127 (e8m0);   x^ = e2m1( x * 2^-e ), the factor built from its exponent bits.
 * x: bf16 (dtype 1) or fp16 (dtype 2).  q: [M, K/2]; scales: swizzled like the NVFP4 scales, padded to
 * [ceil(M/128)*128, ceil(K/group/4)*4], padding zero.
 */
ORACLE_API void oracle_quantize_nvfp4(const uint16_t *x_bf16, int64_t M, int64_t K, const float *global_scale,
                                      uint8_t *q, uint8_t *scales_swizzled) {
  oracle_quantize_nvfp4_dt(x_bf16, 1, M, K, global_scale, q, scales_swizzled);
}

ORACLE_API void oracle_quantize_mx4(const uint16_t *x, int dtype, int64_t M, int64_t K, int group, int round_add,
                                    uint8_t *q, uint8_t *scales_swizzled) {
  int64_t nblk = K / group;
  int64_t ncb = (nblk + 3) / 4;
  int64_t nrb = (M + 127) / 128;
  memset(scales_swizzled, 0, (size_t)(nrb * ncb * 512));
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m) {
    for (int64_t j = 0; j < nblk; ++j) {
      const uint16_t *xb = x + m * K + j * group;
      float amax = 0.f;
      for (int i = 0; i < group; ++i) {
        float v = fabsf(dtype == 2 ? f16_to_f32(xb[i]) : bf16_to_f32(xb[i]));
        if (v > amax) amax = v;
      }
      int e;
      if (round_add < 0) e = (int)floorf(log2f(amax == 0.f ? 1.17549435e-38f : amax) + 0.5f) - 2;   /* nearest */
      else e = (int)(((f32_to_bits(amax) + (uint32_t)round_add) & 0x7F800000u) >> 23) - 127 - 2;
      if (e > 125) e = 125;
      if (e < -127) e = -127;
      scales_swizzled[oracle_nvfp4_scale_offset(m, j, ncb)] = (uint8_t)(e + 127);
      float inv = bits_to_f32((uint32_t)(127 - e) << 23);
      for (int i = 0; i < group; i += 2) {
        volatile float a = (dtype == 2 ? f16_to_f32(xb[i]) : bf16_to_f32(xb[i])) * inv;
        volatile float b = (dtype == 2 ? f16_to_f32(xb[i + 1]) : bf16_to_f32(xb[i + 1])) * inv;
        q[m * (K / 2) + (j * group + i) / 2] = (uint8_t)(oracle_f32_to_e2m1(a) | (oracle_f32_to_e2m1(b) << 4));
      }
    }
  }
}

/*
 * Philox-4x32 with 7 rounds (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", 2011), the generator behind
 * the reference's tl.randint(seed, offset, n_rounds=7) for 32-bit offsets: key = (seed low word, seed high word),
 * counter = (offset, 0, 0, 0), result = first word of the output block.
 */
ORACLE_API uint32_t oracle_philox7_first_word(uint64_t seed, uint32_t offset) {
  const uint32_t MA = 0xD2511F53u, MB = 0xCD9E8D57u;
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32), c0 = offset, c1 = 0, c2 = 0, c3 = 0;
  for (int r = 0; r < 7; ++r) {
    uint64_t pa = (uint64_t)MA * c0, pb = (uint64_t)MB * c2;
    uint32_t n0 = (uint32_t)(pb >> 32) ^ c1 ^ k0, n2 = (uint32_t)(pa >> 32) ^ c3 ^ k1;
    c1 = (uint32_t)pb;
    c3 = (uint32_t)pa;
    c0 = n0;
    c2 = n2;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return c0;
}

/*
 * MXFP4 quantize with stochastic rounding (rounding mode 3; mslk/quantize/triton/fp4_primitives/scale.py:141-143 and
 * 213-261): as oracle_quantize_mx4 with
 *   e        from bits(max|x|) + (philox(seed, row * (K / group) + j) & (2^22 - 1))
 *   x * 2^-e perturbed in its bits by (philox(seed ^ 0x5A5A5A5A, row * K + column) & (2^22 - 1)) - (2^21 - 1)
 * before the round-to-nearest conversion (a bit pattern that became a NaN saturates to +-6 like the GPU's
 * cvt.rn.satfinite does), offsets in wrapping 32-bit arithmetic.  `stream_rows` gives the row index the random streams
 * use for each row of x (the stacked kernel counts rows of the padded scale matrix); NULL = the row itself.
 */
ORACLE_API void oracle_quantize_mx4_stochastic(const uint16_t *x, int dtype, int64_t M, int64_t K, int group,
                                               uint64_t seed, const int32_t *stream_rows, uint8_t *q,
                                               uint8_t *scales_swizzled) {
  int64_t nblk = K / group;
  int64_t ncb = (nblk + 3) / 4;
  int64_t nrb = (M + 127) / 128;
  memset(scales_swizzled, 0, (size_t)(nrb * ncb * 512));
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m) {
    uint32_t srow = stream_rows ? (uint32_t)stream_rows[m] : (uint32_t)m;
    for (int64_t j = 0; j < nblk; ++j) {
      const uint16_t *xb = x + m * K + j * group;
      float amax = 0.f;
      for (int i = 0; i < group; ++i) {
        float v = fabsf(dtype == 2 ? f16_to_f32(xb[i]) : bf16_to_f32(xb[i]));
        if (v > amax) amax = v;
      }
      uint32_t rg = oracle_philox7_first_word(seed, srow * (uint32_t)nblk + (uint32_t)j) & 0x3FFFFFu;
      int e = (int)(((f32_to_bits(amax) + rg) & 0x7F800000u) >> 23) - 127 - 2;
      if (e > 125) e = 125;
      if (e < -127) e = -127;
      scales_swizzled[oracle_nvfp4_scale_offset(m, j, ncb)] = (uint8_t)(e + 127);
      float inv = bits_to_f32((uint32_t)(127 - e) << 23);
      uint8_t nib[2];
      for (int i = 0; i < group; i += 2) {
        for (int h = 0; h < 2; ++h) {
          volatile float a = (dtype == 2 ? f16_to_f32(xb[i + h]) : bf16_to_f32(xb[i + h])) * inv;
          uint32_t re = oracle_philox7_first_word(seed ^ 0x5A5A5A5Aull,
                                                  srow * (uint32_t)K + (uint32_t)(j * group + i + h)) & 0x3FFFFFu;
          nib[h] = oracle_f32_to_e2m1(bits_to_f32(f32_to_bits(a) + re - 0x1FFFFFu));
        }
        q[m * (K / 2) + (j * group + i) / 2] = (uint8_t)(nib[0] | (nib[1] << 4));
      }
    }
  }
}

/*
 * NVFP4 GEMM: y = bf16( alpha * sum_blocks (sx*sw) * sum_16 x^*w^ ), fp32 math,
 * alpha = *global_scale (csrc/gemm/cutlass/f4f4bf16/f4f4bf16_common.cuh:78-315;
 * dequantisation as mslk/quantize/triton/legacy/fp4_utils.py:19-45,95-120).
 */
ORACLE_API void oracle_gemm_nvfp4(const uint8_t *xq, const uint8_t *wq, const uint8_t *sx,
                                  const uint8_t *sw, const float *alpha, int64_t M,
                                  int64_t N, int64_t K, uint16_t *y_bf16) {
  int64_t nblk = K / 16, ncb = (nblk + 3) / 4;
  float a = alpha ? *alpha : 1.0f;
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m) {
    float *xrow = (float *)malloc(sizeof(float) * (size_t)(K > 0 ? K : 1));
    for (int64_t k = 0; k < K; ++k) {
      uint8_t byte = xq[m * (K / 2) + k / 2];
      float s = oracle_e4m3_to_f32(sx[oracle_nvfp4_scale_offset(m, k / 16, ncb)]);
      xrow[k] = kE2M1[(k & 1) ? (byte >> 4) : (byte & 15)] * s;
    }
    for (int64_t n = 0; n < N; ++n) {
      float acc = 0.f;
      for (int64_t j = 0; j < nblk; ++j) {
        float s = oracle_e4m3_to_f32(sw[oracle_nvfp4_scale_offset(n, j, ncb)]);
        float part = 0.f;
        for (int i = 0; i < 16; ++i) {
          int64_t k = j * 16 + i;
          uint8_t byte = wq[n * (K / 2) + k / 2];
          part += xrow[k] * kE2M1[(k & 1) ? (byte >> 4) : (byte & 15)];
        }
        acc += part * s;
      }
      y_bf16[m * N + n] = oracle_f32_to_bf16(acc * a);
    }
    free(xrow);
  }
}

/* ------------------------------------------------------------------------ */
/* self-check used by the CPU tests: x/s computed as q0=x*r, e=fma(-q0,s,x),  */
/* q=fma(e,r,q0) with r=1/s equals IEEE x/s.  Returns the number of           */
/* mismatches over `n` (x, s) pairs.  The CUDA quantizer uses this 3-op form  */
/* instead of a full division; this proves the two agree on the inputs given. */
/* ------------------------------------------------------------------------ */
ORACLE_API int64_t oracle_check_fma_division(const float *x, const float *s, int64_t n) {
  int64_t bad = 0;
  for (int64_t i = 0; i < n; ++i) {
    volatile float r = 1.0f / s[i];
    volatile float q0 = x[i] * r;
    volatile float e = fmaf(-q0, s[i], x[i]);
    volatile float q1 = fmaf(e, r, q0);
    volatile float ref = x[i] / s[i];
    if (f32_to_bits(q1) != f32_to_bits(ref)) {
      /* only mismatches that survive the e4m3 cast matter, but count all */
      ++bad;
    }
  }
  return bad;
}

/* ------------------------------------------------------------------------ */
/* fused SwiGLU + per-row FP8 quantize                                       */
/* mslk/moe/activation.py:220-294 (_mslk_silu_mul_quant), :181-217 (silu_mul) */
/* ------------------------------------------------------------------------ */

/* y = x0 * sigmoid(x0) * x1 in fp32.  The reference's GPU kernel evaluates the
 * sigmoid with the hardware's approximate exp2 and an approximate division, which no
 * CPU can restate bit for bit; this function uses correctly rounded expf and IEEE
 * division instead, so it agrees with the GPU to a few fp32 ulps (the captured GPU
 * fixtures, not this function, pin the exact bits). */
static inline float silu_mul_f32(float x0, float x1) {
  float sig = 1.0f / (1.0f + expf(-x0));
  return (x0 * sig) * x1;
}

ORACLE_API void oracle_silu_mul(const void *x0, const void *x1, int dtype, int64_t T, int64_t D, int64_t stride0,
                                int64_t stride1, int64_t valid, float *y) {
  for (int64_t t = 0; t < T && t < valid; ++t)
    for (int64_t k = 0; k < D; ++k)
      y[t * D + k] = silu_mul_f32(load_elem(x0, dtype, t * stride0 + k), load_elem(x1, dtype, t * stride1 + k));
}

/* Rows >= valid are left untouched.  scale_ub may be NULL.  inv_scale = 1 / (448 / rmax),
 * q = e4m3(y * (448 / rmax)) -- multiplication by the reciprocal scale, as the reference. */
ORACLE_API void oracle_silu_mul_quant(const void *x0, const void *x1, int dtype, int64_t T, int64_t D, int64_t stride0,
                                      int64_t stride1, const float *scale_ub, int64_t valid, uint8_t *q,
                                      float *inv_scale) {
  float *y = (float *)malloc(sizeof(float) * (size_t)(D > 0 ? D : 1));
  for (int64_t t = 0; t < T && t < valid; ++t) {
    float amax = 0.f;
    for (int64_t k = 0; k < D; ++k) {
      y[k] = silu_mul_f32(load_elem(x0, dtype, t * stride0 + k), load_elem(x1, dtype, t * stride1 + k));
      float a = fabsf(y[k]);
      if (a > amax) amax = a;
    }
    float rmax = amax > 1e-12f ? amax : 1e-12f;
    if (scale_ub && rmax > *scale_ub) rmax = *scale_ub;
    float y_scale = 448.0f / rmax;
    inv_scale[t] = 1.0f / y_scale;
    for (int64_t k = 0; k < D; ++k) q[t * D + k] = oracle_f32_to_e4m3(y[k] * y_scale);
  }
  free(y);
}

/* ------------------------------------------------------------------------ */
/* MoE token gather / scatter (mslk/moe/gather_scatter.py)                    */
/* ------------------------------------------------------------------------ */

static inline int64_t load_index(const void *p, int bits, int64_t i) {
  return bits == 64 ? ((const int64_t *)p)[i] : (int64_t)((const int32_t *)p)[i];
}

/* :431-486  out[i] = bf16(f32(x[tok[i]]) * f32(scores[tok[i], exp[i]])); x and out are bf16.  Exact. */
ORACLE_API void oracle_gather_scale_bf16(const uint16_t *x, int64_t D, const void *tok, int tok_bits, const void *exp_,
                                         int exp_bits, const void *scores, int scores_dtype, int64_t stride_t,
                                         int64_t stride_e, int64_t a, int64_t valid, uint16_t *out) {
  for (int64_t i = 0; i < a && i < valid; ++i) {
    int64_t ti = load_index(tok, tok_bits, i), ei = load_index(exp_, exp_bits, i);
    float score = load_elem(scores, scores_dtype, ti * stride_t + ei * stride_e);
    for (int64_t k = 0; k < D; ++k) out[i * D + k] = oracle_f32_to_bf16(bf16_to_f32(x[ti * D + k]) * score);
  }
}

/* :537-655  the same product quantized per row: os = 448 / rmax, inv_scale = 1 / os, q = e4m3(v * os).
 * The GPU kernels use an approximate division for the two quotients; IEEE division here, so the
 * scale agrees to a few ulps and single bytes may differ by one code at rounding boundaries. */
ORACLE_API void oracle_gather_scale_quant_bf16(const uint16_t *x, int64_t D, const void *tok, int tok_bits,
                                               const void *exp_, int exp_bits, const void *scores, int scores_dtype,
                                               int64_t stride_t, int64_t stride_e, int64_t a, int64_t valid,
                                               const float *scale_ub, uint8_t *q, float *inv_scale) {
  for (int64_t i = 0; i < a && i < valid; ++i) {
    int64_t ti = load_index(tok, tok_bits, i), ei = load_index(exp_, exp_bits, i);
    float score = load_elem(scores, scores_dtype, ti * stride_t + ei * stride_e);
    float amax = 0.f;
    for (int64_t k = 0; k < D; ++k) {
      float v = fabsf(bf16_to_f32(x[ti * D + k]) * score);
      if (v > amax) amax = v;
    }
    float rmax = amax > 1e-12f ? amax : 1e-12f;
    if (scale_ub && rmax > *scale_ub) rmax = *scale_ub;
    float os = 448.0f / rmax;
    inv_scale[i] = 1.0f / os;
    for (int64_t k = 0; k < D; ++k) q[i * D + k] = oracle_f32_to_e4m3((bf16_to_f32(x[ti * D + k]) * score) * os);
  }
}

/* :489-526 / :677-740  out[tok[i]] += in[src_plane(i), i], one rounding per add, rows applied in order
 * (one of the orders the reference's atomics may take).  dtype: 0 fp32, 1 bf16, 3 int32.
 * counts == NULL: dense variant (plane 0, rows = min(a, valid)).  Otherwise the stacked row count is
 * sum(counts) and the plane of row i is (expert owning i) / (E / EP). */
ORACLE_API void oracle_scatter_add(void *out, const void *in, int dtype, int64_t rows, int64_t D, const void *tok,
                                   int tok_bits, int64_t valid, const void *counts, int count_bits, int64_t E,
                                   int64_t EP) {
  int64_t n = rows < valid ? rows : valid;
  int64_t total = 0;
  if (counts) {
    for (int64_t e = 0; e < E; ++e) total += load_index(counts, count_bits, e);
    n = rows < total ? rows : total;
  }
  int64_t e = 0, end = counts ? load_index(counts, count_bits, 0) : 0;
  for (int64_t i = 0; i < n; ++i) {
    int64_t plane = 0;
    if (counts) {
      while (i >= end) end += load_index(counts, count_bits, ++e);
      plane = e / (E / EP);
    }
    int64_t to = load_index(tok, tok_bits, i);
    for (int64_t k = 0; k < D; ++k) {
      int64_t s = (plane * rows + i) * D + k, d = to * D + k;
      if (dtype == 0) ((float *)out)[d] += ((const float *)in)[s];
      else if (dtype == 1)
        ((uint16_t *)out)[d] = oracle_f32_to_bf16(bf16_to_f32(((uint16_t *)out)[d]) + bf16_to_f32(((const uint16_t *)in)[s]));
      else ((int32_t *)out)[d] += ((const int32_t *)in)[s];
    }
  }
}
