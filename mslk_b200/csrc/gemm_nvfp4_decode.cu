// NVFP4 GEMM for few tokens (decode shapes, 1 <= M <= 128): weight streaming, HBM-bound.
//
// Same plan as the few-token FP8 kernel (gemm_f8_rowwise_decode.cu).  The operands are
// swapped with respect to gemm_nvfp4.cu: the 128 accumulator rows (UMMA M) run over WEIGHT
// rows n, the accumulator columns (UMMA N = BT, the token count padded to 16/32/64/128) over
// tokens m.  A pipeline stage (256 K-elements) holds 16 KB of packed weights, 2 KB of weight
// scales (four 512-byte atoms of 128 rows x 4 scales), BT x 128 bytes of activations and the
// 2 KB of activation scale atoms, so the shared-memory ring is almost entirely weight bytes
// in flight; two CTAs share an SM.
//
// One CTA computes one (128 weight rows) x (K range) tile.  With fewer row blocks than CTA
// slots the K dimension is split over `splits` CTAs: every CTA stores its fp32 partial tile
// to scratch memory and draws a per-(tile, warp) ticket (atomicInc wraps to zero after the
// last ticket: the counters are zeroed once per call on the stream); the warp that draws the
// last ticket sums the partials in split order — the result does not depend on which CTA
// finishes last — and writes y = bf16(alpha * sum).
// Scratch layout: [n_tile][split][BT tokens][128 weight rows] fp32, then tickets [n_tile][4] u32.
//
// Scale factors: an atom copied to tensor memory with tcgen05.cp (32x128b, replicated to the
// four quadrants) occupies 4 columns, row i + 32 j of the atom in lane i of column j.  For the
// weight side (UMMA M = 128) all four columns are read; for the token side (UMMA N = BT) the
// first BT / 32 columns (rows 0..BT-1).  Two column sets alternate between K blocks.
//
// Roles: warp 0 TMA producer, warp 1 MMA issuer / TMEM owner, warps 2..5 epilogue
// (thread = weight row).  All pipeline waits are bounded (common.cuh).
#include "gemm_nvfp4_decode.h"

#include "common.cuh"

#include <atomic>
#include <algorithm>
#include <cstdlib>

namespace mslk_b200 {
namespace nvfp4_decode {
namespace {

constexpr int kWRows = 128;          // weight rows per tile (UMMA M)
constexpr int kBKBytes = 128;        // bytes of packed K per stage row (256 elements)
constexpr int kMmaKBytes = 32;       // 64 K-elements per instruction
constexpr int kAtomBytes = 512;      // 128 rows x 4 scales
constexpr int kNumThreads = 192;

template <int BT>
struct DCfg {
  static constexpr int kStageW = kWRows * kBKBytes;
  static constexpr int kStageX = BT * kBKBytes;
  static constexpr int kStageSF = 4 * kAtomBytes;              // per operand
  static constexpr int kStageBytes = kStageW + kStageX + 2 * kStageSF;
  // two CTAs per SM: keep each below ~112 KB
  static constexpr int kStages = BT <= 16 ? 5 : BT == 32 ? 4 : 3;
  static constexpr int kAccCols = BT < 32 ? 32 : BT;
  static constexpr int kSfCols = 32;                           // one set: 16 columns weight scales + 16 columns token scales
  static constexpr int kTmemCols = BT <= 64 ? 128 : 256;       // accumulator + two scale sets, rounded to a power of two
  static_assert(kAccCols + 2 * kSfCols <= kTmemCols, "tensor memory budget");
  // block-scaled instruction descriptor: e2m1 x e2m1, ue4m3 scales, K-major, M = 128, N = BT
  static constexpr uint32_t kIdesc = (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BT >> 3) << 17) |
                                     (static_cast<uint32_t>(kWRows >> 4) << 24);
};

template <int BT>
struct DSmemTail {
  uint64_t full[DCfg<BT>::kStages];
  uint64_t empty[DCfg<BT>::kStages];
  uint64_t acc_full;
  uint32_t tmem_base;
  int abort_flag;
};

template <int BT>
constexpr size_t decode_smem_bytes() {
  return 1024 + static_cast<size_t>(DCfg<BT>::kStages) * DCfg<BT>::kStageBytes + sizeof(DSmemTail<BT>);
}

struct KParams {
  const uint8_t *sfx;      // token scale atoms: [1 row block][ncb]
  const uint8_t *sfw;      // weight scale atoms: [ceil(N/128)][ncb]
  const float *alpha;      // device scalar
  __nv_bfloat16 *y;
  float *partials;         // scratch (splits > 1)
  unsigned int *tickets;   // scratch (splits > 1), zero at launch, self-resetting
  int *status;
  int M, N, K;
  int ncb;                 // scale atoms per 128-row block = ceil(K / 64); one scale per 32 elements: ceil(K / 128)
  int scale_mode;          // kScaleNvfp4 / kScaleMxfp4 / kScaleMxfp4_16 (common.cuh); alpha is null for the MX formats
  int x_box_rows;          // rows of the token box (M rounded up to 8): no out-of-range fill
  int splits;
  int kb_per_split;        // K blocks (of 256 elements) per split
  int cluster_reduce;      // 1: the `splits` CTAs of a tile form one thread-block cluster and meet in shared memory
};

template <int BT>
__global__ void __launch_bounds__(kNumThreads, 2)
    gemm_nvfp4_decode_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                             const KParams p) {
  using C = DCfg<BT>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *ring = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  DSmemTail<BT> &S = *reinterpret_cast<DSmemTail<BT> *>(ring + static_cast<size_t>(C::kStages) * C::kStageBytes);

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  const int n_tile = blockIdx.x;
  const int split = blockIdx.y;
  const int k_blocks_total = (p.K / 2 + kBKBytes - 1) / kBKBytes;
  const int kb0 = split * p.kb_per_split;
  const int kb1 = min(k_blocks_total, kb0 + p.kb_per_split);
  const int my_kb = max(0, kb1 - kb0);
  volatile int *abort_flag = &S.abort_flag;

  if (threadIdx.x == 0) {
    prefetch_tensormap(&tmap_w);
    prefetch_tensormap(&tmap_x);
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&S.full[s], 1);
      mbar_init(&S.empty[s], 1);
    }
    mbar_init(&S.acc_full, 1);
    S.abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  // one stage: 128 weight rows, the token rows and the scale atoms of both for K block kb
  auto issue_stage = [&](int kb, int stage) {
    const uint8_t *sfw_row = p.sfw + static_cast<size_t>(n_tile) * p.ncb * kAtomBytes;
    uint8_t *sw = ring + static_cast<size_t>(stage) * C::kStageBytes;
    uint8_t *sx = sw + C::kStageW;
    uint8_t *ssfw = sx + C::kStageX;
    uint8_t *ssfx = ssfw + C::kStageSF;
    // scale atoms (4 scales per row each: 64 K-elements, MXFP4 128) left in this K block of 256 elements
    const int apk = p.scale_mode == kScaleMxfp4 ? 2 : 4;
    const int atoms = min(apk, p.ncb - apk * kb);
    const uint32_t sf_bytes = static_cast<uint32_t>(atoms) * kAtomBytes;
    mbar_arrive_expect_tx(&S.full[stage], C::kStageW + p.x_box_rows * kBKBytes + 2 * sf_bytes);
    tma_load_2d(sw, &tmap_w, &S.full[stage], kb * kBKBytes, n_tile * kWRows);
    tma_load_2d(sx, &tmap_x, &S.full[stage], kb * kBKBytes, 0);
    bulk_load_1d(ssfw, sfw_row + static_cast<size_t>(apk * kb) * kAtomBytes, sf_bytes, &S.full[stage]);
    bulk_load_1d(ssfx, p.sfx + static_cast<size_t>(apk * kb) * kAtomBytes, sf_bytes, &S.full[stage]);
  };
  // the first stages go out right away: the copies fly while tensor memory is allocated and the warps meet below
  const int pre = min(C::kStages, my_kb);
  if (threadIdx.x == 0)
    for (int i = 0; i < pre; ++i) issue_stage(kb0 + i, i);
  if (warp == 1) {
    tmem_alloc(&S.tmem_base, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = S.tmem_base;

  // state of the epilogue threads (warps 2..5), kept across the cluster barrier below
  const int quad = warp & 3;
  const int n = n_tile * kWRows + quad * 32 + lane;
  const bool n_ok = n < p.N;
  float acc[BT];
  bool do_epilogue = false;

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (elect_one()) {  // one lane, chosen so that the compiler keeps the issue loop on the uniform datapath
      int stage = pre == C::kStages ? 0 : pre;
      uint32_t phase = pre == C::kStages ? 1u : 0u;
      for (int kb = kb0 + pre; kb < kb1; ++kb) {
        if (!mbar_wait(&S.empty[stage], phase ^ 1, abort_flag, p.status, kStatusProducerTimeout)) break;
        issue_stage(kb, stage);
        if (++stage == C::kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {  // one lane, chosen so that the compiler keeps the issue loop on the uniform datapath
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int i = 0; i < my_kb; ++i) {
        if (!mbar_wait(&S.full[stage], phase, abort_flag, p.status, kStatusMmaTimeout)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sw = smem_u32(ring + static_cast<size_t>(stage) * C::kStageBytes);
        const uint32_t ssfw = sw + C::kStageW + C::kStageX;
        const uint32_t ssfx = ssfw + C::kStageSF;
        const uint32_t sfw_t = tmem_base + C::kAccCols + (i & 1) * C::kSfCols;
        const uint32_t sfx_t = sfw_t + 16;
        const uint64_t dw = make_kmajor_sw128_desc(sw);
        const uint64_t dx = make_kmajor_sw128_desc(sw + C::kStageW);
        if (p.scale_mode == kScaleMxfp4) {
          // one scale per 32 K-elements: an atom holds the scales of TWO instructions, which pick their two bytes of
          // the scale column through the scale-id fields of the descriptor
          const int mmas = min(4, (p.K - (kb0 + i) * (2 * kBKBytes) + 63) / 64);
          const int atoms = (mmas + 1) / 2;
          for (int a = 0; a < atoms; ++a) {
            tc_cp_32x128b_warpx4(sfw_t + 4 * a, make_sf_atom_desc(ssfw + a * kAtomBytes));
            tc_cp_32x128b_warpx4(sfx_t + 4 * a, make_sf_atom_desc(ssfx + a * kAtomBytes));
          }
          for (int k = 0; k < mmas; ++k)
            mma_mxf4_2x(tmem_base, dw + static_cast<uint64_t>(k * (kMmaKBytes >> 4)),
                        dx + static_cast<uint64_t>(k * (kMmaKBytes >> 4)),
                        C::kIdesc | kIdescScaleE8M0 | idesc_scale_ids((k & 1) * 2), sfw_t + 4 * (k >> 1),
                        sfx_t + 4 * (k >> 1), (i | k) != 0 ? 1u : 0u);
        } else {
          const uint32_t idesc = C::kIdesc | (p.scale_mode == kScaleMxfp4_16 ? kIdescScaleE8M0 : 0u);
          const int atoms = min(4, p.ncb - 4 * (kb0 + i));
          for (int k = 0; k < atoms; ++k) {
            tc_cp_32x128b_warpx4(sfw_t + 4 * k, make_sf_atom_desc(ssfw + k * kAtomBytes));
            tc_cp_32x128b_warpx4(sfx_t + 4 * k, make_sf_atom_desc(ssfx + k * kAtomBytes));
          }
          for (int k = 0; k < atoms; ++k)
            mma_nvfp4(tmem_base, dw + static_cast<uint64_t>(k * (kMmaKBytes >> 4)),
                      dx + static_cast<uint64_t>(k * (kMmaKBytes >> 4)), idesc, sfw_t + 4 * k, sfx_t + 4 * k,
                      (i | k) != 0 ? 1u : 0u);
        }
        tc_commit(&S.empty[stage]);
        if (++stage == C::kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok) tc_commit(&S.acc_full);
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue: thread = weight row
    bool have = false;
    if (my_kb > 0) {
      const bool got = mbar_wait(&S.acc_full, 0, abort_flag, p.status, kStatusEpilogueTimeout);
      have = __all_sync(0xffffffffu, got);
    }
    if (have) {
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
      if constexpr (BT >= 32) {
#pragma unroll
        for (int c = 0; c < BT / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[c * 32 + j] = __uint_as_float(r[j]);
        }
      } else {
        uint32_t r[32];  // only the first BT columns are meaningful (32 columns are allocated)
        tmem_ld_32x32(taddr, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < BT; ++j) acc[j] = __uint_as_float(r[j]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < BT; ++j) acc[j] = 0.f;
    }
    const bool aborted = (my_kb > 0) && !have;

    do_epilogue = !aborted;
    if (p.cluster_reduce) {
      // Partial tile into this CTA's own shared memory ([token][weight row] fp32 over the ring, whose
      // stages have all been consumed once the accumulator is complete); collected after the barrier below.
      float *red = reinterpret_cast<float *>(ring);
#pragma unroll
      for (int m = 0; m < BT; ++m)
        if (m < p.M) red[m * kWRows + quad * 32 + lane] = acc[m];
    } else if (p.splits > 1 && !aborted) {
      float *mine = p.partials + ((static_cast<size_t>(n_tile) * p.splits + split) * BT) * kWRows + quad * 32 + lane;
#pragma unroll
      for (int m = 0; m < BT; ++m)
        if (m < p.M) mine[static_cast<size_t>(m) * kWRows] = acc[m];
      __threadfence();
      __syncwarp();
      unsigned int ticket = 0;
      if (lane == 0) ticket = atomicInc(p.tickets + n_tile * 4 + quad, static_cast<unsigned int>(p.splits - 1));
      ticket = __shfl_sync(0xffffffffu, ticket, 0);
      do_epilogue = ticket == static_cast<unsigned int>(p.splits - 1);
      if (do_epilogue) {
        __threadfence();
        const float *base = p.partials + (static_cast<size_t>(n_tile) * p.splits * BT) * kWRows + quad * 32 + lane;
#pragma unroll
        for (int m = 0; m < BT; ++m) acc[m] = 0.f;
        for (int s = 0; s < p.splits; ++s) {
          const float *ps = base + static_cast<size_t>(s) * BT * kWRows;
#pragma unroll
          for (int m = 0; m < BT; ++m)
            if (m < p.M) acc[m] += __ldcg(ps + static_cast<size_t>(m) * kWRows);
        }
      }
    }
  }

  if (p.cluster_reduce) {
    // Split K inside a thread-block cluster: every CTA of the cluster (all threads, all roles) meets at
    // the hardware barrier; then CTA r finishes the tokens m = r, r + splits, ...: it adds the partial
    // sums of all CTAs, read from their shared memory in rank order (deterministic), and stores the
    // result.  The second barrier keeps every CTA resident until its peers have read it.  No scratch
    // memory, no tickets, no extra launch.
    cluster_sync_all();
    if (warp >= 2 && do_epilogue && n_ok) {
      const float alpha = p.alpha ? *p.alpha : 1.0f;   // the MX formats have no global scale
      const uint32_t mine = smem_u32(ring) + static_cast<uint32_t>(quad * 32 + lane) * 4u;
      uint32_t peer[8];
#pragma unroll
      for (int s = 0; s < 8; ++s) peer[s] = mapa_u32(mine, static_cast<uint32_t>(s < p.splits ? s : 0));
      for (int m = split; m < p.M; m += p.splits) {
        float part[8];
#pragma unroll
        for (int s = 0; s < 8; ++s)
          part[s] = s < p.splits ? ld_shared_cluster_f32(peer[s] + static_cast<uint32_t>(m * kWRows) * 4u) : 0.f;
        float a = part[0];
#pragma unroll
        for (int s = 1; s < 8; ++s) a += part[s];
        p.y[static_cast<size_t>(m) * p.N + n] = __float2bfloat16_rn(a * alpha);
      }
    }
    cluster_sync_all();
  } else if (warp >= 2 && do_epilogue && n_ok) {
    const float alpha = p.alpha ? *p.alpha : 1.0f;   // the MX formats have no global scale
#pragma unroll
    for (int m = 0; m < BT; ++m)
      if (m < p.M) p.y[static_cast<size_t>(m) * p.N + n] = __float2bfloat16_rn(acc[m] * alpha);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <int BT>
int launch_decode(const CUtensorMap &tw, const CUtensorMap &tx, const KParams &p, int n_tiles, cudaStream_t st) {
  static std::atomic<bool> attr_set[64];   // zero-initialised; two first calls may both set the (idempotent) attribute
  int dev = 0;
  if (int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
  constexpr size_t smem = decode_smem_bytes<BT>();
  static_assert(smem <= 113 * 1024, "two CTAs per SM need at most ~113 KB each");
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (int rc = check_cuda(cudaFuncSetAttribute(gemm_nvfp4_decode_kernel<BT>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)),
                            "cudaFuncSetAttribute(gemm_nvfp4_decode)"))
      return rc;
    attr_set[dev] = true;
  }
  if (p.cluster_reduce) {
    // the splits of one tile (grid y) form a thread-block cluster
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_tiles, p.splits, 1);
    cfg.blockDim = dim3(kNumThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = static_cast<unsigned>(p.splits);
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return check_cuda(cudaLaunchKernelEx(&cfg, gemm_nvfp4_decode_kernel<BT>, tw, tx, p),
                      "f4f4bf16 decode launch (cluster)");
  }
  gemm_nvfp4_decode_kernel<BT><<<dim3(n_tiles, p.splits, 1), kNumThreads, smem, st>>>(tw, tx, p);
  return check_cuda(cudaGetLastError(), "f4f4bf16 decode launch");
}

int token_tile(int64_t M) { return M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128; }

// Number of K splits.  Measured (CUDA graphs, weights rotated through more than the L2 size): a CTA
// costs about as much as ten K blocks before its first instruction issues, and clearing the tickets is a
// launch of its own, so splitting pays only for long K -- M = 64, N = 8192, K = 28672: 53 us unsplit,
// 44 us in two or three splits; K = 8192 never gained (N = 8192: 16.1 us unsplit, 16.6 in four;
// N = 28672: 24 us unsplit, 33 us in two).  Rule: splits of at least 32 K blocks, at most as many
// CTAs as the device holds at two per SM.
int choose_splits(int64_t N, int64_t K, int sms) {
  const int64_t n_tiles = (N + kWRows - 1) / kWRows;
  const int64_t k_blocks = (K / 2 + kBKBytes - 1) / kBKBytes;
  const int64_t slots = 2 * static_cast<int64_t>(sms);
  const int64_t s_max = std::max<int64_t>(1, std::min<int64_t>(32, k_blocks / 2));
  const int64_t s = std::min<int64_t>(k_blocks / 32, slots / n_tiles);
  return static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(s, s_max)));
}

// Cluster size (2, 4 or 8 CTAs along K) for the split that needs no scratch: K is split only when the
// unsplit launch would leave more than half of the SMs without a CTA; then the largest size that still
// fits all CTAs on the device at once (two per SM) and leaves every CTA at least eight K blocks.
int cluster_splits(int64_t N, int64_t K, int sms) {
  const int64_t n_tiles = (N + kWRows - 1) / kWRows;
  const int64_t k_blocks = (K / 2 + kBKBytes - 1) / kBKBytes;
  if (2 * n_tiles > sms) return 1;
  int s = 1;
  while (s < 8 && n_tiles * (2 * s) <= 2 * static_cast<int64_t>(sms) && k_blocks / (2 * s) >= 8) s *= 2;
  return s;
}

}  // namespace

size_t scratch_bytes(int64_t M, int64_t N, int64_t K, int sms) {
  if (M < 1 || M > kMaxTokens) return 0;
  const int splits = choose_splits(N, K, sms);
  if (splits <= 1) return 0;
  const int64_t n_tiles = (N + kWRows - 1) / kWRows;
  const size_t partial = static_cast<size_t>(n_tiles) * splits * token_tile(M) * kWRows * sizeof(float);
  return partial + static_cast<size_t>(n_tiles) * 4 * sizeof(unsigned int);
}

int launch_decode_kernel(const void *xq, const void *wq, const void *x_scale, const void *w_scale, const float *alpha,
                         void *y, int *status, int64_t M, int64_t N, int64_t K, void *scratch, size_t scratch_size,
                         cudaStream_t st, int scale_mode) {
  const int sms = sm_count();
  const int64_t n_tiles = (N + kWRows - 1) / kWRows;
  const int k_blocks = static_cast<int>((K / 2 + kBKBytes - 1) / kBKBytes);
  int splits = choose_splits(N, K, sms);
  const int bt = token_tile(M);
  const size_t partial_bytes = static_cast<size_t>(n_tiles) * splits * bt * kWRows * sizeof(float);
  const size_t ticket_bytes = static_cast<size_t>(n_tiles) * 4 * sizeof(unsigned int);
  // K split inside thread-block clusters (partial tiles meet in shared memory) whenever that applies;
  // the scratch form only for what clusters do not cover (more than eight splits are never chosen).
  bool cluster_reduce = false;
  const int cs = cluster_splits(N, K, sms);
  if (cs > 1 || !scratch || scratch_size < partial_bytes + ticket_bytes) {
    splits = cs;
    cluster_reduce = cs > 1;
  }

  KParams p;
  p.sfx = static_cast<const uint8_t *>(x_scale);
  p.sfw = static_cast<const uint8_t *>(w_scale);
  p.alpha = alpha;
  p.y = static_cast<__nv_bfloat16 *>(y);
  p.status = status;
  p.M = static_cast<int>(M);
  p.N = static_cast<int>(N);
  p.K = static_cast<int>(K);
  p.ncb = static_cast<int>(scale_mode == kScaleMxfp4 ? (K + 127) / 128 : (K + 63) / 64);
  p.scale_mode = scale_mode;
  p.x_box_rows = std::min<int>(bt, static_cast<int>((M + 7) / 8 * 8));
  p.splits = splits;
  p.kb_per_split = (k_blocks + splits - 1) / splits;
  p.cluster_reduce = cluster_reduce ? 1 : 0;
  p.partials = nullptr;
  p.tickets = nullptr;
  if (splits > 1 && !cluster_reduce) {
    p.partials = static_cast<float *>(scratch);
    p.tickets = reinterpret_cast<unsigned int *>(static_cast<uint8_t *>(scratch) + partial_bytes);
    if (int rc = check_cuda(cudaMemsetAsync(p.tickets, 0, ticket_bytes, st), "zero split-K tickets")) return rc;
  }

  CUtensorMap tw, tx;
  if (int rc = make_tmap_2d_bytes(&tw, wq, K / 2, N, K / 2, kBKBytes, kWRows, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  if (int rc = make_tmap_2d_bytes(&tx, xq, K / 2, M, K / 2, kBKBytes, p.x_box_rows, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  switch (bt) {
    case 16: return launch_decode<16>(tw, tx, p, static_cast<int>(n_tiles), st);
    case 32: return launch_decode<32>(tw, tx, p, static_cast<int>(n_tiles), st);
    case 64: return launch_decode<64>(tw, tx, p, static_cast<int>(n_tiles), st);
    default: return launch_decode<128>(tw, tx, p, static_cast<int>(n_tiles), st);
  }
}

}  // namespace nvfp4_decode
}  // namespace mslk_b200
