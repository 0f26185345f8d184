// Rowwise-scaled FP8 GEMM for few tokens (decode shapes): weight streaming, HBM-bound.
//
// Operands are swapped with respect to the large-M kernels: the 128 accumulator
// rows (UMMA M) run over WEIGHT rows n, the accumulator columns (UMMA N = BT, the
// token count padded to 16/32/64/128) over tokens m.  A pipeline stage then holds
// 16 KB of weights and only BT x 128 bytes of activations, so the shared-memory
// ring is almost entirely weight bytes in flight (two CTAs per SM, up to ~100 KB
// each), which is what an HBM-bound kernel needs.
//
// One CTA computes one (128 weight rows) x (K range) tile.  When there are fewer
// 128-row blocks than SMs the K dimension is split over `splits` CTAs:
//   * every CTA stores its fp32 partial tile to scratch memory,
//   * bumps a per-(tile, warp) ticket with atomicInc (which wraps to zero after the
//     last ticket, so the counters need zeroing only once),
//   * the warp that draws the last ticket sums all partials in split order (the
//     result does not depend on which CTA finishes last) and runs the epilogue.
// Scratch layout: [n_tile][split][BT tokens][128 weight rows] fp32, then the
// tickets [n_tile][4] u32.
//
// Roles: warp 0 TMA producer, warp 1 MMA issuer / TMEM owner, warps 2..5 epilogue
// (thread = weight row).  All pipeline waits are bounded (common.cuh).
#include "gemm_f8_common.cuh"

#include <atomic>
#include <algorithm>
#include <cstdlib>
#include <mutex>

namespace mslk_b200 {
namespace gemm_f8 {
namespace {

constexpr int kWRows = 128;  // weight rows per tile (UMMA M)

template <int BT>
struct DCfg {
  static constexpr int kStageW = kWRows * kBK;
  static constexpr int kStageX = BT * kBK;
  static constexpr int kStageBytes = kStageW + kStageX;
  // two CTAs per SM: keep each below ~110 KB
  static constexpr int kStages = BT <= 32 ? 5 : BT == 64 ? 4 : 3;
  static constexpr int kTmemCols = BT < 32 ? 32 : BT;
  static constexpr uint32_t kIdesc =
      (1u << 4) | (static_cast<uint32_t>(BT >> 3) << 17) | (static_cast<uint32_t>(kWRows >> 4) << 24);
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

struct DecodeParams {
  const float *x_scale;
  const float *w_scale;
  const void *bias;
  __nv_bfloat16 *y;
  float *partials;         // scratch (splits > 1)
  unsigned int *tickets;   // scratch (splits > 1), zero before first use, self-resetting
  int *status;
  int bias_kind;
  int M, N, K;
  int splits;
  int kb_per_split;        // K blocks (of 128) per split
  int x_box_rows;          // rows of the token box (M rounded up to 8): absent rows are not zero-filled
  int cluster_reduce;      // 1: the `splits` CTAs of a tile form one thread-block cluster and meet in shared memory
};

template <int BT>
__global__ void __launch_bounds__(kNumThreads, 2)
    gemm_f8_rowwise_decode_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                                  const DecodeParams p) {
  using C = DCfg<BT>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *ring = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  DSmemTail<BT> &S = *reinterpret_cast<DSmemTail<BT> *>(ring + static_cast<size_t>(C::kStages) * C::kStageBytes);

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  const int n_tile = blockIdx.x;
  const int split = blockIdx.y;
  const int k_blocks_total = (p.K + kBK - 1) / kBK;
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
    // the first stages go out right away: the copies fly while tensor memory is allocated and the warps meet below
    for (int kb = kb0; kb < kb0 + min(C::kStages, my_kb); ++kb) {
      const int st = kb - kb0;
      uint8_t *sw = ring + static_cast<size_t>(st) * C::kStageBytes;
      mbar_arrive_expect_tx(&S.full[st], C::kStageW + p.x_box_rows * kBK);
      tma_load_2d(sw, &tmap_w, &S.full[st], kb * kBK, n_tile * kWRows);
      tma_load_2d(sw + C::kStageW, &tmap_x, &S.full[st], kb * kBK, 0);
    }
  }
  const int pre = min(C::kStages, my_kb);   // stages issued above
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
    if (elect_one()) {  // one lane, chosen so that the compiler keeps the issue loop on the uniform datapath
      int stage = pre == C::kStages ? 0 : pre;
      uint32_t phase = pre == C::kStages ? 1u : 0u;
      for (int kb = kb0 + pre; kb < kb1; ++kb) {
        if (!mbar_wait(&S.empty[stage], phase ^ 1, abort_flag, p.status, kStatusProducerTimeout)) break;
        uint8_t *sw = ring + static_cast<size_t>(stage) * C::kStageBytes;
        uint8_t *sx = sw + C::kStageW;
        mbar_arrive_expect_tx(&S.full[stage], C::kStageW + p.x_box_rows * kBK);
        tma_load_2d(sw, &tmap_w, &S.full[stage], kb * kBK, n_tile * kWRows);
        tma_load_2d(sx, &tmap_x, &S.full[stage], kb * kBK, 0);
        if (++stage == C::kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
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
        const uint64_t dw = make_kmajor_sw128_desc(sw);
        const uint64_t dx = make_kmajor_sw128_desc(sw + C::kStageW);
#pragma unroll
        for (int k = 0; k < kBK / kUmmaK; ++k)
          mma_f8f6f4(tmem_base, dw + static_cast<uint64_t>(k * (kUmmaK >> 4)),
                     dx + static_cast<uint64_t>(k * (kUmmaK >> 4)), C::kIdesc, (i | k) != 0 ? 1u : 0u);
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
      // stages have all been consumed once the accumulator is complete); the cluster's first CTA
      // collects them after the barrier below.
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

  // scale, bias and store of one output element (token m, this thread's weight row n)
  float ws = 0.f, bias_f = 0.f;
  if (warp >= 2 && n_ok) {
    ws = p.w_scale[n];
    if (p.bias_kind == MSLK_B200_BIAS_F32) bias_f = static_cast<const float *>(p.bias)[n];
    if (p.bias_kind == MSLK_B200_BIAS_BF16) bias_f = __bfloat162float(static_cast<const __nv_bfloat16 *>(p.bias)[n]);
  }
  auto store_token = [&](int m, float a) {
    float v = (a * p.x_scale[m]) * ws;
    if (p.bias_kind == MSLK_B200_BIAS_F32) v += bias_f;
    if (p.bias_kind == MSLK_B200_BIAS_BF16) v = __bfloat162float(__float2bfloat16_rn(v)) + bias_f;
    p.y[static_cast<size_t>(m) * p.N + n] = __float2bfloat16_rn(v);
  };

  if (p.cluster_reduce) {
    // Split K inside a thread-block cluster: every CTA of the cluster (all threads, all roles) meets at
    // the hardware barrier; then CTA r finishes the tokens m = r, r + splits, ...: it adds the partial
    // sums of all CTAs, read from their shared memory in rank order (deterministic), and stores the
    // result.  The second barrier keeps every CTA resident until its peers have read it.  No scratch
    // memory, no tickets, no extra launch.
    cluster_sync_all();
    if (warp >= 2 && do_epilogue && n_ok) {
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
        store_token(m, a);
      }
    }
  } else if (warp >= 2 && do_epilogue && n_ok) {
#pragma unroll
    for (int m = 0; m < BT; ++m)
      if (m < p.M) store_token(m, acc[m]);
  }
  if (p.cluster_reduce) cluster_sync_all();

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <int BT>
int launch_decode(const CUtensorMap &tw, const CUtensorMap &tx, const DecodeParams &p, int n_tiles, cudaStream_t st) {
  static std::atomic<bool> attr_set[64];   // zero-initialised; two first calls may both set the (idempotent) attribute
  int dev = 0;
  if (int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
  constexpr size_t smem = decode_smem_bytes<BT>();
  static_assert(smem <= 113 * 1024, "two CTAs per SM need at most ~113 KB each");
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (int rc = check_cuda(cudaFuncSetAttribute(gemm_f8_rowwise_decode_kernel<BT>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)),
                            "cudaFuncSetAttribute(gemm_f8_rowwise_decode)"))
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
    return check_cuda(cudaLaunchKernelEx(&cfg, gemm_f8_rowwise_decode_kernel<BT>, tw, tx, p),
                      "f8f8bf16_rowwise decode launch (cluster)");
  }
  gemm_f8_rowwise_decode_kernel<BT><<<dim3(n_tiles, p.splits, 1), kNumThreads, smem, st>>>(tw, tx, p);
  return check_cuda(cudaGetLastError(), "f8f8bf16_rowwise decode launch");
}

}  // namespace

int decode_token_tile(int64_t M) { return M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128; }

// Number of K splits for a decode-shaped problem.  Two CTAs fit on an SM; the launch costs
// waves(s) * (K blocks per split + a fixed per-CTA overhead of about three K blocks), waves(s) =
// ceil(tiles * s / (2 * SMs)): a split count that leaves a mostly empty last wave (e.g. 224 tiles
// x 2 splits on 296 slots) is worse than none.  Each split keeps at least two K blocks.
int decode_splits(int64_t N, int64_t K, int sms) {
  const int64_t n_tiles = (N + kWRows - 1) / kWRows;
  const int64_t k_blocks = (K + kBK - 1) / kBK;
  const int64_t slots = 2 * static_cast<int64_t>(sms);
  const int64_t s_max = std::max<int64_t>(1, std::min<int64_t>(32, k_blocks / 2));
  int64_t best = 1, best_cost = -1;
  for (int64_t s = 1; s <= s_max; ++s) {
    const int64_t waves = (n_tiles * s + slots - 1) / slots;
    const int64_t cost = waves * ((k_blocks + s - 1) / s + 3);
    if (best_cost < 0 || cost < best_cost) {
      best = s;
      best_cost = cost;
    }
  }
  return static_cast<int>(best);
}

// Cluster size (2, 4 or 8 CTAs along K) for the split that needs no scratch.  K is split only when the
// unsplit launch would leave more than half of the SMs without a CTA; then the largest size that still
// fits all CTAs on the device at once (two per SM) and leaves every CTA at least eight K blocks.
// Measured (M = 16, CUDA graphs): (4096, 4096) 7.9 us in clusters of 4 against 10.8 unsplit and 8.8 on the
// general kernel; (4096, 14336) 13.7 (8) against 27.6 / 20.5; (8192, 8192) 15.8 (4) against 19.5 / 23.3;
// (14336, 4096): 112 row blocks, unsplit 14.2 us, clusters of 2 15.7.
int cluster_splits(int64_t N, int64_t K, int sms) {
  const int64_t n_tiles = (N + kWRows - 1) / kWRows;
  const int64_t k_blocks = (K + kBK - 1) / kBK;
  if (2 * n_tiles > sms) return 1;
  int s = 1;
  while (s < 8 && n_tiles * (2 * s) <= 2 * static_cast<int64_t>(sms) && k_blocks / (2 * s) >= 8) s *= 2;
  return s;
}

size_t decode_scratch_bytes(int64_t M, int64_t N, int64_t K, int sms) {
  const int splits = decode_splits(N, K, sms);
  if (splits <= 1) return 0;
  const int64_t n_tiles = (N + kWRows - 1) / kWRows;
  const size_t partial = static_cast<size_t>(n_tiles) * splits * decode_token_tile(M) * kWRows * sizeof(float);
  return partial + static_cast<size_t>(n_tiles) * 4 * sizeof(unsigned int);
}

int launch_decode_kernel(const void *xq, const void *wq, const GemmParams &gp, void *scratch, size_t scratch_bytes,
                         bool scratch_is_clean, cudaStream_t st) {
  const int sms = sm_count();
  const int64_t n_tiles = (static_cast<int64_t>(gp.N) + kWRows - 1) / kWRows;
  const int k_blocks = (gp.K + kBK - 1) / kBK;
  int splits = decode_splits(gp.N, gp.K, sms);
  const int bt = decode_token_tile(gp.total_m);
  const size_t partial_bytes = static_cast<size_t>(n_tiles) * splits * bt * kWRows * sizeof(float);
  const size_t ticket_bytes = static_cast<size_t>(n_tiles) * 4 * sizeof(unsigned int);
  bool cluster_reduce = false;
  if (!scratch || scratch_bytes < partial_bytes + ticket_bytes) {
    // no scratch: K is split inside thread-block clusters, whose CTAs meet in shared memory
    splits = cluster_splits(gp.N, gp.K, sms);
    cluster_reduce = splits > 1;
  }

  DecodeParams p;
  p.x_scale = gp.x_scale;
  p.w_scale = gp.w_scale;
  p.bias = gp.bias;
  p.y = gp.y;
  p.status = gp.status;
  p.bias_kind = gp.bias_kind;
  p.M = gp.total_m;
  p.N = gp.N;
  p.K = gp.K;
  p.splits = splits;
  p.kb_per_split = (k_blocks + splits - 1) / splits;
  p.x_box_rows = std::min<int>(bt, (gp.total_m + 7) / 8 * 8);
  p.cluster_reduce = cluster_reduce ? 1 : 0;
  p.partials = nullptr;
  p.tickets = nullptr;
  if (splits > 1 && !cluster_reduce) {
    p.partials = static_cast<float *>(scratch);
    p.tickets = reinterpret_cast<unsigned int *>(static_cast<uint8_t *>(scratch) + partial_bytes);
    if (!scratch_is_clean)
      if (int rc = check_cuda(cudaMemsetAsync(p.tickets, 0, ticket_bytes, st), "zero split-K tickets")) return rc;
  }

  CUtensorMap tw, tx;
  if (int rc = make_tmap_2d_bytes(&tw, wq, gp.K, gp.N, gp.K, kBK, kWRows, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  if (int rc = make_tmap_2d_bytes(&tx, xq, gp.K, gp.total_m, gp.K, kBK, p.x_box_rows, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  switch (bt) {
    case 16: return launch_decode<16>(tw, tx, p, static_cast<int>(n_tiles), st);
    case 32: return launch_decode<32>(tw, tx, p, static_cast<int>(n_tiles), st);
    case 64: return launch_decode<64>(tw, tx, p, static_cast<int>(n_tiles), st);
    default: return launch_decode<128>(tw, tx, p, static_cast<int>(n_tiles), st);
  }
}

}  // namespace gemm_f8
}  // namespace mslk_b200

// ---------------------------------------------------------------------------
// Few-token GEMM with built-in scratch: for callers that must not allocate.
//
// Some hosts of this library cannot obtain device memory at call time: a serving
// engine that has handed all free HBM to its KV-cache pool at start-up (a late
// cudaMalloc simply fails there), a runtime whose memory plan is fixed before
// the first request, or a plugin called from a thread that is forbidden to
// touch the allocator because cudaMalloc/cudaFree synchronise the whole device.
// For them the split-K scratch of the weight-streaming kernel lives in the
// array below, which is part of the library image: every GPU that loads the
// library carries these 8 MiB until the process exits, and nothing is
// allocated or freed by the call.
//
// The host cannot use the array's name as a pointer (on the host it is only a
// handle for the symbol); the device address is looked up once per device with
// cudaGetSymbolAddress, with that device current.  The look-up happens in the
// first call made on a device, so make that first call outside stream capture.
//
// All calls on a device share the one array.  The partial sums left by the
// previous call are simply overwritten; the completion tickets must start at
// zero and are cleared on the stream before every launch.  Two calls that can
// run at the same time on one GPU (different streams, or graph branches) would
// mix their partial sums and tickets: keep such calls ordered.
// ---------------------------------------------------------------------------
namespace mslk_b200 {
namespace gemm_f8 {
namespace {

constexpr size_t kBuiltinScratchBytes = 8u << 20;  // 8 MiB: bounds the shapes with 33..128 tokens (fewer tokens use no scratch)
constexpr int kNoAllocMaxTokens = 128;             // what the weight-streaming kernel itself can take
static __device__ __align__(256) unsigned char g_builtin_scratch[kBuiltinScratchBytes];

constexpr int kMaxDevicesTracked = 64;
std::mutex g_builtin_mu;
void *g_builtin_ptr[kMaxDevicesTracked];

// Device address of g_builtin_scratch on the current device (looked up once per device).
int builtin_scratch_ptr(void **out) {
  int dev = 0;
  if (int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
  if (dev < 0 || dev >= kMaxDevicesTracked) return fail(2, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_builtin_mu);
  if (!g_builtin_ptr[dev]) {
    void *ptr = nullptr;
    if (int rc = check_cuda(cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_builtin_scratch),
                            "cudaGetSymbolAddress(built-in scratch)"))
      return rc;
    g_builtin_ptr[dev] = ptr;
  }
  *out = g_builtin_ptr[dev];
  return 0;
}

}  // namespace
}  // namespace gemm_f8
}  // namespace mslk_b200

MSLK_API int mslk_b200_f8f8bf16_rowwise_noalloc(const void *xq, const void *wq, const float *x_scale,
                                                const float *w_scale, const void *bias, int bias_kind, void *y,
                                                int64_t M, int64_t N, int64_t K, void *stream) {
  using namespace mslk_b200;
  using namespace mslk_b200::gemm_f8;
  clear_error();
  const char *name = "f8f8bf16_rowwise_noalloc";
  if (bias_kind < 0 || bias_kind > 2) return fail(1, "%s: bad bias_kind %d", name, bias_kind);
  if (M < 1 || M > kNoAllocMaxTokens)
    return fail(1, "%s: this entry point serves 1..%d tokens (got M=%lld); use f8f8bf16_rowwise for more", name,
                kNoAllocMaxTokens, (long long)M);
  if (N < 128 || N > 0x7fffff00LL) return fail(1, "%s: N (%lld) must be at least 128", name, (long long)N);
  if (K < 16 || K > 0x7fffff00LL || K % 16 != 0)
    return fail(1, "%s: K (%lld) must be a positive multiple of 16", name, (long long)K);
  if (!xq || !wq || !x_scale || !w_scale || !y) return fail(1, "%s: null pointer argument", name);
  if (bias_kind != MSLK_B200_BIAS_NONE && !bias) return fail(1, "%s: bias_kind set but bias is null", name);
  // Up to 32 tokens K is split inside thread-block clusters: no scratch, no size limit, no address look-up.
  // Above, the split-K partial tiles live in the built-in array, whose size bounds the shapes served.
  void *scratch = nullptr;
  if (M > kDecodeMaxTokens) {
    const size_t need = decode_scratch_bytes(M, N, K, sm_count());
    if (need > kBuiltinScratchBytes)
      return fail(1, "%s: M=%lld N=%lld K=%lld needs %zu bytes of scratch, the built-in buffer holds %zu", name,
                  (long long)M, (long long)N, (long long)K, need, kBuiltinScratchBytes);
    if (int rc = builtin_scratch_ptr(&scratch)) return rc;
  }
  int *status = device_status_ptr();
  if (!status) return 2;
  GemmParams p;
  p.x_scale = x_scale;
  p.w_scale = w_scale;
  p.bias = bias;
  p.y = static_cast<__nv_bfloat16 *>(y);
  p.m_sizes = nullptr;
  p.status = status;
  p.bias_kind = bias_kind;
  p.G = 1;
  p.total_m = static_cast<int>(M);
  p.group_m = static_cast<int>(M);
  p.N = static_cast<int>(N);
  p.K = static_cast<int>(K);
  default_placement(p);
  // The tickets in the built-in array are zeroed on the stream before the launch.
  if (M <= kDecodeMaxTokens)
    return launch_decode_kernel(xq, wq, p, nullptr, 0, false, static_cast<cudaStream_t>(stream));
  return launch_decode_kernel(xq, wq, p, scratch, kBuiltinScratchBytes, false, static_cast<cudaStream_t>(stream));
}

