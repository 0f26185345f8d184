// Rowwise-scaled FP8 GEMM for sm_100a, dense and grouped (stacked MoE) in one
// persistent, warp-specialised tcgen05 kernel.
//
//   y[m, n] = bf16((x_scale[m] * sum_k xq[m,k] * wq[n,k]) * w_scale[n] (+ bias[n]))
//
// Both operands are K-major e4m3 bytes, so an operand tile is a TMA box of
// {128 bytes of K, rows} written to shared memory with the 128-byte swizzle and
// consumed in place by tcgen05.mma (kind::f8f6f4, 128 x BN x 32 per instruction,
// fp32 accumulators in tensor memory).
//
// Roles (192 threads, one CTA per SM):
//   warp 0      TMA producer: fills a kStages-deep ring of {A 128x128, B BNx128} tiles
//   warp 1      MMA issuer (one elected lane) and owner of the TMEM allocation
//   warps 2..5  epilogue: tcgen05.ld the finished accumulator, apply the row and
//               column scales (+ bias), convert to bf16 and store
// Two accumulators (2 x BN TMEM columns) let the epilogue of tile i overlap the
// main loop of tile i+1.
//
// Tile scheduler (device side, static round-robin over a linear tile index): the
// kernel reads the per-group row counts from device memory, builds prefix tables
// in shared memory and maps tile -> (group, 128-row block, BN-column block).  A
// dense GEMM is the one-group case.  Groups with zero rows own no tiles.  Tiles
// of a group are visited in bands of kBandM row blocks so that CTAs running at
// the same time share operand tiles in L2.  Row blocks may run past the end of
// their group (or of the tensor: TMA zero-fills); the epilogue masks those rows.
//
// Every pipeline wait is bounded (see common.cuh); on expiry the CTA records a
// status code, drains, frees its tensor memory and returns.
#include "gemm_f8_common.cuh"

#include <atomic>
#include <cstdlib>

namespace mslk_b200 {
namespace gemm_f8 {
namespace {

template <int BN>
struct Config {
  static constexpr int kStageA = kBM * kBK;
  static constexpr int kStageB = BN * kBK;
  static constexpr int kStageBytes = kStageA + kStageB;
  // ring depth: as many stages as fit beside ~16 KB of tables
  static constexpr int kStages = BN == 256 ? 4 : BN == 128 ? 6 : BN == 64 ? 8 : 10;
  static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;
  static constexpr uint32_t kIdesc = (1u << 4)                                   // fp32 accumulate
                                     | (0u << 7) | (0u << 10)                    // A, B = e4m3
                                     | (static_cast<uint32_t>(BN >> 3) << 17)    // N
                                     | (static_cast<uint32_t>(kBM >> 4) << 24);  // M
};

// Shared-memory carve-up after the operand ring (which starts 1024-byte aligned).
template <int BN>
struct SmemTail {
  float w_scale[4][BN];  // one private copy per epilogue warp (no cross-warp sync in the epilogue)
  float bias[4][BN];
  int tile_start[kMaxGroups + 1];
  int row_start[kMaxGroups + 1];
  uint64_t full[Config<BN>::kStages];
  uint64_t empty[Config<BN>::kStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

template <int BN>
constexpr size_t smem_bytes() {
  return 1024 + static_cast<size_t>(Config<BN>::kStages) * Config<BN>::kStageBytes + sizeof(SmemTail<BN>);
}

template <int BN>
__global__ void __launch_bounds__(kNumThreads, 1)
    gemm_f8_rowwise_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                           const GemmParams p) {
  using Cfg = Config<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *ring = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  SmemTail<BN> &S = *reinterpret_cast<SmemTail<BN> *>(ring + static_cast<size_t>(Cfg::kStages) * Cfg::kStageBytes);

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  const int n_tiles = (p.N + BN - 1) / BN;
  const int k_blocks = (p.K + kBK - 1) / kBK;
  volatile int *abort_flag = &S.abort_flag;

  // ------------------------------------------------------------------ setup
  if (threadIdx.x == 0) {
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&S.full[s], 1);
      mbar_init(&S.empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&S.tmem_full[a], 1);
      mbar_init(&S.tmem_empty[a], kNumEpilogueThreads / 32);
    }
    S.abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  // Dense problems: the thread that has just initialised the barriers also issues the first stages of this CTA's first
  // tile, before the CTA-wide barrier below -- the copies then fly while tensor memory is allocated and the other
  // warps arrive (a microsecond on few-token shapes whose whole launch takes ten).  The group tables of a dense
  // problem are two entries each, written here; every thread derives the number of stages issued early by itself.
  const bool dense = p.G == 1 && p.m_sizes == nullptr && p.end_offsets == nullptr;
  const int dense_tiles = ((p.total_m + kBM - 1) / kBM) * n_tiles;
  const int pre = (dense && static_cast<int>(blockIdx.x) < dense_tiles) ? min(Cfg::kStages, k_blocks) : 0;
  if (threadIdx.x == 0 && dense) {
    S.row_start[0] = 0;
    S.row_start[1] = p.total_m;
    S.tile_start[0] = 0;
    S.tile_start[1] = dense_tiles;
    griddep_wait();   // the operands may come from the previous kernel of the stream
    Scheduler first{S.tile_start, S.row_start, p.G, p.N, n_tiles, BN, kBM, kBandM, 0};
    Tile t0;
    if (pre > 0 && first.get(blockIdx.x, t0)) {
      for (int kb = 0; kb < pre; ++kb) {
        uint8_t *sa = ring + static_cast<size_t>(kb) * Cfg::kStageBytes;
        mbar_arrive_expect_tx(&S.full[kb], p.a_box_rows * kBK + Cfg::kStageB);
        tma_load_2d(sa, &tmap_a, &S.full[kb], kb * kBK, t0.row0);
        tma_load_2d(sa + Cfg::kStageA, &tmap_b, &S.full[kb], kb * kBK, t0.wrow0);
      }
    }
  }
  if (warp == 1) {
    tmem_alloc(&S.tmem_base, Cfg::kTmemCols);
    tmem_relinquish();
  }
  // everything above touched shared and tensor memory only (and, after its own wait, the early copies): it may run
  // under the tail of the previous kernel of the stream; from here on global memory is read (group sizes, operands,
  // scales) and written
  griddep_wait();
  griddep_launch_dependents();
  if (warp == 2 && !dense) build_group_tables(p, n_tiles, kBM, lane, S.row_start, S.tile_start);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = S.tmem_base;

  Scheduler sched{S.tile_start, S.row_start, p.G, p.N, n_tiles, BN, kBM, kBandM, 0};

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (elect_one()) {  // one lane, chosen so that the compiler keeps the issue loop on the uniform datapath
      // the first `pre` stages of the first tile are already on their way (setup above)
      int stage = pre == Cfg::kStages ? 0 : pre;
      uint32_t phase = pre == Cfg::kStages ? 1u : 0u;
      long long issued = pre;
      bool ok = true;
      Tile t;
      int kb_first = pre;
      for (int tile = blockIdx.x; ok && sched.get(tile, t); tile += gridDim.x) {
        for (int kb = kb_first; kb < k_blocks; ++kb) {
          if (!mbar_wait(&S.empty[stage], phase ^ 1, abort_flag, p.status, kStatusProducerTimeout)) {
            ok = false;
            break;
          }
          uint8_t *sa = ring + static_cast<size_t>(stage) * Cfg::kStageBytes;
          uint8_t *sb = sa + Cfg::kStageA;
          mbar_arrive_expect_tx(&S.full[stage], p.a_box_rows * kBK + Cfg::kStageB);
          tma_load_2d(sa, &tmap_a, &S.full[stage], kb * kBK, t.row0);
          tma_load_2d(sb, &tmap_b, &S.full[stage], kb * kBK, t.wrow0);
          ++issued;
          if (++stage == Cfg::kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        kb_first = 0;
      }
      if (!ok) {
        // bounded drain: give copies already issued time to land before the CTA exits
        const unsigned long long t0 = globaltimer_ns();
        const int pending = issued < Cfg::kStages ? static_cast<int>(issued) : Cfg::kStages;
        for (int i = 0; i < pending; ++i) {
          int s = stage - 1 - i;
          uint32_t ph = phase;
          if (s < 0) {
            s += Cfg::kStages;
            ph ^= 1;
          }
          while (!mbar_try_wait(&S.full[s], ph)) {
            if (globaltimer_ns() - t0 > 1000000ull) {
              atomicCAS(p.status, 0, kStatusDrainTimeout);
              break;
            }
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {  // one lane, chosen so that the compiler keeps the issue loop on the uniform datapath
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      Tile t;
      for (int tile = blockIdx.x; ok && sched.get(tile, t); tile += gridDim.x, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&S.tmem_empty[acc], acc_phase ^ 1, abort_flag, p.status, kStatusMmaTimeout)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&S.full[stage], phase, abort_flag, p.status, kStatusMmaTimeout)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(ring + static_cast<size_t>(stage) * Cfg::kStageBytes);
          const uint64_t da = make_kmajor_sw128_desc(sa);
          const uint64_t db = make_kmajor_sw128_desc(sa + Cfg::kStageA);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            // advancing K inside the 128-byte swizzle row: +32 bytes on the start address
            mma_f8f6f4(d_tmem, da + static_cast<uint64_t>(k * (kUmmaK >> 4)),
                       db + static_cast<uint64_t>(k * (kUmmaK >> 4)), Cfg::kIdesc, (kb | k) != 0 ? 1u : 0u);
          }
          tc_commit(&S.empty[stage]);  // frees the stage once these MMAs have read it
          if (++stage == Cfg::kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        tc_commit(&S.tmem_full[acc]);  // accumulator complete
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quad = warp & 3;             // TMEM lane quadrant this warp may read
    const int row_in_tile = quad * 32 + lane;
    bool y_vec_ok = (p.ldy % 8 == 0) && (p.col0 % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.y) & 15u) == 0);
    for (int d = 0; d < p.n_extra; ++d) y_vec_ok = y_vec_ok && ((reinterpret_cast<uintptr_t>(p.y_extra[d]) & 15u) == 0);
    int local = 0;
    bool ok = true;
    Tile t;
    for (int tile = blockIdx.x; ok && sched.get(tile, t); tile += gridDim.x, ++local) {
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      // stage the column scales (and bias) of this tile in this warp's private buffer
      float *ws_s = S.w_scale[warp - 2];
      float *bs_s = S.bias[warp - 2];
      for (int c = lane; c < BN; c += 32) {
        const bool in = t.n0 + c < p.N;
        ws_s[c] = in ? p.w_scale[t.ws0 + c] : 0.f;
        float b = 0.f;
        if (in && p.bias_kind == MSLK_B200_BIAS_F32) b = static_cast<const float *>(p.bias)[t.ws0 + c];
        if (in && p.bias_kind == MSLK_B200_BIAS_BF16)
          b = __bfloat162float(static_cast<const __nv_bfloat16 *>(p.bias)[t.ws0 + c]);
        bs_s[c] = b;
      }
      __syncwarp();
      bool row_ok = row_in_tile < t.rows;
      const float xs = row_ok ? p.x_scale[t.row0 + row_in_tile] : 0.f;
      long long out_row = t.row0 + row_in_tile;
      if (p.scatter_idx && row_ok) {
        out_row = p.scatter_bits == 64 ? static_cast<const long long *>(p.scatter_idx)[t.row0 + row_in_tile]
                                       : static_cast<long long>(static_cast<const int *>(p.scatter_idx)[t.row0 + row_in_tile]);
        if (out_row < 0 || out_row >= p.scatter_rows) {   // reported, not followed
          atomicOr(p.status, kStatusBadScatterIndex);
          row_ok = false;
        }
      }
      // warp-uniform decision: either every lane saw the accumulator complete or the warp leaves
      const bool got = mbar_wait(&S.tmem_full[acc], acc_phase, abort_flag, p.status, kStatusEpilogueTimeout);
      if (!__all_sync(0xffffffffu, got)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + static_cast<uint32_t>(acc * BN) + (static_cast<uint32_t>(quad * 32) << 16);
      const size_t yoff = static_cast<size_t>(out_row) * p.ldy + p.col0 + t.n0;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int cols_left = p.N - (t.n0 + c * 32);
        if (cols_left <= 0) break;
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        const float *ws = ws_s + c * 32;
        const float *bs = bs_s + c * 32;
        if (p.bias_kind == MSLK_B200_BIAS_NONE)
          epilogue_chunk<BN, MSLK_B200_BIAS_NONE>(r, xs, ws, bs, p, yoff + c * 32, row_ok, cols_left, y_vec_ok);
        else if (p.bias_kind == MSLK_B200_BIAS_F32)
          epilogue_chunk<BN, MSLK_B200_BIAS_F32>(r, xs, ws, bs, p, yoff + c * 32, row_ok, cols_left, y_vec_ok);
        else
          epilogue_chunk<BN, MSLK_B200_BIAS_BF16>(r, xs, ws, bs, p, yoff + c * 32, row_ok, cols_left, y_vec_ok);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&S.tmem_empty[acc]);
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <int BN>
int launch(const CUtensorMap &ta, const CUtensorMap &tb, const GemmParams &p, int grid, cudaStream_t st) {
  static std::atomic<bool> attr_set[64];   // zero-initialised; two first calls may both set the (idempotent) attribute
  int dev = 0;
  if (int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
  constexpr size_t smem = smem_bytes<BN>();
  static_assert(smem <= 232448, "shared memory budget exceeded");
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (int rc = check_cuda(cudaFuncSetAttribute(gemm_f8_rowwise_kernel<BN>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)),
                            "cudaFuncSetAttribute(gemm_f8_rowwise)"))
      return rc;
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(kNumThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_attribute(&attr[0]);   // the prologue may overlap the tail of the previous kernel of the stream
  return check_cuda(cudaLaunchKernelEx(&cfg, gemm_f8_rowwise_kernel<BN>, ta, tb, p), "f8f8bf16_rowwise launch");
}

int run(const void *xq, const void *wq, const float *xs, const float *ws, const void *bias, int bias_kind, void *y,
        const int64_t *m_sizes, int64_t G, int64_t total_m, int64_t N, int64_t K, void *scratch, size_t scratch_bytes,
        cudaStream_t st, const char *name, const GemmParams *placement = nullptr) {
  if (total_m < 0 || N < 0 || K < 0 || G < 1) return fail(1, "%s: bad shape", name);
  if (total_m == 0 || N == 0) return 0;
  if (G > kMaxGroups) return fail(1, "%s: at most %d groups are supported (got %lld)", name, kMaxGroups, (long long)G);
  if (total_m > 0x7fffff00LL || G * N > 0x7fffff00LL || K > 0x7fffff00LL)
    return fail(1, "%s: dimension too large for 32-bit tile coordinates", name);
  if (!y) return fail(1, "%s: null output pointer", name);
  if (K == 0) {
    // empty reduction: the reference returns zeros
    return check_cuda(cudaMemsetAsync(y, 0, static_cast<size_t>(total_m) * N * 2, st), "memset");
  }
  if (!xq || !wq || !xs || !ws) return fail(1, "%s: null pointer argument", name);
  if (bias_kind != MSLK_B200_BIAS_NONE && !bias) return fail(1, "%s: bias_kind set but bias is null", name);
  if (K % 16 != 0) return fail(1, "%s: K (%lld) must be a multiple of 16 (TMA row pitch)", name, (long long)K);
  int *status = device_status_ptr();
  if (!status) return 2;

  const int sms = sm_count();
  // upper bound of the row blocks: exact for equal groups, one ragged block per group otherwise
  const int64_t group_m = total_m / G;
  if (!m_sizes && group_m * G != total_m) return fail(1, "%s: rows are not a multiple of the batch count", name);
  const int64_t m_tiles_ub = m_sizes ? (total_m + kBM - 1) / kBM + G : G * ((group_m + kBM - 1) / kBM);
  // Column block of the one-CTA kernel: a tile streams (128 + BN) rows of K bytes, and the tiles run in waves of one
  // per SM, so the launch costs about waves x (128 + BN) row loads (+ a constant per tile).  M = 128, N = 6144:
  // BN = 32 gives 192 tiles = two waves (15.7 us), BN = 64 gives 96 tiles in one (the reference's 128 x 64 tiles: 9.8 us).
  int bn = 256;
  {
    int64_t best_cost = -1;
    for (int cand = 256; cand >= 32; cand /= 2) {
      if (cand > 32 && cand / 2 >= N) continue;   // half the width already covers N
      const int64_t tiles = m_tiles_ub * ((N + cand - 1) / cand);
      const int64_t cost = ((tiles + sms - 1) / sms) * (128 + cand + 32);
      if (best_cost < 0 || cost < best_cost) {
        best_cost = cost;
        bn = cand;
      }
    }
  }

  GemmParams p;
  p.x_scale = xs;
  p.w_scale = ws;
  p.bias = bias;
  p.y = static_cast<__nv_bfloat16 *>(y);
  p.m_sizes = m_sizes;
  p.status = status;
  p.bias_kind = bias_kind;
  p.G = static_cast<int>(G);
  p.total_m = static_cast<int>(total_m);
  p.group_m = static_cast<int>(group_m);
  p.N = static_cast<int>(N);
  p.K = static_cast<int>(K);
  default_placement(p);
  if (placement) {
    p.n_extra = placement->n_extra;
    p.ldy = placement->ldy;
    p.col0 = placement->col0;
    for (int i = 0; i < 7; ++i) p.y_extra[i] = placement->y_extra[i];
    p.rs_rows = placement->rs_rows;
    p.rs_slot = placement->rs_slot;
    p.scatter_idx = placement->scatter_idx;
    p.scatter_bits = placement->scatter_bits;
    p.scatter_rows = placement->scatter_rows;
  }

  // few tokens AND scratch given: weight-streaming kernel with the K dimension split over independent
  // CTAs (partial tiles and completion tickets in the caller's scratch memory).
  if (!m_sizes && G == 1 && !placement && scratch && total_m <= kDecodeMaxTokens && N >= 128)
    return launch_decode_kernel(xq, wq, p, scratch, scratch_bytes, false, st);
  // Without scratch the same kernel splits K inside thread-block clusters (partial tiles meet in shared
  // memory) or runs unsplit, one CTA per 128 weight rows at two CTAs per SM.  M = 1 / 16 / 32 against the
  // general kernel's 32-column tiles: (4096, 4096) 7.0 / 7.9 / 9.4 us against 8.8 / 8.8 / 9.0; (6144, 4096)
  // 8.2 / 9.6 / 10.9 against 13.8; (4096, 14336) 12.9 / 13.7 / 14.6 against 20.5; (8192, 8192) 14.6 / 15.8 /
  // 16.9 against 23.3; (28672, 4096) 21.3 / 21.8 / 22.8 against 24.1 / 24.6 / 25.0.  Above 32 tokens the
  // general kernel is faster (M = 128, (8192, 8192): 23.9 against 32.9 us).
  // 33..128 tokens: only with long K and few weight blocks, i.e. when the cluster split applies -- M = 64:
  // (4096, 14336) 16.3 against 20.7 us, (8192, 8192) 20.5 against 23.5, (8192, 28672) 45.1 against 69.0;
  // M = 128: (8192, 28672) 50.9 against 69.8, but (8192, 8192) 24.4 against 24.1.
  const bool few_blocks = 2 * ((static_cast<int64_t>(N) + 127) / 128) <= sm_count();
  const bool more_tokens_ok = few_blocks && ((total_m <= 64 && K >= 8192) || (total_m <= 128 && K >= 16384));
  if (!m_sizes && G == 1 && !placement && !scratch && N >= 2048 &&
      (total_m <= kDecodeMaxTokens || more_tokens_ok))
    return launch_decode_kernel(xq, wq, p, nullptr, 0, false, st);

  // CTA pairs (256 x 256 tiles) when there are enough such tiles to occupy every pair of SMs
  static const int force = [] {
    const char *e = getenv("MSLK_B200_GEMM_KERNEL");  // "1cta" | "2cta": tuning aid, default = heuristic
    return !e ? 0 : (e[0] == '2' ? 2 : 1);
  }();
  const int64_t pair_tiles = (m_sizes ? (total_m + 2 * kBM - 1) / (2 * kBM) : G * ((group_m + 2 * kBM - 1) / (2 * kBM))) *
                             ((N + 255) / 256);
  // grouped problems run on pairs with swapped operand roles (tokens as the N operand, padded to 16
  // only), which pays off unless the groups are tiny
  const bool groups_tall = !m_sizes || total_m / G >= 128;
  // (a dense problem of at most 128 rows stays on one CTA per tile: half of every 256-row pair tile would be padding)
  // scatter-add epilogue: in the pair kernel for grouped problems with swapped roles, else in this file's kernel
  const bool want_pair = (!p.scatter_idx || (m_sizes && total_m / G < 2048)) &&
                         (force == 2 || p.rs_rows > 0 ||
                          (force == 0 && groups_tall && bn == 256 && pair_tiles >= sms / 2 && (m_sizes || G > 1 || total_m > kBM)));
  if (want_pair) {
    const int rc = launch_pair_kernel(xq, wq, p, st);
    if (rc >= 0) return rc;  // -1: pairs unavailable on this device, fall through to one CTA per tile
    if (p.rs_rows > 0) return fail(2, "%s: the row-scatter GEMM needs CTA pairs, which this device cannot run", name);
  }

  CUtensorMap ta, tb;
  if (!m_sizes && G == 1 && total_m < kBM) p.a_box_rows = static_cast<int>((total_m + 7) / 8 * 8);
  if (int rc = make_tmap_2d_bytes(&ta, xq, K, total_m, K, kBK, p.a_box_rows, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  if (int rc = make_tmap_2d_bytes(&tb, wq, K, G * N, K, kBK, bn, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;

  const int64_t tiles_ub = m_tiles_ub * ((N + bn - 1) / bn);
  const int grid = static_cast<int>(tiles_ub < sms ? tiles_ub : sms);
  switch (bn) {
    case 256: return launch<256>(ta, tb, p, grid, st);
    case 128: return launch<128>(ta, tb, p, grid, st);
    case 64: return launch<64>(ta, tb, p, grid, st);
    default: return launch<32>(ta, tb, p, grid, st);
  }
}

}  // namespace
}  // namespace gemm_f8
}  // namespace mslk_b200

MSLK_API int mslk_b200_f8f8bf16_rowwise(const void *xq, const void *wq, const float *x_scale, const float *w_scale,
                                        const void *bias, int bias_kind, void *y, int64_t M, int64_t N, int64_t K,
                                        void *stream) {
  using namespace mslk_b200;
  using namespace mslk_b200::gemm_f8;
  clear_error();
  if (bias_kind < 0 || bias_kind > 2) return fail(1, "f8f8bf16_rowwise: bad bias_kind %d", bias_kind);
  return run(xq, wq, x_scale, w_scale, bias, bias_kind, y, nullptr, 1, M, N, K, nullptr, 0,
             static_cast<cudaStream_t>(stream), "f8f8bf16_rowwise");
}

MSLK_API int mslk_b200_f8f8bf16_rowwise_allgather(const void *xq, const void *wq_shard, const float *x_scale,
                                                  const float *w_scale_shard, const void *bias_shard, int bias_kind,
                                                  void *const *y_bases, int world, int rank, int64_t M,
                                                  int64_t N_local, int64_t K, void *stream) {
  using namespace mslk_b200;
  using namespace mslk_b200::gemm_f8;
  clear_error();
  const char *name = "f8f8bf16_rowwise_allgather";
  if (bias_kind < 0 || bias_kind > 2) return fail(1, "%s: bad bias_kind %d", name, bias_kind);
  if (world < 1 || world > 8 || rank < 0 || rank >= world) return fail(1, "%s: need 1 <= world <= 8 and 0 <= rank < world", name);
  if (!y_bases) return fail(1, "%s: y_bases is null", name);
  for (int r = 0; r < world; ++r)
    if (!y_bases[r]) return fail(1, "%s: y_bases[%d] is null", name, r);
  if (N_local * world > 0x7fffff00LL) return fail(1, "%s: N too large", name);
  GemmParams place;
  place.N = static_cast<int>(N_local);
  default_placement(place);
  place.ldy = static_cast<int>(N_local * world);
  place.col0 = static_cast<int>(N_local * rank);
  // peers in ring order starting after this rank, so that the ranks do not all write to the same peer first
  for (int i = 1; i < world; ++i) place.y_extra[i - 1] = static_cast<__nv_bfloat16 *>(y_bases[(rank + i) % world]);
  place.n_extra = world - 1;
  return run(xq, wq_shard, x_scale, w_scale_shard, bias_shard, bias_kind, y_bases[rank], nullptr, 1, M, N_local, K,
             nullptr, 0, static_cast<cudaStream_t>(stream), name, &place);
}

MSLK_API int mslk_b200_f8f8bf16_rowwise_scatter(const void *xq_kshard, const void *wq_kshard, const float *x_scale,
                                                const float *w_scale, void *const *stage_bases, int world, int rank,
                                                int64_t M, int64_t N, int64_t K_local, void *stream) {
  using namespace mslk_b200;
  using namespace mslk_b200::gemm_f8;
  clear_error();
  const char *name = "f8f8bf16_rowwise_scatter";
  if (world < 1 || world > 8 || rank < 0 || rank >= world) return fail(1, "%s: need 1 <= world <= 8 and 0 <= rank < world", name);
  if (!stage_bases) return fail(1, "%s: stage_bases is null", name);
  for (int r = 0; r < world; ++r)
    if (!stage_bases[r]) return fail(1, "%s: stage_bases[%d] is null", name, r);
  if (M <= 0 || M % (32 * world) != 0) return fail(1, "%s: M (%lld) must be a positive multiple of 32*world", name, (long long)M);
  if (N % 64 != 0) return fail(1, "%s: N (%lld) must be a multiple of 64", name, (long long)N);
  GemmParams place;
  place.N = static_cast<int>(N);
  default_placement(place);
  for (int i = 1; i < world; ++i) place.y_extra[i - 1] = static_cast<__nv_bfloat16 *>(stage_bases[i]);
  place.n_extra = world - 1;
  place.rs_rows = static_cast<int>(M / world);
  place.rs_slot = rank;
  return run(xq_kshard, wq_kshard, x_scale, w_scale, nullptr, MSLK_B200_BIAS_NONE, stage_bases[0], nullptr, 1, M, N,
             K_local, nullptr, 0, static_cast<cudaStream_t>(stream), name, &place);
}

MSLK_API size_t mslk_b200_f8f8bf16_rowwise_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  using namespace mslk_b200;
  using namespace mslk_b200::gemm_f8;
  if (M <= 0 || M > kDecodeMaxTokens || N < 128 || K <= 0) return 0;
  return decode_scratch_bytes(M, N, K, sm_count());
}

MSLK_API int mslk_b200_f8f8bf16_rowwise_ws(const void *xq, const void *wq, const float *x_scale, const float *w_scale,
                                           const void *bias, int bias_kind, void *y, int64_t M, int64_t N, int64_t K,
                                           void *workspace, size_t workspace_bytes, void *stream) {
  using namespace mslk_b200;
  using namespace mslk_b200::gemm_f8;
  clear_error();
  if (bias_kind < 0 || bias_kind > 2) return fail(1, "f8f8bf16_rowwise: bad bias_kind %d", bias_kind);
  if (workspace && (reinterpret_cast<uintptr_t>(workspace) & 15u))
    return fail(1, "f8f8bf16_rowwise: workspace must be 16-byte aligned");
  return run(xq, wq, x_scale, w_scale, bias, bias_kind, y, nullptr, 1, M, N, K, workspace, workspace_bytes,
             static_cast<cudaStream_t>(stream), "f8f8bf16_rowwise");
}

MSLK_API int mslk_b200_f8f8bf16_rowwise_grouped_stacked(const void *xq, const void *wq, const float *x_scale,
                                                        const float *w_scale, const int64_t *M_sizes, int64_t G,
                                                        int64_t total_M, int64_t N, int64_t K, void *y,
                                                        void *stream) {
  using namespace mslk_b200;
  using namespace mslk_b200::gemm_f8;
  clear_error();
  if (!M_sizes) return fail(1, "f8f8bf16_rowwise_grouped_stacked: M_sizes is null");
  return run(xq, wq, x_scale, w_scale, nullptr, MSLK_B200_BIAS_NONE, y, M_sizes, G, total_M, N, K, nullptr, 0,
             static_cast<cudaStream_t>(stream), "f8f8bf16_rowwise_grouped_stacked");
}

MSLK_API int mslk_b200_f8f8bf16_rowwise_batched(const void *xq, const void *wq, const float *x_scale,
                                                const float *w_scale, const void *bias, int bias_kind, void *y,
                                                int64_t B, int64_t M, int64_t N, int64_t K, void *stream) {
  using namespace mslk_b200;
  using namespace mslk_b200::gemm_f8;
  clear_error();
  if (bias_kind < 0 || bias_kind > 2) return fail(1, "f8f8bf16_rowwise_batched: bad bias_kind %d", bias_kind);
  if (B < 0 || M < 0) return fail(1, "f8f8bf16_rowwise_batched: bad shape");
  if (B == 0 || M == 0) return 0;
  // B equal groups of M stacked rows, group b multiplying its own weight block wq[b]
  return run(xq, wq, x_scale, w_scale, bias, bias_kind, y, nullptr, B, B * M, N, K, nullptr, 0,
             static_cast<cudaStream_t>(stream), "f8f8bf16_rowwise_batched");
}

MSLK_API int mslk_b200_f8f8bf16_rowwise_grouped_stacked_scatter_add(const void *xq, const void *wq, const float *x_scale,
                                                                    const float *w_scale, const int64_t *M_sizes,
                                                                    int64_t G, int64_t total_M, int64_t N, int64_t K,
                                                                    const void *scatter_indices, int index_bits,
                                                                    void *y, int64_t y_rows, void *stream) {
  using namespace mslk_b200;
  using namespace mslk_b200::gemm_f8;
  clear_error();
  const char *name = "f8f8bf16_rowwise_grouped_stacked_scatter_add";
  if (!M_sizes) return fail(1, "%s: M_sizes is null", name);
  if (!scatter_indices) return fail(1, "%s: scatter_indices is null", name);
  if (index_bits != 32 && index_bits != 64) return fail(1, "%s: indices must be int32 or int64", name);
  if (y_rows < 0 || y_rows > 0x7fffffffLL) return fail(1, "%s: bad output row count", name);
  if (K == 0) return 0;   // an empty reduction adds nothing
  GemmParams placement;
  placement.N = static_cast<int>(N);
  default_placement(placement);
  placement.scatter_idx = scatter_indices;
  placement.scatter_bits = index_bits;
  placement.scatter_rows = static_cast<int>(y_rows);
  return run(xq, wq, x_scale, w_scale, nullptr, MSLK_B200_BIAS_NONE, y, M_sizes, G, total_M, N, K, nullptr, 0,
             static_cast<cudaStream_t>(stream), name, &placement);
}
