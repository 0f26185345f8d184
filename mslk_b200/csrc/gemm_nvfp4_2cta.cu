// NVFP4 GEMM on CTA pairs (tcgen05 cta_group::2, block-scaled) for sm_100a; dense problems.
//
// Two CTAs on neighbouring SMs compute one 256 x 256 output tile with 256 x 256 x 64 instructions.
// Each CTA loads its own 128 rows of A and its own 128 of the 256 rows of B: 38 KB per SM and K block
// (256 elements of K) instead of the 54 KB of the one-CTA kernel with 256-column tiles.  That matters
// because this GEMM is bound by how fast operands arrive from L2 (bytes in flight per SM / latency),
// not by the tensor pipe: with three of four instructions and all scale copies removed the one-CTA
// kernel ran only 20 % faster.  Scale factors: each
// CTA needs, in its own tensor memory, the A scales of its own 128 rows and the B scales of ALL 256
// columns; both CTAs therefore fetch both B scale blocks themselves (4 KB per K block; no load is
// multicast).  Scale atoms travel as TMA boxes of {512 bytes, atoms of one stage} over a 2-D view of the scale
// buffer, so that, like the operand tiles, they can signal the leader's barrier from either CTA.
//
//   CTA rank 0 ("leader")                              CTA rank 1
//   warp 0  producer: own empty[s] -> 5 TMA loads into own smem, bytes counted on the LEADER's full[s]
//   warp 1  MMA issuer: tcgen05.cp (pair-wide: every CTA copies its own atoms into its own tensor
//           memory) one K block ahead, then the pair-wide MMAs; commits to both CTAs' barriers
//                                                       (idle; takes part in TMEM alloc)
//   warps 2..5 epilogue on the CTA's own 128 accumulator rows; all eight warps arrive on the
//           leader's tmem_empty barrier
//
// Waits are bounded as everywhere else (common.cuh); cluster-wide hardware barriers only at start-up
// and teardown, reached on every path.
#include "gemm_nvfp4_pair.h"

#include "common.cuh"

#include <atomic>
#include <cstdlib>

namespace mslk_b200 {
namespace nvfp4_pair {
namespace {

constexpr int kBM = 128;                 // rows per CTA
constexpr int kPairRows = 256;           // rows of the pair tile
constexpr int kPairBN = 256;             // columns of the pair tile
constexpr int kMmaKBytes = 32;           // 64 K-elements per instruction
constexpr int kAtomBytes = 512;          // 128 rows x 4 scales = the scales of one instruction
constexpr int kNumThreads = 192;
constexpr int kAccCols = kPairBN;        // one accumulator
constexpr int kSfBase = kAccCols;
constexpr int kTmemCols = 512;
constexpr int kBand = 8;                 // 8 x 256 rows per scheduling band
// block-scaled instruction descriptor: e2m1 x e2m1, ue4m3 scales, K-major, N = 256, M = 256 over the pair
constexpr uint32_t kIdesc = (1u << 7) | (1u << 10) | (static_cast<uint32_t>(kPairBN >> 3) << 17) | (0u << 23) |
                            (static_cast<uint32_t>(kPairRows >> 4) << 24);

// K extent of a pipeline stage: BK bytes of packed K per row.  Operand arrival from L2 bounds this
// kernel, so eleven small stages (64-byte rows = 128 elements of K, 64-byte swizzle, two instructions)
// were tried against five large ones (128-byte rows, four instructions): on 8192^3 the small stages
// took 387 us against 282 us -- 64-byte row segments use the L2-to-SM path badly -- so 128 is the default.
template <int BK>
struct PCfg {
  static_assert(BK == 64 || BK == 128, "stage rows are 64 or 128 bytes");
  static constexpr int kBKBytes = BK;
  static constexpr int kBKElems = 2 * BK;
  static constexpr int kMmasPerStage = BK / kMmaKBytes;
  static constexpr int kStageA = kBM * BK;
  static constexpr int kStageB = (kPairBN / 2) * BK;
  static constexpr int kStageSFA = kMmasPerStage * kAtomBytes;
  static constexpr int kStageSFB = 2 * kMmasPerStage * kAtomBytes;   // both 128-column blocks
  static constexpr int kStageBytes = kStageA + kStageB + kStageSFA + kStageSFB;
  static_assert(kStageBytes % (BK * 8) == 0, "stages keep the alignment of the swizzled tiles");
  static constexpr int kStages = BK == 128 ? 5 : 11;
  static constexpr int kSfCols = 12 * kMmasPerStage;   // one set of scale columns: A (4 per instruction) + B (8)
  static_assert(kSfBase + 2 * kSfCols <= 512, "tensor memory budget");
};

template <int BK>
struct SmemTail {
  uint64_t full[PCfg<BK>::kStages];
  uint64_t empty[PCfg<BK>::kStages];
  uint64_t tmem_full;
  uint64_t tmem_empty;
  uint32_t tmem_base;
  int abort_flag;
};

template <int BK>
constexpr size_t smem_bytes() {
  return 1024 + static_cast<size_t>(PCfg<BK>::kStages) * PCfg<BK>::kStageBytes + sizeof(SmemTail<BK>);
}

__device__ __forceinline__ void tile_coords(int tile, int m_tiles, int n_tiles, int &m_tile, int &n_tile) {
  const int per_band = kBand * n_tiles;
  const int band = tile / per_band;
  const int in_band = tile - band * per_band;
  const int first_m = band * kBand;
  const int band_m = min(m_tiles - first_m, kBand);
  n_tile = in_band / band_m;
  m_tile = first_m + (in_band - n_tile * band_m);
}

template <int BK>
__global__ void __launch_bounds__(kNumThreads, 1)
    gemm_nvfp4_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                           const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb,
                           const PairParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *ring = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  using C = PCfg<BK>;
  constexpr int kStages = C::kStages, kStageBytes = C::kStageBytes, kStageA = C::kStageA, kStageB = C::kStageB;
  constexpr int kStageSFA = C::kStageSFA, kMmasPerStage = C::kMmasPerStage, kSfCols = C::kSfCols;
  constexpr int kBKBytes = C::kBKBytes, kBKElems = C::kBKElems;
  SmemTail<BK> &S = *reinterpret_cast<SmemTail<BK> *>(ring + static_cast<size_t>(kStages) * kStageBytes);

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair_id = blockIdx.x / 2;
  const int num_pairs = gridDim.x / 2;
  const int m_tiles = (p.M + kPairRows - 1) / kPairRows;
  const int n_tiles = (p.N + kPairBN - 1) / kPairBN;
  const int num_tiles = m_tiles * n_tiles;
  const int k_blocks = (p.K + kBKElems - 1) / kBKElems;
  volatile int *abort_flag = &S.abort_flag;

  if (threadIdx.x == 0) {
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
    prefetch_tensormap(&tmap_sfa);
    prefetch_tensormap(&tmap_sfb);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&S.full[s], 1);
      mbar_init(&S.empty[s], 1);
    }
    mbar_init(&S.tmem_full, 1);
    mbar_init(&S.tmem_empty, 8);   // four epilogue warps in each CTA
    S.abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc_pair(&S.tmem_base, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything is signalled on them
  tc_fence_after();
  const uint32_t tmem_base = S.tmem_base;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer (both CTAs)
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair_id; ok && tile < num_tiles; tile += num_pairs) {
        int m_tile, n_tile;
        tile_coords(tile, m_tiles, n_tiles, m_tile, n_tile);
        const int a_block = m_tile * 2 + static_cast<int>(rank);   // 128-row block of this CTA's A rows
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&S.empty[stage], phase ^ 1, abort_flag, p.status, kStatusProducerTimeout)) {
            ok = false;
            break;
          }
          uint8_t *sa = ring + static_cast<size_t>(stage) * kStageBytes;
          uint8_t *sb = sa + kStageA;
          uint8_t *ssfa = sb + kStageB;
          uint8_t *ssfb = ssfa + kStageSFA;
          const uint32_t leader_full = mapa_u32(smem_u32(&S.full[stage]), 0);
          // every box is transferred whole (out-of-range rows and atoms are zero-filled), so the byte
          // count is the same for every stage
          if (leader) mbar_arrive_expect_tx(&S.full[stage], 2 * kStageBytes);
          tma_load_2d_pair(sa, &tmap_a, leader_full, kb * kBKBytes, a_block * kBM);
          tma_load_2d_pair(sb, &tmap_b, leader_full, kb * kBKBytes, n_tile * kPairBN + static_cast<int>(rank) * kBM);
          tma_load_2d_pair(ssfa, &tmap_sfa, leader_full, 0, a_block * p.ncb + kMmasPerStage * kb);
          tma_load_2d_pair(ssfb, &tmap_sfb, leader_full, 0, (n_tile * 2) * p.ncb + kMmasPerStage * kb);
          tma_load_2d_pair(ssfb + kMmasPerStage * kAtomBytes, &tmap_sfb, leader_full, 0,
                           (n_tile * 2 + 1) * p.ncb + kMmasPerStage * kb);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer (leader only)
    // The K blocks of all tiles of this pair form one stream; the scale atoms of block i+1 are copied
    // to tensor memory (into the other of two column sets) before the instructions of block i issue.
    if (leader && elect_one()) {
      struct Pos {
        int tile, kb, stage, local;
        uint32_t phase;
      };
      auto advance = [&](Pos &q) {
        if (++q.kb == k_blocks) {
          q.kb = 0;
          q.tile += num_pairs;
          ++q.local;
        }
        if (++q.stage == kStages) {
          q.stage = 0;
          q.phase ^= 1;
        }
      };
      auto copy_scales = [&](const Pos &q, int buf) {
        const uint32_t sa = smem_u32(ring + static_cast<size_t>(q.stage) * kStageBytes);
        const uint32_t ssfa = sa + kStageA + kStageB;
        const uint32_t ssfb = ssfa + kStageSFA;
        const uint32_t sfa_t = tmem_base + kSfBase + buf * kSfCols;
        const uint32_t sfb_t = sfa_t + 4 * kMmasPerStage;
        const int atoms = min(kMmasPerStage, p.ncb - kMmasPerStage * q.kb);
        for (int k = 0; k < atoms; ++k) {
          tc_cp_32x128b_warpx4_pair(sfa_t + 4 * k, make_sf_atom_desc(ssfa + k * kAtomBytes));
          tc_cp_32x128b_warpx4_pair(sfb_t + 8 * k, make_sf_atom_desc(ssfb + k * kAtomBytes));
          tc_cp_32x128b_warpx4_pair(sfb_t + 8 * k + 4, make_sf_atom_desc(ssfb + (kMmasPerStage + k) * kAtomBytes));
        }
      };
      Pos pos{pair_id, 0, 0, 0, 0u};
      bool ok = pos.tile < num_tiles;
      if (ok) {
        ok = mbar_wait(&S.full[pos.stage], pos.phase, abort_flag, p.status, kStatusMmaTimeout);
        if (ok) {
          tc_fence_after();
          copy_scales(pos, 0);
        }
      }
      int n = 0;
      while (ok && pos.tile < num_tiles) {
        Pos nxt = pos;
        advance(nxt);
        if (nxt.tile < num_tiles) {
          if (!mbar_wait(&S.full[nxt.stage], nxt.phase, abort_flag, p.status, kStatusMmaTimeout)) {
            ok = false;
            break;
          }
          tc_fence_after();
          copy_scales(nxt, (n + 1) & 1);
        }
        if (pos.kb == 0) {
          if (!mbar_wait(&S.tmem_empty, (pos.local & 1) ^ 1, abort_flag, p.status, kStatusMmaTimeout)) {
            ok = false;
            break;
          }
          tc_fence_after();
        }
        const uint32_t sa = smem_u32(ring + static_cast<size_t>(pos.stage) * kStageBytes);
        const uint64_t da = kBKBytes == 128 ? make_kmajor_sw128_desc(sa) : make_kmajor_sw64_desc(sa);
        const uint64_t db = kBKBytes == 128 ? make_kmajor_sw128_desc(sa + kStageA) : make_kmajor_sw64_desc(sa + kStageA);
        const uint32_t sfa_t = tmem_base + kSfBase + (n & 1) * kSfCols;
        const uint32_t sfb_t = sfa_t + 4 * kMmasPerStage;
        const int atoms = min(kMmasPerStage, p.ncb - kMmasPerStage * pos.kb);
        for (int k = 0; k < atoms; ++k)
          mma_nvfp4_pair(tmem_base, da + static_cast<uint64_t>(k * (kMmaKBytes >> 4)),
                         db + static_cast<uint64_t>(k * (kMmaKBytes >> 4)), kIdesc, sfa_t + 4 * k, sfb_t + 8 * k,
                         (pos.kb | k) != 0 ? 1u : 0u);
        const uint32_t e = smem_u32(&S.empty[pos.stage]);
        tc_commit_pair(mapa_u32(e, 0));
        tc_commit_pair(mapa_u32(e, 1));
        if (pos.kb == k_blocks - 1) {
          const uint32_t f = smem_u32(&S.tmem_full);
          tc_commit_pair(mapa_u32(f, 0));
          tc_commit_pair(mapa_u32(f, 1));
        }
        pos = nxt;
        ++n;
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- epilogue (both CTAs, own 128 rows)
    const int quad = warp & 3;
    const int row_in_cta = quad * 32 + lane;
    const bool y_vec_ok = (p.N % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.y) & 15u) == 0);
    const float alpha = *p.alpha;
    int local = 0;
    for (int tile = pair_id; tile < num_tiles; tile += num_pairs, ++local) {
      int m_tile, n_tile;
      tile_coords(tile, m_tiles, n_tiles, m_tile, n_tile);
      const int row = m_tile * kPairRows + static_cast<int>(rank) * kBM + row_in_cta;
      const bool row_ok = row < p.M;
      const bool got = mbar_wait(&S.tmem_full, local & 1, abort_flag, p.status, kStatusEpilogueTimeout);
      if (!__all_sync(0xffffffffu, got)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
      __nv_bfloat16 *yrow = p.y + static_cast<size_t>(row) * p.N + n_tile * kPairBN;
      // drain the whole accumulator (scaled, packed to bf16) and hand it back before the stores
      uint32_t packed[kPairBN / 2];
#pragma unroll
      for (int c = 0; c < kPairBN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; j += 2)
          packed[c * 16 + j / 2] = pack_bf16x2(__uint_as_float(r[j]) * alpha, __uint_as_float(r[j + 1]) * alpha);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&S.tmem_empty), 0));
      if (row_ok) {
#pragma unroll
        for (int c = 0; c < kPairBN / 32; ++c) {
          const int cols_left = p.N - (n_tile * kPairBN + c * 32);
          __nv_bfloat16 *dst = yrow + c * 32;
          if (y_vec_ok && cols_left >= 32) {
            uint4 *d4 = reinterpret_cast<uint4 *>(dst);
#pragma unroll
            for (int j = 0; j < 4; ++j)
              __stcs(d4 + j, make_uint4(packed[c * 16 + 4 * j], packed[c * 16 + 4 * j + 1], packed[c * 16 + 4 * j + 2],
                                        packed[c * 16 + 4 * j + 3]));   // streaming: the output must not evict the operands from L2
          } else if (cols_left > 0) {
            uint16_t *d = reinterpret_cast<uint16_t *>(dst);
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < cols_left) d[j] = static_cast<uint16_t>(packed[c * 16 + j / 2] >> ((j & 1) * 16));
          }
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA frees tensor memory while the pair may still use it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

template <int BK>
int launch_bk(const void *xq, const void *wq, const void *x_scale, const void *w_scale, const PairParams &p,
              cudaStream_t st) {
  using C = PCfg<BK>;
  constexpr size_t kSmemBytes = smem_bytes<BK>();
  static_assert(kSmemBytes <= 232448, "shared memory budget exceeded");
  static std::atomic<int> max_pairs[64];   // zero-initialised; a racing first call computes the same value
  int dev = 0;
  if (int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
  if (dev < 0 || dev >= 64) return -1;

  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(kNumThreads, 1, 1);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = 1;

  if (max_pairs[dev] == 0) {
    if (int rc = check_cuda(cudaFuncSetAttribute(gemm_nvfp4_pair_kernel<BK>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 static_cast<int>(kSmemBytes)),
                            "cudaFuncSetAttribute(gemm_nvfp4_pair)"))
      return rc;
    cfg.gridDim = dim3(2 * (sm_count() / 2), 1, 1);
    int n = 0;
    cudaError_t e = cudaOccupancyMaxActiveClusters(&n, gemm_nvfp4_pair_kernel<BK>, &cfg);
    if (e != cudaSuccess || n <= 0) {
      cudaGetLastError();
      max_pairs[dev] = -1;
    } else {
      max_pairs[dev] = n;
    }
  }
  if (max_pairs[dev] < 0) return -1;

  const int64_t m_tiles = (static_cast<int64_t>(p.M) + kPairRows - 1) / kPairRows;
  const int64_t n_tiles = (static_cast<int64_t>(p.N) + kPairBN - 1) / kPairBN;
  const int64_t tiles = m_tiles * n_tiles;
  const int64_t mp = max_pairs[dev].load();
  const int pairs = static_cast<int>(tiles < mp ? tiles : mp);

  const int64_t kbytes = p.K / 2;
  const uint64_t a_blocks = (static_cast<uint64_t>(p.M) + kBM - 1) / kBM, b_blocks = (static_cast<uint64_t>(p.N) + kBM - 1) / kBM;
  CUtensorMap ta, tb, tsa, tsb;
  const CUtensorMapSwizzle swz = BK == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  if (int rc = make_tmap_2d_bytes(&ta, xq, kbytes, p.M, kbytes, BK, kBM, swz)) return rc;
  if (int rc = make_tmap_2d_bytes(&tb, wq, kbytes, p.N, kbytes, BK, kBM, swz)) return rc;
  // scale buffers as [atoms, 128 words]: a box holds the atoms of one K block of one 128-row block
  if (int rc = make_tmap_2d_u32(&tsa, x_scale, kAtomBytes / 4, a_blocks * p.ncb, kAtomBytes, kAtomBytes / 4, C::kMmasPerStage))
    return rc;
  if (int rc = make_tmap_2d_u32(&tsb, w_scale, kAtomBytes / 4, b_blocks * p.ncb, kAtomBytes, kAtomBytes / 4, C::kMmasPerStage))
    return rc;

  cfg.gridDim = dim3(2 * pairs, 1, 1);
  return check_cuda(cudaLaunchKernelEx(&cfg, gemm_nvfp4_pair_kernel<BK>, ta, tb, tsa, tsb, p), "f4f4bf16 pair launch");
}

}  // namespace

int launch_pair_kernel(const void *xq, const void *wq, const void *x_scale, const void *w_scale, const PairParams &p,
                       cudaStream_t st) {
  static const int bk = [] {
    const char *e = getenv("MSLK_B200_NVFP4_PAIR_BK");   // "64" | "128": tuning aid, default 128 (measured faster)
    return e && atoi(e) == 64 ? 64 : 128;
  }();
  return bk == 128 ? launch_bk<128>(xq, wq, x_scale, w_scale, p, st) : launch_bk<64>(xq, wq, x_scale, w_scale, p, st);
}

}  // namespace nvfp4_pair
}  // namespace mslk_b200
