// NVFP4 GEMM for sm_100a:  y = bf16(alpha * sum_blocks (sx * sw) * sum_16 x^ * w^)
//
// Operands are packed e2m1 (two per byte, K-major) with one ue4m3 scale per 16
// K-elements, stored in 512-byte atoms of 128 rows x 4 scales (the layout the
// quantizer writes).  The block-scaled tensor-core instruction
// tcgen05.mma.kind::mxf4nvf4.block_scale.scale_vec::4X consumes 128 x BN x 64 per
// issue: data tiles straight from 128-byte-swizzled shared memory (a TMA box of
// {128 bytes = 256 elements of K, rows}), scales from tensor memory, where one
// atom occupies 4 columns (row i + 32 j of the atom sits in lane i, column j, of
// every 32-lane quadrant).  tcgen05.cp (32x128b, replicated to the four
// quadrants) moves an atom from shared to tensor memory; it is issued by the MMA
// thread right before the instruction that uses it and is ordered with it.
//
// Pipeline and roles are those of the FP8 kernel (gemm_f8_rowwise.cu): TMA
// producer warp, single-thread MMA issuer, four epilogue warps, bounded waits.
// Per stage (256 K-elements): A 16 KB, B BN/128 x 16 KB, scale atoms 2 KB for A
// and BN/128 x 2 KB for B (plain bulk copies: four consecutive atoms of one
// 128-row block are contiguous in memory).
// Tensor memory: BN = 128 keeps two accumulators (epilogue overlaps the next
// tile); BN = 256 has room for one accumulator beside the scale columns.
#include "../../include/mslk_b200.h"
#include "common.cuh"
#include "gemm_f8_common.cuh"   // group tables and the tile scheduler shared with the FP8 kernels
#include "gemm_nvfp4_decode.h"
#include "gemm_nvfp4_pair.h"
#include "host.h"

#include <atomic>
#include <cstdlib>

namespace mslk_b200 {
namespace {

using gemm_f8::build_group_tables;
using gemm_f8::GemmParams;
using gemm_f8::kBandM;
using gemm_f8::kMaxGroups;
using gemm_f8::Scheduler;
using gemm_f8::Tile;

constexpr int kBM = 128;
constexpr int kBKBytes = 128;        // bytes of packed K per stage row
constexpr int kBKElems = 256;        // K elements per stage
constexpr int kMmaKBytes = 32;       // 64 K-elements per instruction
constexpr int kAtomBytes = 512;      // 128 rows x 4 scales
constexpr int kNumThreads = 192;

struct Fp4Params {
  const uint8_t *sfa;   // swizzled scales of A: [row blocks of 128][ncb] atoms
  const uint8_t *sfb;   // swizzled scales of B: [G][ceil(N/128)][ncb] atoms
  const float *alpha;   // device: one scalar (dense) or one per group
  __nv_bfloat16 *y;
  int *status;
  int M, N, K;          // M = stacked rows of all groups
  int ncb;              // scale atoms per 128-row block = ceil(K / 64), MXFP4 (one scale per 32): ceil(K / 128)
  // Grouped (stacked) problems: G weight blocks of N rows, group g owning m_sizes[g] consecutive rows
  // of X / Y.  The scale rows of every group start on a 128-row boundary of their own:
  // sfa_row_start[g] (a multiple of 128) is the first row of group g in the padded scale matrix.
  // Dense: G = 1, m_sizes = sfa_row_start = nullptr.
  const int64_t *m_sizes;
  const int32_t *end_offsets;      // alternative to m_sizes: int32 end offsets of the groups
  const int64_t *sfa_row_start;    // may be null: groups then follow each other, each padded to 128 rows
  int G;
  int alpha_per_group;
  // K-grouped problems (the "2D-2D" form: X [M, K], W [N, K], group g contracting the K range
  // (k_end_offsets[g-1], k_end_offsets[g]] into y[g] of a [G, M, N] output): int32 END offsets along K, multiples
  // of 32.  Every group's scales are a swizzled block of their own ([row blocks][atoms of that group]), the blocks
  // following each other.  Null for every other form.
  const int32_t *k_end_offsets;
  long long sfa_atoms, sfb_atoms;   // K-grouped: 512-byte atoms the two scale tensors hold (the kernel reads no further)
  int a_box_rows;       // rows of the A box: 128, or fewer for a dense problem with fewer rows (no out-of-range fill)
  int scale_mode;       // kScaleNvfp4 / kScaleMxfp4 / kScaleMxfp4_16 (common.cuh); ncb counts the atoms of that format
};

template <int BN>
struct Cfg {
  static constexpr int kNB = BN / 128;                     // 128-row blocks of B per tile
  static constexpr int kStageA = kBM * kBKBytes;
  static constexpr int kStageB = BN * kBKBytes;
  static constexpr int kStageSFA = 4 * kAtomBytes;
  static constexpr int kStageSFB = kNB * 4 * kAtomBytes;
  static constexpr int kStageBytes = kStageA + kStageB + kStageSFA + kStageSFB;
  static constexpr int kStages = BN == 128 ? 6 : 4;
  static constexpr int kAccStages = BN == 128 ? 2 : 1;
  static constexpr int kSfaCol = kAccStages * BN;          // first TMEM column of the scale area
  static constexpr int kSfCols = 16 + 16 * kNB;            // one set: A scales (16 columns) + B scales (16 * kNB)
  static_assert(kSfaCol + 2 * kSfCols <= 512, "two scale column sets must fit beside the accumulators");
  static constexpr int kTmemCols = 512;
  // block-scaled instruction descriptor: e2m1 x e2m1, ue4m3 scales, K-major, dense K = 64
  static constexpr uint32_t kIdesc = (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BN >> 3) << 17) | (0u << 23) |
                                     (static_cast<uint32_t>(kBM >> 4) << 24);
};

template <int BN>
struct SmemTail {
  uint64_t full[Cfg<BN>::kStages];
  uint64_t empty[Cfg<BN>::kStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int kgroup_reject;                // K-grouped: the scale tensors are too short for the offsets, every group yields zeros
  int row_start[kMaxGroups + 1];    // first stacked row of every group
  int tile_start[kMaxGroups + 1];   // first linear tile of every group
};

template <int BN>
constexpr size_t smem_bytes() {
  return 1024 + static_cast<size_t>(Cfg<BN>::kStages) * Cfg<BN>::kStageBytes + sizeof(SmemTail<BN>);
}

// Tile lookup of the epilogue warps as a real call: the scheduler's temporaries then do not share the
// register budget of the accumulator drain (128 packed registers for BN = 256).
__device__ __noinline__ bool epilogue_tile(const int *tile_start, const int *row_start, int G, int N, int n_tiles, int bn,
                                           int tile, int &g, int &row0, int &rows, int &n0) {
  Scheduler sched{tile_start, row_start, G, N, n_tiles, bn, kBM, kBandM, g};
  Tile t;
  if (!sched.get(tile, t)) return false;
  g = sched.g;
  row0 = t.row0;
  rows = t.rows;
  n0 = t.n0;
  return true;
}

// One tile of a K-grouped problem: tiles of a group are consecutive, columns fastest.  k_start / atom_start are the
// group tables (first K element and first scale atom per 128-row block of every group).
struct KTile {
  int g, m_tile, n_tile;
  int k0, kg;        // first K element of the group and its extent (0: empty group, the output is zero)
  int ncb, atom0;    // scale atoms per 128-row block of this group, and of all groups before it
};

__device__ __noinline__ bool kgroup_tile(const int *k_start, const int *atom_start, int reject, int G, int m_tiles,
                                         int n_tiles, int tile, KTile &t) {
  const int per_group = m_tiles * n_tiles;
  if (tile >= G * per_group) return false;
  t.g = tile / per_group;
  const int r = tile - t.g * per_group;
  t.m_tile = r / n_tiles;
  t.n_tile = r - t.m_tile * n_tiles;
  t.k0 = k_start[t.g];
  t.kg = k_start[t.g + 1] - t.k0;
  if (((t.k0 | t.kg) & 31) || reject) t.kg = 0;   // rejected (the prologue has recorded kStatusBadGroupOffset)
  t.atom0 = atom_start[t.g];
  t.ncb = atom_start[t.g + 1] - t.atom0;
  return true;
}

template <int BN, bool KG>
__global__ void __launch_bounds__(kNumThreads, 1)
    gemm_nvfp4_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const Fp4Params p) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *ring = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  SmemTail<BN> &S = *reinterpret_cast<SmemTail<BN> *>(ring + static_cast<size_t>(C::kStages) * C::kStageBytes);

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  const int n_tiles = (p.N + BN - 1) / BN;
  const int k_blocks = (p.K + kBKElems - 1) / kBKElems;
  const int n_row_blocks_b = (p.N + 127) / 128;
  volatile int *abort_flag = &S.abort_flag;

  if (threadIdx.x == 0) {
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&S.full[s], 1);
      mbar_init(&S.empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&S.tmem_full[a], 1);
      mbar_init(&S.tmem_empty[a], 4);
    }
    S.abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc(&S.tmem_base, C::kTmemCols);
    tmem_relinquish();
  }
  // everything above touched shared and tensor memory only: it may run under the tail of the previous kernel of the
  // stream; from here on global memory is read (group sizes, operands, scales) and written
  griddep_wait();
  griddep_launch_dependents();
  if (warp == 2) {
    GemmParams gp{};
    gp.m_sizes = p.m_sizes;
    gp.end_offsets = p.end_offsets;
    gp.G = p.G;
    gp.total_m = p.M;
    gp.group_m = p.M;   // dense: one group of all rows (only read when m_sizes is null)
    if constexpr (KG) {
      // the same prefix sums over the K extents: row_start = first K element of every group, tile_start = scale
      // atoms (of 4 scales per row) in front of it
      gp.end_offsets = p.k_end_offsets;
      gp.total_m = p.K;
      build_group_tables(gp, 1, p.scale_mode == kScaleMxfp4 ? 128 : 64, lane, S.row_start, S.tile_start);
      bool bad = false;
      for (int g = lane; g < p.G; g += 32) {
        const int e = p.k_end_offsets[g];
        bad |= (e & 31) != 0 || e < (g > 0 ? p.k_end_offsets[g - 1] : 0) || e > p.K;
      }
      __syncwarp();
      const long long atoms = S.tile_start[p.G];
      const bool too_short = atoms * ((p.M + kBM - 1) / kBM) > p.sfa_atoms || atoms * n_row_blocks_b > p.sfb_atoms;
      if (lane == 0) S.kgroup_reject = too_short ? 1 : 0;
      if ((bad || too_short) && blockIdx.x == 0) atomicOr(p.status, kStatusBadGroupOffset);
    } else {
      build_group_tables(gp, n_tiles, kBM, lane, S.row_start, S.tile_start);
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = S.tmem_base;
  const int m_tiles_kg = (p.M + kBM - 1) / kBM;
  const int num_tiles = KG ? p.G * m_tiles_kg * n_tiles : S.tile_start[p.G];
  Scheduler sched{S.tile_start, S.row_start, p.G, p.N, n_tiles, BN, kBM, kBandM, 0};

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (elect_one()) {  // one lane, chosen so that the compiler keeps the issue loop on the uniform datapath
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      Tile t;
      KTile kt;
      for (int tile = blockIdx.x; ok && (KG ? kgroup_tile(S.row_start, S.tile_start, S.kgroup_reject, p.G, m_tiles_kg, n_tiles, tile, kt)
                                            : sched.get(tile, t));
           tile += gridDim.x) {
        // per tile: rows of the two operand boxes, first packed K byte, K blocks, scale atoms per 128-row block
        // and the first atom of the tile's row block of A / of its first row block of B
        int n_tile, a_row, b_row, kbyte0, kbs, ncb;
        int64_t sfa_atom0, sfb_atom0;
        if constexpr (KG) {
          n_tile = kt.n_tile;
          a_row = kt.m_tile * kBM;
          b_row = n_tile * BN;
          kbyte0 = kt.k0 / 2;
          kbs = (kt.kg + kBKElems - 1) / kBKElems;
          ncb = kt.ncb;
          sfa_atom0 = static_cast<int64_t>(kt.atom0) * m_tiles_kg + static_cast<int64_t>(kt.m_tile) * ncb;
          sfb_atom0 = static_cast<int64_t>(kt.atom0) * n_row_blocks_b + static_cast<int64_t>(n_tile) * C::kNB * ncb;
        } else {
          const int g = sched.g;
          n_tile = t.n0 / BN;
          a_row = t.row0;
          b_row = t.wrow0;
          kbyte0 = 0;
          kbs = k_blocks;
          ncb = p.ncb;
          // 128-row block of this tile in the padded scale matrix of A, and of its columns in that of B
          // (without an explicit table the padded blocks of the groups are consecutive, so the first block
          // of group g is its first tile divided by the tiles per row block)
          const int64_t sfa_block = (p.sfa_row_start ? p.sfa_row_start[g] / kBM : S.tile_start[g] / n_tiles) +
                                    (t.row0 - S.row_start[g]) / kBM;
          sfa_atom0 = sfa_block * ncb;
          sfb_atom0 = (static_cast<int64_t>(g) * n_row_blocks_b + n_tile * C::kNB) * ncb;
        }
        int nb_live = 0;  // 128-row blocks of B that exist for this tile
        for (int b = 0; b < C::kNB; ++b) nb_live += (n_tile * C::kNB + b) < n_row_blocks_b ? 1 : 0;
        for (int kb = 0; kb < kbs; ++kb) {
          if (!mbar_wait(&S.empty[stage], phase ^ 1, abort_flag, p.status, kStatusProducerTimeout)) {
            ok = false;
            break;
          }
          uint8_t *sa = ring + static_cast<size_t>(stage) * C::kStageBytes;
          uint8_t *sb = sa + C::kStageA;
          uint8_t *ssfa = sb + C::kStageB;
          uint8_t *ssfb = ssfa + C::kStageSFA;
          // scale atoms (4 scales per row each: 64 K-elements, MXFP4 128) left in this K block of 256 elements
          const int apk = p.scale_mode == kScaleMxfp4 ? 2 : 4;
          const int atoms = min(apk, ncb - apk * kb);
          const uint32_t sf_bytes = static_cast<uint32_t>(atoms) * kAtomBytes;
          mbar_arrive_expect_tx(&S.full[stage], p.a_box_rows * kBKBytes + C::kStageB + sf_bytes * (1 + nb_live));
          tma_load_2d(sa, &tmap_a, &S.full[stage], kbyte0 + kb * kBKBytes, a_row);
          tma_load_2d(sb, &tmap_b, &S.full[stage], kbyte0 + kb * kBKBytes, b_row);
          bulk_load_1d(ssfa, p.sfa + static_cast<size_t>(sfa_atom0 + apk * kb) * kAtomBytes, sf_bytes, &S.full[stage]);
          for (int b = 0; b < nb_live; ++b)
            bulk_load_1d(ssfb + b * 4 * kAtomBytes,
                         p.sfb + static_cast<size_t>(sfb_atom0 + static_cast<int64_t>(b) * ncb + apk * kb) * kAtomBytes,
                         sf_bytes, &S.full[stage]);
          if (++stage == C::kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    // Per stage: the stage's scale atoms are copied to tensor memory (alternating between two sets of scale
    // columns, so a copy never lands on scales an earlier instruction still reads), then its instructions
    // are issued; copies and instructions execute in issue order.  The descriptors of a stage differ from
    // those of stage 0 only in the address field (16-byte units), so they are formed by one addition.
    if (elect_one()) {  // one lane, chosen so that the compiler keeps the issue loop on the uniform datapath
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      uint32_t n = 0;
      bool ok = true;
      const uint32_t ring0 = smem_u32(ring);
      const uint64_t da0 = make_kmajor_sw128_desc(ring0);
      const uint64_t db0 = make_kmajor_sw128_desc(ring0 + C::kStageA);
      const uint64_t dsfa0 = make_sf_atom_desc(ring0 + C::kStageA + C::kStageB);
      const uint64_t dsfb0 = make_sf_atom_desc(ring0 + C::kStageA + C::kStageB + C::kStageSFA);
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++local) {
        const int acc = local % C::kAccStages;
        const uint32_t acc_phase = (local / C::kAccStages) & 1;
        if (!mbar_wait(&S.tmem_empty[acc], acc_phase ^ 1, abort_flag, p.status, kStatusMmaTimeout)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        int kbs = k_blocks, k_len = p.K, ncb = p.ncb;
        if constexpr (KG) {
          KTile kt;
          kgroup_tile(S.row_start, S.tile_start, S.kgroup_reject, p.G, m_tiles_kg, n_tiles, tile, kt);
          k_len = kt.kg;
          kbs = (kt.kg + kBKElems - 1) / kBKElems;
          ncb = kt.ncb;
        }
        for (int kb = 0; kb < kbs; ++kb, ++n) {
          if (!mbar_wait(&S.full[stage], phase, abort_flag, p.status, kStatusMmaTimeout)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t soff = static_cast<uint64_t>((static_cast<uint32_t>(stage) * C::kStageBytes) >> 4);
          const uint64_t da = da0 + soff, db = db0 + soff, dsfa = dsfa0 + soff, dsfb = dsfb0 + soff;
          const uint32_t sfa_t = tmem_base + C::kSfaCol + (n & 1u) * C::kSfCols;
          const uint32_t sfb_t = sfa_t + 16;
          if (p.scale_mode == kScaleMxfp4) {
            // one scale per 32 K-elements: an atom holds the scales of TWO instructions, which pick their two bytes
            // of the scale column through the scale-id fields of the descriptor
            const int mmas = min(4, (k_len - kb * kBKElems + 63) / 64);
            const int atoms = (mmas + 1) / 2;
            if (mmas == 4) {
#pragma unroll
              for (int a = 0; a < 2; ++a) {
                tc_cp_32x128b_warpx4(sfa_t + 4 * a, dsfa + static_cast<uint64_t>(a * (kAtomBytes >> 4)));
#pragma unroll
                for (int b = 0; b < C::kNB; ++b)
                  tc_cp_32x128b_warpx4(sfb_t + 4 * C::kNB * a + 4 * b,
                                       dsfb + static_cast<uint64_t>((b * 4 + a) * (kAtomBytes >> 4)));
              }
#pragma unroll
              for (int k = 0; k < 4; ++k)
                mma_mxf4_2x(d_tmem, da + static_cast<uint64_t>(k * (kMmaKBytes >> 4)),
                            db + static_cast<uint64_t>(k * (kMmaKBytes >> 4)),
                            C::kIdesc | kIdescScaleE8M0 | idesc_scale_ids((k & 1) * 2), sfa_t + 4 * (k >> 1),
                            sfb_t + 4 * C::kNB * (k >> 1), (kb | k) != 0 ? 1u : 0u);
            } else {
              for (int a = 0; a < atoms; ++a) {
                tc_cp_32x128b_warpx4(sfa_t + 4 * a, dsfa + static_cast<uint64_t>(a * (kAtomBytes >> 4)));
#pragma unroll
                for (int b = 0; b < C::kNB; ++b)
                  tc_cp_32x128b_warpx4(sfb_t + 4 * C::kNB * a + 4 * b,
                                       dsfb + static_cast<uint64_t>((b * 4 + a) * (kAtomBytes >> 4)));
              }
              for (int k = 0; k < mmas; ++k)
                mma_mxf4_2x(d_tmem, da + static_cast<uint64_t>(k * (kMmaKBytes >> 4)),
                            db + static_cast<uint64_t>(k * (kMmaKBytes >> 4)),
                            C::kIdesc | kIdescScaleE8M0 | idesc_scale_ids((k & 1) * 2), sfa_t + 4 * (k >> 1),
                            sfb_t + 4 * C::kNB * (k >> 1), (kb | k) != 0 ? 1u : 0u);
            }
          } else {
          const uint32_t idesc = C::kIdesc | (p.scale_mode == kScaleMxfp4_16 ? kIdescScaleE8M0 : 0u);
          const int atoms = min(4, ncb - 4 * kb);
          if (atoms == 4) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              tc_cp_32x128b_warpx4(sfa_t + 4 * k, dsfa + static_cast<uint64_t>(k * (kAtomBytes >> 4)));
#pragma unroll
              for (int b = 0; b < C::kNB; ++b)
                tc_cp_32x128b_warpx4(sfb_t + 4 * C::kNB * k + 4 * b,
                                     dsfb + static_cast<uint64_t>((b * 4 + k) * (kAtomBytes >> 4)));
            }
#pragma unroll
            for (int k = 0; k < 4; ++k)
              mma_nvfp4(d_tmem, da + static_cast<uint64_t>(k * (kMmaKBytes >> 4)),
                        db + static_cast<uint64_t>(k * (kMmaKBytes >> 4)), idesc, sfa_t + 4 * k,
                        sfb_t + 4 * C::kNB * k, (kb | k) != 0 ? 1u : 0u);
          } else {
            for (int k = 0; k < atoms; ++k) {
              tc_cp_32x128b_warpx4(sfa_t + 4 * k, dsfa + static_cast<uint64_t>(k * (kAtomBytes >> 4)));
#pragma unroll
              for (int b = 0; b < C::kNB; ++b)
                tc_cp_32x128b_warpx4(sfb_t + 4 * C::kNB * k + 4 * b,
                                     dsfb + static_cast<uint64_t>((b * 4 + k) * (kAtomBytes >> 4)));
            }
            for (int k = 0; k < atoms; ++k)
              mma_nvfp4(d_tmem, da + static_cast<uint64_t>(k * (kMmaKBytes >> 4)),
                        db + static_cast<uint64_t>(k * (kMmaKBytes >> 4)), idesc, sfa_t + 4 * k,
                        sfb_t + 4 * C::kNB * k, (kb | k) != 0 ? 1u : 0u);
          }
          }
          tc_commit(&S.empty[stage]);
          if (++stage == C::kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        tc_commit(&S.tmem_full[acc]);
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    const bool y_vec_ok = (p.N % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.y) & 15u) == 0);
    int local = 0;
    int g = 0, row0, rows, n0;
    KTile kt;
    kt.kg = 1;
    for (int tile = blockIdx.x;
         KG ? kgroup_tile(S.row_start, S.tile_start, S.kgroup_reject, p.G, m_tiles_kg, n_tiles, tile, kt)
            : epilogue_tile(S.tile_start, S.row_start, p.G, p.N, n_tiles, BN, tile, g, row0, rows, n0);
         tile += gridDim.x, ++local) {
      if constexpr (KG) {
        g = kt.g;
        row0 = kt.g * p.M + kt.m_tile * kBM;   // y is [G, M, N]
        rows = min(kBM, p.M - kt.m_tile * kBM);
        n0 = kt.n_tile * BN;
      }
      const bool empty_group = KG && kt.kg == 0;   // nothing was accumulated: the tile is zero
      const int n_tile = n0 / BN;
      const float alpha = p.alpha ? p.alpha[p.alpha_per_group ? g : 0] : 1.0f;   // the MX formats have no global scale
      const int acc = local % C::kAccStages;
      const uint32_t acc_phase = (local / C::kAccStages) & 1;
      const int row = row0 + row_in_tile;
      const bool row_ok = row_in_tile < rows;
      const bool got = mbar_wait(&S.tmem_full[acc], acc_phase, abort_flag, p.status, kStatusEpilogueTimeout);
      if (!__all_sync(0xffffffffu, got)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + static_cast<uint32_t>(acc * BN) + (static_cast<uint32_t>(quad * 32) << 16);
      __nv_bfloat16 *yrow = p.y + static_cast<size_t>(row) * p.N + n_tile * BN;
      // Drain the whole accumulator into registers (already scaled and packed to bf16) and hand
      // it back to the MMA warp BEFORE the global stores: with a single accumulator the next
      // tile's main loop would otherwise wait for the store phase as well.
      uint32_t packed[BN / 2];
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; j += 2)
          packed[c * 16 + j / 2] =
              empty_group ? 0u : pack_bf16x2(__uint_as_float(r[j]) * alpha, __uint_as_float(r[j + 1]) * alpha);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&S.tmem_empty[acc]);
      if (row_ok) {
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
          const int cols_left = p.N - (n_tile * BN + c * 32);
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

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <int BN, bool KG = false>
int launch(const CUtensorMap &ta, const CUtensorMap &tb, const Fp4Params &p, int grid, cudaStream_t st) {
  static std::atomic<bool> attr_set[64];   // zero-initialised; two first calls may both set the (idempotent) attribute
  int dev = 0;
  if (int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
  constexpr size_t smem = smem_bytes<BN>();
  static_assert(smem <= 232448, "shared memory budget exceeded");
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (int rc = check_cuda(cudaFuncSetAttribute(gemm_nvfp4_kernel<BN, KG>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 static_cast<int>(smem)),
                            "cudaFuncSetAttribute(gemm_nvfp4)"))
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
  return check_cuda(cudaLaunchKernelEx(&cfg, gemm_nvfp4_kernel<BN, KG>, ta, tb, p), "f4f4bf16 launch");
}

}  // namespace
}  // namespace mslk_b200

namespace mslk_b200 {
namespace {

int run_fp4(const char *name, const void *xq, const void *wq, const void *x_scale, const void *w_scale,
            const float *global_scale, void *y, const int64_t *m_sizes, const int32_t *end_offsets,
            const int64_t *sfa_row_start, int64_t G, int64_t M, int64_t N, int64_t K, cudaStream_t st,
            void *scratch = nullptr, size_t scratch_size = 0, int scale_mode = kScaleNvfp4) {
  const bool grouped = m_sizes || end_offsets;
  const bool mx = scale_mode != kScaleNvfp4;
  if (M < 0 || N < 0 || K < 0 || G < 1) return fail(1, "%s: bad shape", name);
  if (M == 0 || N == 0) return 0;
  if (G > kMaxGroups) return fail(1, "%s: at most %d groups are supported (got %lld)", name, kMaxGroups, (long long)G);
  if (!y) return fail(1, "%s: null output pointer", name);
  if (K == 0) return check_cuda(cudaMemsetAsync(y, 0, static_cast<size_t>(M) * N * 2, st), "memset");
  if (!xq || !wq || !x_scale || !w_scale || (!global_scale && !mx)) return fail(1, "%s: null pointer argument", name);
  if (K % 32 != 0) return fail(1, "%s: K (%lld) must be a multiple of 32 (16-byte rows of packed e2m1)", name, (long long)K);
  if (M > 0x7fffff00LL || G * N > 0x7fffff00LL || K > 0x7fffff00LL) return fail(1, "%s: dimension too large", name);
  if ((reinterpret_cast<uintptr_t>(x_scale) | reinterpret_cast<uintptr_t>(w_scale)) & 15u)
    return fail(1, "%s: scale tensors must be 16-byte aligned", name);
  int *status = device_status_ptr();
  if (!status) return 2;

  Fp4Params p;
  p.sfa = static_cast<const uint8_t *>(x_scale);
  p.sfb = static_cast<const uint8_t *>(w_scale);
  p.alpha = global_scale;
  p.y = static_cast<__nv_bfloat16 *>(y);
  p.status = status;
  p.M = static_cast<int>(M);
  p.N = static_cast<int>(N);
  p.K = static_cast<int>(K);
  p.ncb = static_cast<int>(scale_mode == kScaleMxfp4 ? (K + 127) / 128 : (K + 63) / 64);
  p.scale_mode = scale_mode;
  p.m_sizes = m_sizes;
  p.end_offsets = end_offsets;
  p.sfa_row_start = sfa_row_start;
  p.k_end_offsets = nullptr;
  p.G = static_cast<int>(G);
  p.alpha_per_group = (grouped && global_scale) ? 1 : 0;
  p.a_box_rows = (!grouped && M < kBM) ? static_cast<int>((M + 7) / 8 * 8) : kBM;

  const int sms = sm_count();
  // CTA pairs (256 x 256 tiles, a third less shared-memory traffic per flop) for dense problems with
  // enough such tiles to occupy every pair of SMs
  static const int force = [] {
    const char *e = getenv("MSLK_B200_NVFP4_KERNEL");  // "1cta" | "2cta": tuning aid, default = heuristic
    return !e ? 0 : (e[0] == '2' ? 2 : 1);
  }();
  // few tokens: weight-streaming kernel (weights on the 128 accumulator rows, two CTAs per SM, K split
  // over CTAs when the caller passed scratch memory)
  // (65..128 tokens: when the general kernel's 128-column tiles need more than one wave -- M = 128,
  // N = 28672: 30.7 against 36.4 us -- or when K is long and is split inside clusters -- M = 128, (N, K) =
  // (4096, 14336): 18.1 against 29.7 us, M = 100, (8192, 28672): 32.1 against 54.0, (8192, 8192): 18.5 against
  // 19.9; with K = 4096 the general kernel wins, (4096, 4096): 12.5 against 19.2 us)
  const int64_t w_blocks = (N + 127) / 128;
  if (!grouped && force == 0 && N >= 128 &&
      (M <= 64 || (M <= nvfp4_decode::kMaxTokens && (w_blocks > sms || (2 * w_blocks <= sms && K >= 8192)))))
    return nvfp4_decode::launch_decode_kernel(xq, wq, x_scale, w_scale, global_scale, y, status, M, N, K, scratch,
                                              scratch_size, st, scale_mode);
  const int64_t pair_tiles = ((M + 255) / 256) * ((N + 255) / 256);
  // (few-token shapes stay on one CTA per tile: a 256-row pair tile would be mostly padding; grouped problems take
  // pairs when their groups average at least 128 rows and there are few enough groups for the kernel's tables)
  const bool pair_ok = grouped ? (G <= nvfp4_pair::kPairMaxGroups && M / G >= 128) : M > 128;
  if (force == 2 || (force == 0 && pair_ok && pair_tiles >= sms / 2)) {
    nvfp4_pair::PairParams pp{};
    pp.alpha = global_scale;
    pp.y = static_cast<__nv_bfloat16 *>(y);
    pp.status = status;
    pp.M = static_cast<int>(M);
    pp.N = static_cast<int>(N);
    pp.K = static_cast<int>(K);
    pp.ncb = p.ncb;
    pp.scale_mode = scale_mode;
    pp.m_sizes = m_sizes;
    pp.end_offsets = end_offsets;
    pp.sfa_row_start = sfa_row_start;
    pp.G = static_cast<int>(G);
    pp.alpha_per_group = p.alpha_per_group;
    const int rc = nvfp4_pair::launch_pair_kernel(xq, wq, x_scale, w_scale, pp, st);
    if (rc >= 0) return rc;   // -1: pairs unavailable, fall through to one CTA per tile
  }
  const int64_t m_tiles = (M + kBM - 1) / kBM + (grouped ? G : 0);   // upper bound for ragged groups
  // 256-wide tiles halve the A traffic per flop but hold one accumulator only; use them when
  // there are enough tiles to fill the device, 128-wide (double-buffered) otherwise
  int bn = (m_tiles * ((N + 255) / 256) >= 2 * sms) ? 256 : 128;
  CUtensorMap ta, tb;
  if (int rc = make_tmap_2d_bytes(&ta, xq, K / 2, M, K / 2, kBKBytes, p.a_box_rows, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  if (int rc = make_tmap_2d_bytes(&tb, wq, K / 2, G * N, K / 2, kBKBytes, bn, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  const int64_t tiles = m_tiles * ((N + bn - 1) / bn);
  const int grid = static_cast<int>(tiles < sms ? tiles : sms);
  return bn == 256 ? launch<256>(ta, tb, p, grid, st) : launch<128>(ta, tb, p, grid, st);
}

// K-grouped ("2D-2D") form on the one-CTA kernel: G problems of M x N, group g contracting its own K range.
int run_fp4_kgrouped(const char *name, const void *xq, const void *wq, const void *x_scale, const void *w_scale,
                     const float *global_scale, void *y, const int32_t *k_end_offsets, int64_t G, int64_t M, int64_t N,
                     int64_t K, int scale_mode, size_t x_scale_bytes, size_t w_scale_bytes, cudaStream_t st) {
  const bool mx = scale_mode != kScaleNvfp4;
  if (M < 0 || N < 0 || K < 0 || G < 1) return fail(1, "%s: bad shape", name);
  if (M == 0 || N == 0) return 0;
  if (G > kMaxGroups) return fail(1, "%s: at most %d groups are supported (got %lld)", name, kMaxGroups, (long long)G);
  if (!y) return fail(1, "%s: null output pointer", name);
  if (K == 0) return check_cuda(cudaMemsetAsync(y, 0, static_cast<size_t>(G) * M * N * 2, st), "memset");
  if (!xq || !wq || !x_scale || !w_scale || !k_end_offsets || (!global_scale && !mx))
    return fail(1, "%s: null pointer argument", name);
  if (K % 32 != 0) return fail(1, "%s: K (%lld) must be a multiple of 32 (16-byte rows of packed e2m1)", name, (long long)K);
  if (G * M > 0x7fffff00LL || N > 0x7fffff00LL || K > 0x7fffff00LL) return fail(1, "%s: dimension too large", name);
  if ((reinterpret_cast<uintptr_t>(x_scale) | reinterpret_cast<uintptr_t>(w_scale)) & 15u)
    return fail(1, "%s: scale tensors must be 16-byte aligned", name);
  int *status = device_status_ptr();
  if (!status) return 2;
  Fp4Params p{};
  p.sfa = static_cast<const uint8_t *>(x_scale);
  p.sfb = static_cast<const uint8_t *>(w_scale);
  p.alpha = global_scale;
  p.y = static_cast<__nv_bfloat16 *>(y);
  p.status = status;
  p.M = static_cast<int>(M);
  p.N = static_cast<int>(N);
  p.K = static_cast<int>(K);
  p.scale_mode = scale_mode;
  p.k_end_offsets = k_end_offsets;
  p.sfa_atoms = static_cast<long long>(x_scale_bytes / kAtomBytes);
  p.sfb_atoms = static_cast<long long>(w_scale_bytes / kAtomBytes);
  p.G = static_cast<int>(G);
  p.alpha_per_group = global_scale ? 1 : 0;
  p.a_box_rows = M < kBM ? static_cast<int>((M + 7) / 8 * 8) : kBM;
  const int sms = sm_count();
  static const int force = [] {
    const char *e = getenv("MSLK_B200_NVFP4_KERNEL");  // "1cta" | "2cta": tuning aid, default = heuristic
    return !e ? 0 : (e[0] == '2' ? 2 : 1);
  }();
  // CTA pairs (256 x 256 tiles) when there are enough such tiles to occupy every pair of SMs
  const int64_t pair_tiles = G * ((M + 255) / 256) * ((N + 255) / 256);
  if (force == 2 || (force == 0 && M > 128 && G <= nvfp4_pair::kPairMaxGroups && pair_tiles >= sms / 2)) {
    nvfp4_pair::PairParams pp{};
    pp.alpha = global_scale;
    pp.y = static_cast<__nv_bfloat16 *>(y);
    pp.status = status;
    pp.M = static_cast<int>(M);
    pp.N = static_cast<int>(N);
    pp.K = static_cast<int>(K);
    pp.scale_mode = scale_mode;
    pp.k_end_offsets = k_end_offsets;
    pp.sfa_atoms = p.sfa_atoms;
    pp.sfb_atoms = p.sfb_atoms;
    pp.G = static_cast<int>(G);
    pp.alpha_per_group = p.alpha_per_group;
    if (G <= nvfp4_pair::kPairMaxGroups) {
      const int rc = nvfp4_pair::launch_pair_kernel(xq, wq, x_scale, w_scale, pp, st);
      if (rc >= 0) return rc;   // -1: pairs unavailable, fall through to one CTA per tile
    }
  }
  const int64_t m_tiles = (M + kBM - 1) / kBM;
  const int bn = (G * m_tiles * ((N + 255) / 256) >= 2 * sms) ? 256 : 128;
  CUtensorMap ta, tb;
  if (int rc = make_tmap_2d_bytes(&ta, xq, K / 2, M, K / 2, kBKBytes, p.a_box_rows, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  if (int rc = make_tmap_2d_bytes(&tb, wq, K / 2, N, K / 2, kBKBytes, bn, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  const int64_t tiles = G * m_tiles * ((N + bn - 1) / bn);
  const int grid = static_cast<int>(tiles < sms ? tiles : sms);
  return bn == 256 ? launch<256, true>(ta, tb, p, grid, st) : launch<128, true>(ta, tb, p, grid, st);
}

}  // namespace
}  // namespace mslk_b200

MSLK_API int mslk_b200_f4f4bf16_grouped_mm_2d2d(const void *xq, const void *wq, const void *x_scale, const void *w_scale,
                                                const int32_t *k_end_offsets, const float *global_scale, int64_t G,
                                                int64_t M, int64_t N, int64_t total_K, int block_size,
                                                size_t x_scale_bytes, size_t w_scale_bytes, void *y, void *stream) {
  using namespace mslk_b200;
  clear_error();
  const char *name = "f4f4bf16_grouped_mm (2D-2D)";
  int mode = kScaleNvfp4;
  if (!global_scale) {
    if (block_size == 32) mode = kScaleMxfp4;
    else if (block_size == 16) mode = kScaleMxfp4_16;
    else return fail(1, "%s: block size must be 32 or 16 (got %d)", name, block_size);
  }
  return run_fp4_kgrouped(name, xq, wq, x_scale, w_scale, global_scale, y, k_end_offsets, G, M, N, total_K, mode,
                          x_scale_bytes, w_scale_bytes, static_cast<cudaStream_t>(stream));
}

MSLK_API int mslk_b200_f4f4bf16(const void *xq, const void *wq, const void *x_scale, const void *w_scale,
                                const float *global_scale, void *y, int64_t M, int64_t N, int64_t K, void *stream) {
  using namespace mslk_b200;
  clear_error();
  return run_fp4("f4f4bf16", xq, wq, x_scale, w_scale, global_scale, y, nullptr, nullptr, nullptr, 1, M, N, K,
                 static_cast<cudaStream_t>(stream));
}

MSLK_API int mslk_b200_debug_nvfp4_pair_timers(unsigned long long *dev_counters) {
  mslk_b200::nvfp4_pair::set_pipe_timers(dev_counters);
  return 0;
}

MSLK_API size_t mslk_b200_f4f4bf16_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  using namespace mslk_b200;
  if (M < 1 || N < 128 || K < 32) return 0;
  return nvfp4_decode::scratch_bytes(M, N, K, sm_count());
}

MSLK_API int mslk_b200_f4f4bf16_ws(const void *xq, const void *wq, const void *x_scale, const void *w_scale,
                                   const float *global_scale, void *y, int64_t M, int64_t N, int64_t K,
                                   void *workspace, size_t workspace_bytes, void *stream) {
  using namespace mslk_b200;
  clear_error();
  return run_fp4("f4f4bf16", xq, wq, x_scale, w_scale, global_scale, y, nullptr, nullptr, nullptr, 1, M, N, K,
                 static_cast<cudaStream_t>(stream), workspace, workspace_bytes);
}

// ---- MXFP4 forms (e8m0 scales, no global scale): block_size 32 = OCP MXFP4, 16 = e8m0 scales per 16 elements
static int mx_mode(const char *name, int block_size, int *mode) {
  if (block_size == 32) *mode = mslk_b200::kScaleMxfp4;
  else if (block_size == 16) *mode = mslk_b200::kScaleMxfp4_16;
  else return mslk_b200::fail(1, "%s: block size must be 32 or 16 (got %d)", name, block_size);
  return 0;
}

MSLK_API int mslk_b200_f4f4bf16_mx(const void *xq, const void *wq, const void *x_scale, const void *w_scale, void *y,
                                   int64_t M, int64_t N, int64_t K, int block_size, void *stream) {
  using namespace mslk_b200;
  clear_error();
  int mode;
  if (int rc = mx_mode("f4f4bf16 (MXFP4)", block_size, &mode)) return rc;
  return run_fp4("f4f4bf16 (MXFP4)", xq, wq, x_scale, w_scale, nullptr, y, nullptr, nullptr, nullptr, 1, M, N, K,
                 static_cast<cudaStream_t>(stream), nullptr, 0, mode);
}

MSLK_API int mslk_b200_f4f4bf16_grouped_stacked_mx(const void *xq, const void *wq, const void *x_scale,
                                                   const void *w_scale, const int64_t *M_sizes,
                                                   const int64_t *starting_row_after_padding, int64_t G,
                                                   int64_t total_M, int64_t N, int64_t K, int block_size, void *y,
                                                   void *stream) {
  using namespace mslk_b200;
  clear_error();
  const char *name = "f4f4bf16_grouped_stacked (MXFP4)";
  int mode;
  if (int rc = mx_mode(name, block_size, &mode)) return rc;
  if (!M_sizes) return fail(1, "%s: M_sizes is null", name);
  return run_fp4(name, xq, wq, x_scale, w_scale, nullptr, y, M_sizes, nullptr, starting_row_after_padding, G, total_M, N, K,
                 static_cast<cudaStream_t>(stream), nullptr, 0, mode);
}

MSLK_API int mslk_b200_f4f4bf16_grouped_mm_mx(const void *xq, const void *wq, const void *x_scale, const void *w_scale,
                                              const int32_t *offsets, int64_t G, int64_t total_M, int64_t N, int64_t K,
                                              int block_size, void *y, void *stream) {
  using namespace mslk_b200;
  clear_error();
  const char *name = "f4f4bf16_grouped_mm (MXFP4)";
  int mode;
  if (int rc = mx_mode(name, block_size, &mode)) return rc;
  if (!offsets) return fail(1, "%s: offsets is null", name);
  return run_fp4(name, xq, wq, x_scale, w_scale, nullptr, y, nullptr, offsets, nullptr, G, total_M, N, K,
                 static_cast<cudaStream_t>(stream), nullptr, 0, mode);
}

MSLK_API int mslk_b200_f4f4bf16_grouped_stacked(const void *xq, const void *wq, const void *x_scale,
                                                const void *w_scale, const int64_t *M_sizes,
                                                const float *global_scale,
                                                const int64_t *starting_row_after_padding, int64_t G,
                                                int64_t total_M, int64_t N, int64_t K, void *y, void *stream) {
  using namespace mslk_b200;
  clear_error();
  const char *name = "f4f4bf16_grouped_stacked";
  if (!M_sizes) return fail(1, "%s: M_sizes is null", name);
  return run_fp4(name, xq, wq, x_scale, w_scale, global_scale, y, M_sizes, nullptr, starting_row_after_padding, G, total_M,
                 N, K, static_cast<cudaStream_t>(stream));
}

MSLK_API int mslk_b200_f4f4bf16_grouped_mm(const void *xq, const void *wq, const void *x_scale, const void *w_scale,
                                           const int32_t *offsets, const float *global_scale, int64_t G,
                                           int64_t total_M, int64_t N, int64_t K, void *y, void *stream) {
  using namespace mslk_b200;
  clear_error();
  const char *name = "f4f4bf16_grouped_mm";
  if (!offsets) return fail(1, "%s: offsets is null", name);
  return run_fp4(name, xq, wq, x_scale, w_scale, global_scale, y, nullptr, offsets, nullptr, G, total_M, N, K,
                 static_cast<cudaStream_t>(stream));
}
