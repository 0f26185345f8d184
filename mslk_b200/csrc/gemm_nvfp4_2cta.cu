// NVFP4 GEMM on CTA pairs (tcgen05 cta_group::2, block-scaled) for sm_100a; dense problems and grouped (stacked)
// ones, whose tiles come from the device-side scheduler over the per-group row counts (gemm_f8_common.cuh).
//
// Two CTAs on neighbouring SMs compute one 256 x 256 output tile with 256 x 256 x 64 instructions.
// Each CTA loads its own 128 rows of A and its own 128 of the 256 rows of B: 38 KB per SM and K block
// (256 elements of K) instead of the 54 KB of the one-CTA kernel with 256-column tiles.  Scale factors:
// each CTA needs, in its own tensor memory, the A scales of its own 128 rows and the B scales of ALL 256
// columns; both CTAs therefore fetch both B scale blocks themselves (4 KB per K block; no load is
// multicast).  Scale atoms travel as TMA boxes of {512 bytes, atoms of one stage} over a 2-D view of the scale
// buffer, so that, like the operand tiles, they can signal the leader's barrier from either CTA.
//
//   CTA rank 0 ("leader")                              CTA rank 1
//   warp 0  producer: own empty[s] -> 5 TMA loads into own smem, bytes counted on the LEADER's full[s]
//           (L2 prefetches of the boxes 2..16 K blocks ahead were tried: 247 us against 219 us on 8192^3)
//   warp 1  MMA issuer: per stage, tcgen05.cp of the stage's scale atoms (pair-wide: every CTA copies its
//           own atoms into its own tensor memory; two alternating sets of scale columns, so the copies of
//           stage i+1 never overwrite scales the instructions of stage i still read), then the four
//           pair-wide MMAs; commits to both CTAs' barriers
//                                                       (idle; takes part in TMEM alloc)
//   warps 2..9 epilogue on the CTA's own 128 accumulator rows: two warps per 32-lane quadrant, each draining
//           four 32-column chunks of the accumulator into registers -- first the chunks the NEXT tile's accumulator
//           overlaps (tiles alternate between two accumulators that share 96 columns), handing the accumulator
//           back as soon as those have landed -- then staging 32 x 64 bf16 slabs in swizzled shared memory for
//           TMA stores (128-byte row segments); all sixteen warps of the pair arrive on the leader's tmem_empty
//           barrier
//
// Waits are bounded as everywhere else (common.cuh); cluster-wide hardware barriers only at start-up
// and teardown, reached on every path.
#include "gemm_nvfp4_pair.h"

#include "common.cuh"
#include "gemm_f8_common.cuh"

#include <algorithm>
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
constexpr int kNumEpilogueWarps = 8;
constexpr int kNumThreads = 64 + 32 * kNumEpilogueWarps;
constexpr int kAccCols = kPairBN;        // columns of an accumulator
constexpr int kTmemCols = 512;
// block-scaled instruction descriptor: e2m1 x e2m1, ue4m3 scales, K-major, N = 256, M = 256 over the pair
constexpr uint32_t kIdesc = (1u << 7) | (1u << 10) | (static_cast<uint32_t>(kPairBN >> 3) << 17) | (0u << 23) |
                            (static_cast<uint32_t>(kPairRows >> 4) << 24);

// A pipeline stage holds 128 bytes of packed K per row (256 elements, four instructions).  Stages of 64-byte
// rows (64-byte swizzle, eleven of them) were measured slower: 387 us against 282 us on 8192^3.
constexpr int kBKBytes = 128;
constexpr int kBKElems = 256;
constexpr int kMmasPerStage = kBKBytes / kMmaKBytes;
constexpr int kStageA = kBM * kBKBytes;
constexpr int kStageB = (kPairBN / 2) * kBKBytes;
constexpr int kStageSFA = kMmasPerStage * kAtomBytes;
constexpr int kStageSFB = 2 * kMmasPerStage * kAtomBytes;   // both 128-column blocks
constexpr int kStageBytes = kStageA + kStageB + kStageSFA + kStageSFB;
static_assert(kStageBytes % 1024 == 0, "stages keep the alignment of the swizzled tiles");
constexpr int kStages = 5;
constexpr int kSfCols = 12 * kMmasPerStage;   // one set of scale columns: A (4 per instruction) + B (8)
// Tensor memory: the two sets of scale columns sit at the top; two accumulators of 256 columns share the 416 columns
// below them, [0, 256) and [160, 416), tiles alternating between them.  They overlap in [160, 256): the epilogue of a
// tile drains those 96 columns first and hands the accumulator back at once, so the next tile's instructions wait for
// 3/8 of a drain instead of a whole one while the other 160 columns are read under them.
constexpr int kSfBase = kTmemCols - 2 * kSfCols;
constexpr int kAcc1Base = kSfBase - kAccCols;
constexpr int kChunkCols = 32;                              // columns of one tensor-memory load
static_assert(kAcc1Base >= 0 && kAcc1Base % kChunkCols == 0 && (kAccCols - kAcc1Base) == 3 * kChunkCols,
              "the epilogue's chunk order assumes an overlap of three 32-column chunks");

struct SmemTail {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmem_full;
  uint64_t tmem_empty;
  uint64_t early_done;   // this CTA's epilogue warps: the overlapped chunks of the current tile are in registers
  uint32_t tmem_base;
  int abort_flag;
  int row_start[kPairMaxGroups + 2];    // first stacked row of every group
  int tile_start[kPairMaxGroups + 2];   // first linear tile of every group
  int blk_start[kPairMaxGroups + 2];    // first 128-row block of every group in the padded scale matrix of A
};

constexpr int kOutCols = 64;                        // columns of one staged output slab (128-byte rows)
constexpr int kOutSlabBytes = 32 * kOutCols * 2;    // 32 rows x 64 bf16
constexpr int kOutStageBytes = kNumEpilogueWarps * kOutSlabBytes;
constexpr size_t kSmemBytes = 1024 + static_cast<size_t>(kStages) * kStageBytes + kOutStageBytes + sizeof(SmemTail);
static_assert(kSmemBytes <= 232448, "shared memory budget exceeded");

__device__ __forceinline__ long long clock_now() {
  long long t;
  asm volatile("mov.u64 %0, %clock64;" : "=l"(t));
  return t;
}

// What the three roles need to know about one 256 x 256 tile.
struct PairTile {
  int g;                   // group (alpha index)
  int row0, rows, n0;      // first output row (stacked), rows that belong to the group, first output column
  int a_row, b_row;        // row coordinates of the tile in the tensor maps of A and B
  int kbyte0;              // first packed K byte of the tile's K range in both maps
  int k_len, kbs, ncb;     // K elements, K blocks of 256, scale atoms per 128-row block of that range
  int sfa_atom, sfb_atom;  // atom index of the tile's first 128-row block of A / of B at its first K block
};

// K-grouped problems: tiles of a group are consecutive, columns fastest; k_start / atom_start are the group tables
// (first K element and first scale atom per 128-row block of every group).
__device__ __noinline__ bool pair_kgroup_tile(const int *k_start, const int *atom_start, int reject, int G, int M, int N,
                                              int tile, PairTile &t) {
  const int m_tiles = (M + kPairRows - 1) / kPairRows, n_tiles = (N + kPairBN - 1) / kPairBN;
  const int per_group = m_tiles * n_tiles;
  if (tile >= G * per_group) return false;
  t.g = tile / per_group;
  const int r = tile - t.g * per_group;
  const int m_tile = r / n_tiles, n_tile = r - m_tile * n_tiles;
  const int k0 = k_start[t.g];
  int kg = k_start[t.g + 1] - k0;
  if (((k0 | kg) & 31) || reject) kg = 0;   // rejected (the prologue has recorded kStatusBadGroupOffset): zeros
  const int atom0 = atom_start[t.g];
  t.ncb = atom_start[t.g + 1] - atom0;
  t.row0 = t.g * M + m_tile * kPairRows;     // y is [G, M, N]
  t.rows = min(kPairRows, M - m_tile * kPairRows);
  t.n0 = n_tile * kPairBN;
  t.a_row = m_tile * kPairRows;
  t.b_row = t.n0;
  t.kbyte0 = k0 / 2;
  t.k_len = kg;
  t.kbs = (kg + kBKElems - 1) / kBKElems;
  t.sfa_atom = atom0 * ((M + kBM - 1) / kBM) + m_tile * 2 * t.ncb;
  t.sfb_atom = atom0 * ((N + kBM - 1) / kBM) + n_tile * 2 * t.ncb;
  return true;
}

template <bool KG>
__global__ void __launch_bounds__(kNumThreads, 1)
    gemm_nvfp4_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                           const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb,
                           const __grid_constant__ CUtensorMap tmap_y, const PairParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *ring = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t *out_stage = ring + static_cast<size_t>(kStages) * kStageBytes;   // 1024-byte aligned slabs
  SmemTail &S = *reinterpret_cast<SmemTail *>(out_stage + kOutStageBytes);

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair_id = blockIdx.x / 2;
  const int num_pairs = gridDim.x / 2;
  const int n_tiles = (p.N + kPairBN - 1) / kPairBN;
  const int n_row_blocks_b = (p.N + kBM - 1) / kBM;
  const int k_blocks = (p.K + kBKElems - 1) / kBKElems;
  volatile int *abort_flag = &S.abort_flag;
  const bool timed = p.timers != nullptr;

  if (threadIdx.x == 0) {
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
    prefetch_tensormap(&tmap_sfa);
    prefetch_tensormap(&tmap_sfb);
    prefetch_tensormap(&tmap_y);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&S.full[s], 1);
      mbar_init(&S.empty[s], 1);
    }
    mbar_init(&S.tmem_full, 1);
    mbar_init(&S.tmem_empty, 2 * kNumEpilogueWarps);   // the epilogue warps of both CTAs
    mbar_init(&S.early_done, kNumEpilogueWarps);
    S.abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc_pair(&S.tmem_base, kTmemCols);
    tmem_relinquish_pair();
  }
  // everything above touched shared and tensor memory only: it may run under the tail of the previous kernel of the
  // stream; from here on global memory is read (group sizes, operands, scales) and written
  griddep_wait();
  griddep_launch_dependents();
  if (warp == 2) {
    // group tables: rows and tiles as in the FP8 kernels, plus the 128-row scale blocks in front of every group
    gemm_f8::GemmParams gp{};
    gp.m_sizes = p.m_sizes;
    gp.end_offsets = p.end_offsets;
    gp.G = p.G;
    gp.total_m = p.M;
    gp.group_m = p.M;   // dense: one group of all rows (only read when both size arrays are null)
    if constexpr (KG) {
      // the same prefix sums over the K extents: row_start = first K element of every group, tile_start = scale
      // atoms (of 4 scales per row) in front of it
      gp.end_offsets = p.k_end_offsets;
      gp.total_m = p.K;
      gemm_f8::build_group_tables(gp, 1, p.scale_mode == kScaleMxfp4 ? 128 : 64, lane, S.row_start, S.tile_start);
      bool bad = false;
      for (int g = lane; g < p.G; g += 32) {
        const int e = p.k_end_offsets[g];
        bad |= (e & 31) != 0 || e < (g > 0 ? p.k_end_offsets[g - 1] : 0) || e > p.K;
      }
      __syncwarp();
      const long long atoms = S.tile_start[p.G];
      const bool too_short = atoms * ((p.M + kBM - 1) / kBM) > p.sfa_atoms || atoms * n_row_blocks_b > p.sfb_atoms;
      if (lane == 0) S.blk_start[0] = too_short ? 1 : 0;   // reject flag (the block table is not used in this mode)
      if ((bad || too_short) && blockIdx.x == 0) atomicOr(p.status, kStatusBadGroupOffset);
    } else {
      gemm_f8::build_group_tables(gp, n_tiles, kPairRows, lane, S.row_start, S.tile_start);
      __syncwarp();
      if (lane == 0) {
        int blocks = 0;
        for (int g = 0; g < p.G; ++g) {
          S.blk_start[g] = p.sfa_row_start ? static_cast<int>(p.sfa_row_start[g] / kBM) : blocks;
          blocks += (S.row_start[g + 1] - S.row_start[g] + kBM - 1) / kBM;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything is signalled on them
  tc_fence_after();
  const uint32_t tmem_base = S.tmem_base;
  const int num_tiles = KG ? p.G * ((p.M + kPairRows - 1) / kPairRows) * n_tiles : S.tile_start[p.G];
  gemm_f8::Scheduler sched{S.tile_start, S.row_start, p.G, p.N, n_tiles, kPairBN, kPairRows, p.band, 0};
  PairTile t;
  auto next_tile = [&](int tile) -> bool {
    if constexpr (KG) {
      return pair_kgroup_tile(S.row_start, S.tile_start, S.blk_start[0], p.G, p.M, p.N, tile, t);
    } else {
      gemm_f8::Tile st;
      if (!sched.get(tile, st)) return false;
      const int g = sched.g;
      t.g = g;
      t.row0 = st.row0;
      t.rows = st.rows;
      t.n0 = st.n0;
      t.a_row = st.row0;
      t.b_row = st.wrow0;
      t.kbyte0 = 0;
      t.k_len = p.K;
      t.kbs = k_blocks;
      t.ncb = p.ncb;
      // 128-row block of the tile's rows in the padded scale matrix of A, and of its columns in that of B
      t.sfa_atom = (S.blk_start[g] + (st.row0 - S.row_start[g]) / kBM) * p.ncb;
      t.sfb_atom = (g * n_row_blocks_b + st.n0 / kBM) * p.ncb;
      return true;
    }
  };

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer (both CTAs)
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      long long t_empty = 0;
      const int apk = p.scale_mode == kScaleMxfp4 ? 2 : kMmasPerStage;   // scale atoms per K block and 128-row block
      for (int tile = pair_id; ok && next_tile(tile); tile += num_pairs) {
        const int a_row = t.a_row + static_cast<int>(rank) * kBM;        // first of this CTA's 128 rows of A
        const int b_row = t.b_row + static_cast<int>(rank) * kBM;        // ... and of B
        const int sfa_atom = t.sfa_atom + static_cast<int>(rank) * t.ncb;   // this CTA's 128-row block of A's scales
        const int sfb_atom = t.sfb_atom, ncb = t.ncb, kbyte0 = t.kbyte0, kbs = t.kbs;
        for (int kb = 0; kb < kbs; ++kb) {
          const long long t0 = timed ? clock_now() : 0;
          if (!mbar_wait(&S.empty[stage], phase ^ 1, abort_flag, p.status, kStatusProducerTimeout)) {
            ok = false;
            break;
          }
          if (timed) t_empty += clock_now() - t0;
          uint8_t *sa = ring + static_cast<size_t>(stage) * kStageBytes;
          uint8_t *sb = sa + kStageA;
          uint8_t *ssfa = sb + kStageB;
          uint8_t *ssfb = ssfa + kStageSFA;
          const uint32_t leader_full = mapa_u32(smem_u32(&S.full[stage]), 0);
          // every box is transferred whole (out-of-range rows and atoms are zero-filled), so the byte
          // count is the same for every stage
          // (the scale boxes hold apk atoms per 128-row block: four, or two when one scale covers 32 elements)
          if (leader) mbar_arrive_expect_tx(&S.full[stage], 2 * (kStageA + kStageB + 3 * apk * kAtomBytes));
          tma_load_2d_pair(sa, &tmap_a, leader_full, kbyte0 + kb * kBKBytes, a_row);
          tma_load_2d_pair(sb, &tmap_b, leader_full, kbyte0 + kb * kBKBytes, b_row);
          tma_load_2d_pair(ssfa, &tmap_sfa, leader_full, 0, sfa_atom + apk * kb);
          tma_load_2d_pair(ssfb, &tmap_sfb, leader_full, 0, sfb_atom + apk * kb);
          tma_load_2d_pair(ssfb + kMmasPerStage * kAtomBytes, &tmap_sfb, leader_full, 0, sfb_atom + ncb + apk * kb);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (timed && leader) atomicAdd(p.timers + 3, static_cast<unsigned long long>(t_empty));
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer (leader only)
    if (leader && elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      uint32_t n = 0;     // K blocks issued so far: selects the set of scale columns
      bool ok = true;
      long long t_full = 0, t_acc = 0;
      const long long t_begin = timed ? clock_now() : 0;
      // the descriptors of a stage differ from those of stage 0 only in the address field (bits 0..13, in
      // 16-byte units); shared memory is smaller than 2^18 bytes, so adding to the low word never carries out
      const uint32_t ring0 = smem_u32(ring);
      const uint64_t da0 = make_kmajor_sw128_desc(ring0);
      const uint64_t db0 = make_kmajor_sw128_desc(ring0 + kStageA);
      const uint64_t dsfa0 = make_sf_atom_desc(ring0 + kStageA + kStageB);
      const uint64_t dsfb0 = make_sf_atom_desc(ring0 + kStageA + kStageB + kStageSFA);
      for (int tile = pair_id; ok && tile < num_tiles; tile += num_pairs, ++local) {
        {
          const long long t0 = timed ? clock_now() : 0;
          if (!mbar_wait(&S.tmem_empty, (local & 1) ^ 1, abort_flag, p.status, kStatusMmaTimeout)) {
            ok = false;
            break;
          }
          if (timed) t_acc += clock_now() - t0;
        }
        tc_fence_after();
        const uint32_t acc_t = tmem_base + ((local & 1) ? kAcc1Base : 0);
        int kbs = k_blocks, k_len = p.K, ncb = p.ncb;
        if constexpr (KG) {
          next_tile(tile);
          kbs = t.kbs;
          k_len = t.k_len;
          ncb = t.ncb;
        }
        for (int kb = 0; kb < kbs; ++kb, ++n) {
          const long long t0 = timed ? clock_now() : 0;
          if (!mbar_wait(&S.full[stage], phase, abort_flag, p.status, kStatusMmaTimeout)) {
            ok = false;
            break;
          }
          if (timed) t_full += clock_now() - t0;
          tc_fence_after();
          const uint64_t soff = static_cast<uint64_t>((static_cast<uint32_t>(stage) * kStageBytes) >> 4);
          const uint64_t da = da0 + soff, db = db0 + soff, dsfa = dsfa0 + soff, dsfb = dsfb0 + soff;
          const uint32_t sfa_t = tmem_base + kSfBase + (n & 1u) * kSfCols;
          const uint32_t sfb_t = sfa_t + 4 * kMmasPerStage;
          if (p.scale_mode == kScaleMxfp4) {
            // one scale per 32 K-elements: an atom holds the scales of TWO instructions, which pick their two bytes
            // of the scale column through the scale-id fields of the descriptor
            const int mmas = min(kMmasPerStage, (k_len - kb * kBKElems + 63) / 64);
            const int atoms = (mmas + 1) / 2;
            if (mmas == kMmasPerStage) {
#pragma unroll
              for (int a = 0; a < 2; ++a) {
                tc_cp_32x128b_warpx4_pair(sfa_t + 4 * a, dsfa + static_cast<uint64_t>(a * (kAtomBytes >> 4)));
                tc_cp_32x128b_warpx4_pair(sfb_t + 8 * a, dsfb + static_cast<uint64_t>(a * (kAtomBytes >> 4)));
                tc_cp_32x128b_warpx4_pair(sfb_t + 8 * a + 4,
                                          dsfb + static_cast<uint64_t>((kMmasPerStage + a) * (kAtomBytes >> 4)));
              }
#pragma unroll
              for (int k = 0; k < kMmasPerStage; ++k)
                mma_mxf4_2x_pair(acc_t, da + static_cast<uint64_t>(k * (kMmaKBytes >> 4)),
                                 db + static_cast<uint64_t>(k * (kMmaKBytes >> 4)),
                                 kIdesc | kIdescScaleE8M0 | idesc_scale_ids((k & 1) * 2), sfa_t + 4 * (k >> 1),
                                 sfb_t + 8 * (k >> 1), (kb | k) != 0 ? 1u : 0u);
            } else {
              for (int a = 0; a < atoms; ++a) {
                tc_cp_32x128b_warpx4_pair(sfa_t + 4 * a, dsfa + static_cast<uint64_t>(a * (kAtomBytes >> 4)));
                tc_cp_32x128b_warpx4_pair(sfb_t + 8 * a, dsfb + static_cast<uint64_t>(a * (kAtomBytes >> 4)));
                tc_cp_32x128b_warpx4_pair(sfb_t + 8 * a + 4,
                                          dsfb + static_cast<uint64_t>((kMmasPerStage + a) * (kAtomBytes >> 4)));
              }
              for (int k = 0; k < mmas; ++k)
                mma_mxf4_2x_pair(acc_t, da + static_cast<uint64_t>(k * (kMmaKBytes >> 4)),
                                 db + static_cast<uint64_t>(k * (kMmaKBytes >> 4)),
                                 kIdesc | kIdescScaleE8M0 | idesc_scale_ids((k & 1) * 2), sfa_t + 4 * (k >> 1),
                                 sfb_t + 8 * (k >> 1), (kb | k) != 0 ? 1u : 0u);
            }
            const uint32_t e = smem_u32(&S.empty[stage]);
            tc_commit_pair(mapa_u32(e, 0));
            tc_commit_pair(mapa_u32(e, 1));
            if (++stage == kStages) {
              stage = 0;
              phase ^= 1;
            }
            continue;
          }
          const uint32_t idesc = kIdesc | (p.scale_mode == kScaleMxfp4_16 ? kIdescScaleE8M0 : 0u);
          const int atoms = min(kMmasPerStage, ncb - kMmasPerStage * kb);
          if (atoms == kMmasPerStage) {
#pragma unroll
            for (int k = 0; k < kMmasPerStage; ++k) {
              tc_cp_32x128b_warpx4_pair(sfa_t + 4 * k, dsfa + static_cast<uint64_t>(k * (kAtomBytes >> 4)));
              tc_cp_32x128b_warpx4_pair(sfb_t + 8 * k, dsfb + static_cast<uint64_t>(k * (kAtomBytes >> 4)));
              tc_cp_32x128b_warpx4_pair(sfb_t + 8 * k + 4,
                                        dsfb + static_cast<uint64_t>((kMmasPerStage + k) * (kAtomBytes >> 4)));
            }
#pragma unroll
            for (int k = 0; k < kMmasPerStage; ++k)
              mma_nvfp4_pair(acc_t, da + static_cast<uint64_t>(k * (kMmaKBytes >> 4)),
                             db + static_cast<uint64_t>(k * (kMmaKBytes >> 4)), idesc, sfa_t + 4 * k, sfb_t + 8 * k,
                             (kb | k) != 0 ? 1u : 0u);
          } else {
            for (int k = 0; k < atoms; ++k) {
              tc_cp_32x128b_warpx4_pair(sfa_t + 4 * k, dsfa + static_cast<uint64_t>(k * (kAtomBytes >> 4)));
              tc_cp_32x128b_warpx4_pair(sfb_t + 8 * k, dsfb + static_cast<uint64_t>(k * (kAtomBytes >> 4)));
              tc_cp_32x128b_warpx4_pair(sfb_t + 8 * k + 4,
                                        dsfb + static_cast<uint64_t>((kMmasPerStage + k) * (kAtomBytes >> 4)));
            }
            for (int k = 0; k < atoms; ++k)
              mma_nvfp4_pair(acc_t, da + static_cast<uint64_t>(k * (kMmaKBytes >> 4)),
                             db + static_cast<uint64_t>(k * (kMmaKBytes >> 4)), idesc, sfa_t + 4 * k, sfb_t + 8 * k,
                             (kb | k) != 0 ? 1u : 0u);
          }
          const uint32_t e = smem_u32(&S.empty[stage]);
          tc_commit_pair(mapa_u32(e, 0));
          tc_commit_pair(mapa_u32(e, 1));
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        const uint32_t f = smem_u32(&S.tmem_full);
        tc_commit_pair(mapa_u32(f, 0));
        tc_commit_pair(mapa_u32(f, 1));
      }
      if (timed) {
        atomicAdd(p.timers + 0, static_cast<unsigned long long>(t_full));
        atomicAdd(p.timers + 1, static_cast<unsigned long long>(t_acc));
        atomicAdd(p.timers + 2, static_cast<unsigned long long>(clock_now() - t_begin));
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- epilogue (both CTAs, own 128 rows)
    const int quad = warp & 3;                 // tensor-memory lanes this warp may read: 32 * (warp % 4) ...
    const int half = (warp - 2) >> 2;          // the two warps of a quadrant
    uint8_t *buf = out_stage + (warp - 2) * kOutSlabBytes;
    int local = 0;
    for (int tile = pair_id; next_tile(tile); tile += num_pairs, ++local) {
      const float alpha = p.alpha ? p.alpha[p.alpha_per_group ? t.g : 0] : 1.0f;   // the MX formats have no global scale
      const bool empty_group = KG && t.k_len == 0;   // nothing was accumulated: the tile is zero
      const int slab0 = static_cast<int>(rank) * kBM + quad * 32;   // first row of this warp's slab inside the tile
      const int row0 = t.row0 + slab0;
      const int slab_rows = min(32, t.rows - slab0);                // rows of the slab that belong to the tile's group (<= 0: none)
      // This warp's two 64-column slabs (as 32-column chunks of the accumulator) and which of its four chunks the
      // next tile's accumulator overlaps.  Accumulator 0 is overlapped in its chunks 5..7, accumulator 1 in 0..2:
      //   accumulator 0: warp A slabs {6,7} (both early), {0,1};  warp B slabs {4,5} (5 early), {2,3}
      //   accumulator 1: warp A slabs {0,1} (both early), {6,7};  warp B slabs {2,3} (2 early), {4,5}
      const int acc = local & 1;
      const int slab_a = acc ? (half ? 2 : 0) : (half ? 4 : 6);     // first chunk of the slab with the early chunks
      const int slab_b = acc ? (half ? 4 : 6) : (half ? 2 : 0);
      const bool early0 = half == 0 || acc == 1, early1 = half == 0 || acc == 0;
      const long long te0 = timed ? clock_now() : 0;
      const bool got = mbar_wait(&S.tmem_full, local & 1, abort_flag, p.status, kStatusEpilogueTimeout);
      if (!__all_sync(0xffffffffu, got)) break;
      tc_fence_after();
      const long long te1 = timed ? clock_now() : 0;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(acc ? kAcc1Base : 0);
      const uint32_t ta = taddr + static_cast<uint32_t>(slab_a * kChunkCols), tb = taddr + static_cast<uint32_t>(slab_b * kChunkCols);
      // the overlapped chunks first; the accumulator goes back as soon as they have landed, the rest is read while
      // the next tile's instructions already run; only then scale and pack (two fp32 registers become one packed pair)
      uint32_t r0[32], r1[32], r2[32], r3[32];
      if (early0) tmem_ld_32x32(ta, r0);
      if (early1) tmem_ld_32x32(ta + kChunkCols, r1);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive_cluster(mapa_u32(smem_u32(&S.tmem_empty), 0));
        mbar_arrive(&S.early_done);
      }
      const long long te2 = timed ? clock_now() : 0;
      // the other chunks are read only once every warp of this CTA has its overlapped chunks: tensor-memory reads
      // are served in order, and a fast warp's remaining chunks would otherwise hold up a slow warp's early ones
      const bool all_early = mbar_wait(&S.early_done, local & 1, abort_flag, p.status, kStatusEpilogueTimeout);
      if (!__all_sync(0xffffffffu, all_early)) break;
      if (!early0) tmem_ld_32x32(ta, r0);
      if (!early1) tmem_ld_32x32(ta + kChunkCols, r1);
      tmem_ld_32x32(tb, r2);
      tmem_ld_32x32(tb + kChunkCols, r3);
      tmem_ld_wait();
      if (timed && leader && warp == 2 && lane == 0) {
        atomicAdd(p.timers + 4, static_cast<unsigned long long>(te2 - te1));   // accumulator ready -> handed back
        atomicAdd(p.timers + 5, static_cast<unsigned long long>(te1 - te0));   // waiting for the accumulator
        atomicAdd(p.timers + 6, static_cast<unsigned long long>(clock_now() - te2));   // the rest of the drain
      }
      uint32_t packed[64];
      auto pack = [&](const uint32_t (&r)[32], int c) {
#pragma unroll
        for (int j = 0; j < 32; j += 2)
          packed[c * 16 + j / 2] =
              empty_group ? 0u : pack_bf16x2(__uint_as_float(r[j]) * alpha, __uint_as_float(r[j + 1]) * alpha);
      };
      pack(r0, 0);
      pack(r1, 1);
      pack(r2, 2);
      pack(r3, 3);
      if (p.tma_store && slab_rows == 32) {
#pragma unroll
        for (int s2 = 0; s2 < 2; ++s2) {
          const int col = t.n0 + (s2 ? slab_b : slab_a) * kChunkCols;
          if (col >= p.N) continue;                   // slab entirely outside the matrix (warp-uniform)
          if (lane == 0) tma_store_wait_read<0>();   // the store that last read this buffer is done with it
          __syncwarp();
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const int chunk = q ^ (lane & 7);          // 128-byte swizzle: 16-byte chunk index xor row
            *reinterpret_cast<uint4 *>(buf + lane * 128 + chunk * 16) =
                make_uint4(packed[s2 * 32 + 4 * q], packed[s2 * 32 + 4 * q + 1], packed[s2 * 32 + 4 * q + 2],
                           packed[s2 * 32 + 4 * q + 3]);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tmap_y, buf, col, row0);   // columns past the matrix are clipped
            tma_store_commit();
          }
        }
      } else if (lane < slab_rows) {
        // ragged slab (the group or the matrix ends inside it) or unaligned output: rows of this group only
        __nv_bfloat16 *yrow = p.y + static_cast<size_t>(row0 + lane) * p.N;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int col = t.n0 + ((c < 2 ? slab_a : slab_b) + (c & 1)) * kChunkCols;
          const int cols_left = p.N - col;
          uint16_t *d = reinterpret_cast<uint16_t *>(yrow + col);
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j < cols_left) d[j] = static_cast<uint16_t>(packed[c * 16 + j / 2] >> ((j & 1) * 16));
        }
      }
    }
    if (lane == 0) tma_store_wait<0>();   // every staged slab has been written out before the CTA leaves
    __syncwarp();
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

std::atomic<unsigned long long *> g_timers{nullptr};

}  // namespace

void set_pipe_timers(unsigned long long *dev_counters) { g_timers.store(dev_counters); }

template <bool KG>
int launch_pair_kernel_t(const void *xq, const void *wq, const void *x_scale, const void *w_scale, const PairParams &p,
                         cudaStream_t st) {
  static std::atomic<int> max_pairs[64];   // zero-initialised; a racing first call computes the same value
  int dev = 0;
  if (int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
  if (dev < 0 || dev >= 64) return -1;

  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[2];
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
    if (int rc = check_cuda(cudaFuncSetAttribute(gemm_nvfp4_pair_kernel<KG>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 static_cast<int>(kSmemBytes)),
                            "cudaFuncSetAttribute(gemm_nvfp4_pair)"))
      return rc;
    cfg.gridDim = dim3(2 * (sm_count() / 2), 1, 1);
    int n = 0;
    cudaError_t e = cudaOccupancyMaxActiveClusters(&n, gemm_nvfp4_pair_kernel<KG>, &cfg);
    if (e != cudaSuccess || n <= 0) {
      cudaGetLastError();
      max_pairs[dev] = -1;
    } else {
      max_pairs[dev] = n;
    }
  }
  if (max_pairs[dev] < 0) return -1;

  const bool grouped = p.m_sizes || p.end_offsets;
  if (p.G < 1 || p.G > kPairMaxGroups) return -1;
  // upper bound of the 256-row blocks: one ragged block per group (K-grouped: every group has all of them)
  const int64_t m_tiles = KG ? static_cast<int64_t>(p.G) * ((static_cast<int64_t>(p.M) + kPairRows - 1) / kPairRows)
                             : (static_cast<int64_t>(p.M) + kPairRows - 1) / kPairRows + (grouped ? p.G : 0);
  const int64_t n_tiles = (static_cast<int64_t>(p.N) + kPairBN - 1) / kPairBN;
  const int64_t tiles = m_tiles * n_tiles;
  const int64_t mp = max_pairs[dev].load();
  const int pairs = static_cast<int>(tiles < mp ? tiles : mp);

  const int64_t kbytes = p.K / 2;
  // 128-row blocks of the padded scale matrices: A's groups are padded one by one (the stacked quantizer's buffer
  // holds M + 127 G rows), B holds G blocks of roundup(N, 128) rows
  const uint64_t a_blocks = grouped ? (static_cast<uint64_t>(p.M) + 127ull * p.G) / kBM : (static_cast<uint64_t>(p.M) + kBM - 1) / kBM;
  const uint64_t b_blocks = static_cast<uint64_t>(p.G) * ((static_cast<uint64_t>(p.N) + kBM - 1) / kBM);
  // K-grouped: both operands are plain [rows, K] matrices, the scale tensors are as long as the caller says
  const uint64_t b_rows = KG ? static_cast<uint64_t>(p.N) : static_cast<uint64_t>(p.G) * p.N;
  const uint64_t a_atoms = KG ? static_cast<uint64_t>(p.sfa_atoms) : a_blocks * p.ncb;
  const uint64_t b_atoms = KG ? static_cast<uint64_t>(p.sfb_atoms) : b_blocks * p.ncb;
  const uint64_t y_rows = KG ? static_cast<uint64_t>(p.G) * p.M : static_cast<uint64_t>(p.M);
  CUtensorMap ta, tb, tsa, tsb;
  if (int rc = make_tmap_2d_bytes(&ta, xq, kbytes, p.M, kbytes, kBKBytes, kBM, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  if (int rc = make_tmap_2d_bytes(&tb, wq, kbytes, b_rows, kbytes, kBKBytes, kBM, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  // scale buffers as [atoms, 128 words]: a box holds the atoms of one K block of one 128-row block
  const uint32_t apk = p.scale_mode == kScaleMxfp4 ? 2 : kMmasPerStage;   // scale atoms of one K block
  if (int rc = make_tmap_2d_u32(&tsa, x_scale, kAtomBytes / 4, a_atoms, kAtomBytes, kAtomBytes / 4, apk)) return rc;
  if (int rc = make_tmap_2d_u32(&tsb, w_scale, kAtomBytes / 4, b_atoms, kAtomBytes, kAtomBytes / 4, apk)) return rc;

  PairParams q = p;
  // TMA stores need a 16-byte aligned base and row pitch; otherwise the epilogue stores element by element
  CUtensorMap ty;
  q.tma_store = ((reinterpret_cast<uintptr_t>(p.y) & 15u) == 0 && p.N % 8 == 0) ? 1 : 0;
  if (q.tma_store) {
    if (int rc = make_tmap_2d_bf16(&ty, p.y, p.N, y_rows, static_cast<uint64_t>(p.N) * 2, kOutCols, 32, CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  } else {
    ty = ta;   // never dereferenced
  }
  // Tiles of a band of `band` 256-row blocks run column by column.  All pairs advance through K together, so a wave
  // of P pairs touches (band + P / band) slabs of 256 rows (packed data + scales); while that fits the ~45 MB of L2
  // a kernel can count on, the band's rows of A stay resident between waves and B is read once per band: take the
  // tallest such band, else the squarest wave (8).
  {
    const double slab = static_cast<double>(kPairRows) * (kbytes + kbytes / 8), budget = 45.0 * (1 << 20), P = static_cast<double>(pairs);
    int64_t best = 0;
    for (int64_t b2 = std::min<int64_t>(8, m_tiles); b2 <= m_tiles; ++b2)
      if ((b2 + P / b2) * slab <= budget) best = b2;
    q.band = static_cast<int>(best && !grouped ? best : 8);   // grouped: the groups are short, bands of 8 blocks
  }
  q.timers = g_timers.load();
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.numAttrs = 1 + pdl_attribute(&attr[1]);   // the prologue may overlap the tail of the previous kernel of the stream
  return check_cuda(cudaLaunchKernelEx(&cfg, gemm_nvfp4_pair_kernel<KG>, ta, tb, tsa, tsb, ty, q), "f4f4bf16 pair launch");
}

int launch_pair_kernel(const void *xq, const void *wq, const void *x_scale, const void *w_scale, const PairParams &p,
                       cudaStream_t st) {
  return p.k_end_offsets ? launch_pair_kernel_t<true>(xq, wq, x_scale, w_scale, p, st)
                         : launch_pair_kernel_t<false>(xq, wq, x_scale, w_scale, p, st);
}

}  // namespace nvfp4_pair
}  // namespace mslk_b200
