// Rowwise-scaled FP8 GEMM on CTA pairs (tcgen05 cta_group::2) for sm_100a.
//
// Two CTAs on neighbouring SMs (a cluster of 2) compute one 256 x 256 output tile.
// Each CTA TMA-loads only its own operand slices -- its 128 rows of A and its 128 of
// the 256 rows of B -- so per SM the ring holds {A 128x128, B 128x128} = 32 KB per
// K-block instead of 48 KB, and the tensor core reads 8 KB instead of 12 KB of shared
// memory per instruction.  No load is multicast.
//
//   CTA rank 0 ("leader")                      CTA rank 1
//   warp 0  producer: waits its own empty[s], TMA -> own smem, bytes counted on the
//           LEADER's full[s] (the leader arms it with the bytes of both CTAs)
//   warp 1  MMA issuer (cta_group::2, 256x256x32)     (idle; takes part in TMEM alloc)
//           frees stage s in both CTAs with one tcgen05.commit per CTA,
//           hands the accumulator to both epilogues the same way
//   warps 2..5 epilogue on the CTA's own 128 accumulator rows; every epilogue warp of
//           both CTAs arrives on the leader's tmem_empty barrier
//
// The tile scheduler, epilogue arithmetic and bounded waits are those of the 1-CTA
// kernel (gemm_f8_common.cuh, common.cuh).  Cluster-wide hardware barriers are used
// only at start-up (barriers initialised before the peer touches them) and at
// teardown (no MMA may still write the peer's tensor memory when it is freed); every
// control path of both CTAs reaches them.
#include "gemm_f8_common.cuh"

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <cstring>

namespace mslk_b200 {
namespace gemm_f8 {
namespace {

constexpr int kPairBN = 256;            // output columns of the pair tile
constexpr int kPairRows = 2 * kBM;      // output rows of the pair tile
constexpr int kStageA = kBM * kBK;      // this CTA's rows of A
constexpr int kStageB = (kPairBN / 2) * kBK;  // this CTA's half of the B rows
constexpr int kStageBytes = kStageA + kStageB;
constexpr int kStages = 5;
constexpr int kOutCols = 64;                       // columns of one staged output slab (128-byte rows)
constexpr int kOutSlabBytes = 32 * kOutCols * 2;   // 32 rows x 64 bf16
constexpr int kOutStageBytes = 4 * 2 * kOutSlabBytes;  // four epilogue warps, double-buffered
constexpr int kTmemCols = 512;          // two 256-column accumulators
constexpr int kPairBandM = 8;           // default band: 8 x 256 rows (grouped problems)
// instruction descriptor: fp32 accumulate, e4m3 x e4m3, K-major, M = 256 over the pair, N = n
__host__ __device__ constexpr uint32_t make_idesc(int n) {
  return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(kPairRows >> 4) << 24);
}
constexpr uint32_t kIdesc = make_idesc(kPairBN);

// Swapped operand roles (kSwap), used for grouped problems: the WEIGHT rows are the 256-row M operand
// of the pair-wide instruction and the tokens of a group are its N operand, whose extent may be any
// multiple of 16 up to 256.  A ragged group then wastes at most 15 token columns of tensor work
// instead of up to 255 rows.  The accumulator holds the transposed tile (lane = weight row, column =
// token), which the epilogue writes back with 2-byte stores that are contiguous across a warp.
__device__ __forceinline__ int swap_cols(int rows) { return max(32, (rows + 15) / 16 * 16); }

// Tensor maps of the output buffers (own + up to 7 further destinations), box {64 columns, 32 rows}.
struct OutMaps {
  CUtensorMap m[8];
};

struct SmemTail {
  float w_scale[4][kPairBN];
  float bias[4][kPairBN];
  int tile_start[kMaxGroups + 1];
  int row_start[kMaxGroups + 1];
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

constexpr size_t kSmemBytes = 1024 + static_cast<size_t>(kStages) * kStageBytes + kOutStageBytes + sizeof(SmemTail);
static_assert(kSmemBytes <= 232448, "shared memory budget exceeded");

template <bool kSwap>
__global__ void __launch_bounds__(kNumThreads, 1)
    gemm_f8_rowwise_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                                const __grid_constant__ CUtensorMap tmap_a32, const __grid_constant__ CUtensorMap tmap_a64,
                                const __grid_constant__ OutMaps ymaps, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *ring = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t *out_stage = ring + static_cast<size_t>(kStages) * kStageBytes;  // 1024-byte aligned slabs
  SmemTail &S = *reinterpret_cast<SmemTail *>(out_stage + kOutStageBytes);

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair_id = blockIdx.x / 2;
  const int num_pairs = gridDim.x / 2;
  const int n_tiles = (p.N + kPairBN - 1) / kPairBN;
  const int k_blocks = (p.K + kBK - 1) / kBK;
  volatile int *abort_flag = &S.abort_flag;

  // ------------------------------------------------------------------ setup
  if (threadIdx.x == 0) {
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
    if (kSwap) {
      prefetch_tensormap(&tmap_a32);
      prefetch_tensormap(&tmap_a64);
    }
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&S.full[s], 1);
      mbar_init(&S.empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&S.tmem_full[a], 1);
      mbar_init(&S.tmem_empty[a], 2 * (kNumEpilogueThreads / 32));  // epilogue warps of both CTAs
    }
    S.abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc_pair(&S.tmem_base, kTmemCols);
    tmem_relinquish_pair();
  }
  // everything above touched shared and tensor memory only: it may run under the tail of the previous kernel
  // of the stream; from here on global memory is read (group sizes, operands, scales) and written
  griddep_wait();
  griddep_launch_dependents();
  if (warp == 2) build_group_tables(p, n_tiles, kPairRows, lane, S.row_start, S.tile_start);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything is signalled on them
  tc_fence_after();
  const uint32_t tmem_base = S.tmem_base;

  Scheduler sched{S.tile_start, S.row_start, p.G, p.N, n_tiles, kPairBN, kPairRows, p.band_m > 0 ? p.band_m : kPairBandM, 0,
                  p.G == 1 ? p.band_n : 0};

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer (both CTAs)
    if (elect_one()) {  // one lane, chosen so that the compiler keeps the issue loop on the uniform datapath
      int stage = 0;
      uint32_t phase = 0;
      Tile t;
      bool ok = true;
      for (int tile = pair_id; ok && sched.get(tile, t); tile += num_pairs) {
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&S.empty[stage], phase ^ 1, abort_flag, p.status, kStatusProducerTimeout)) {
            ok = false;
            break;
          }
          uint8_t *sa = ring + static_cast<size_t>(stage) * kStageBytes;
          uint8_t *sb = sa + kStageA;
          const uint32_t leader_full = mapa_u32(smem_u32(&S.full[stage]), 0);
          if (kSwap) {
            // weights -> M operand (this CTA's 128 of the tile's 256 weight rows); tokens -> N operand
            // (this CTA's half of the tile's token columns, fetched with the smallest box of 32 / 64 / 128
            // rows that holds it: a short tile is bound by its loads, not by its instructions)
            const int half = swap_cols(t.rows) / 2;
            const int box = half <= 32 ? 32 : (half <= 64 ? 64 : 128);
            const CUtensorMap *tok = half <= 32 ? &tmap_a32 : (half <= 64 ? &tmap_a64 : &tmap_a);
            if (leader) mbar_arrive_expect_tx(&S.full[stage], 2 * (kStageA + box * kBK));
            tma_load_2d_pair(sa, &tmap_b, leader_full, kb * kBK, t.wrow0 + static_cast<int>(rank) * kBM);
            tma_load_2d_pair(sb, tok, leader_full, kb * kBK, t.row0 + static_cast<int>(rank) * half);
          } else {
            if (leader) mbar_arrive_expect_tx(&S.full[stage], 2 * kStageBytes);
            tma_load_2d_pair(sa, &tmap_a, leader_full, kb * kBK, t.row0 + static_cast<int>(rank) * kBM);
            tma_load_2d_pair(sb, &tmap_b, leader_full, kb * kBK, t.wrow0 + static_cast<int>(rank) * (kPairBN / 2));
          }
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
    if (leader && elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      Tile t;
      for (int tile = pair_id; ok && sched.get(tile, t); tile += num_pairs, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&S.tmem_empty[acc], acc_phase ^ 1, abort_flag, p.status, kStatusMmaTimeout)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kPairBN);
        const uint32_t idesc = kSwap ? make_idesc(swap_cols(t.rows)) : kIdesc;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&S.full[stage], phase, abort_flag, p.status, kStatusMmaTimeout)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(ring + static_cast<size_t>(stage) * kStageBytes);
          const uint64_t da = make_kmajor_sw128_desc(sa);
          const uint64_t db = make_kmajor_sw128_desc(sa + kStageA);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            mma_f8f6f4_pair(d_tmem, da + static_cast<uint64_t>(k * (kUmmaK >> 4)),
                            db + static_cast<uint64_t>(k * (kUmmaK >> 4)), idesc, (kb | k) != 0 ? 1u : 0u);
          }
          // free the stage in both CTAs once these MMAs have read it
          const uint32_t e = smem_u32(&S.empty[stage]);
          tc_commit_pair(mapa_u32(e, 0));
          tc_commit_pair(mapa_u32(e, 1));
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        const uint32_t f = smem_u32(&S.tmem_full[acc]);
        tc_commit_pair(mapa_u32(f, 0));
        tc_commit_pair(mapa_u32(f, 1));
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- epilogue (both CTAs, own 128 rows)
    const int quad = warp & 3;
    const int row_in_cta = quad * 32 + lane;
    const int row_in_tile = static_cast<int>(rank) * kBM + row_in_cta;
    bool y_vec_ok = (p.ldy % 8 == 0) && (p.col0 % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.y) & 15u) == 0);
    for (int d = 0; d < p.n_extra; ++d) y_vec_ok = y_vec_ok && ((reinterpret_cast<uintptr_t>(p.y_extra[d]) & 15u) == 0);
    int local = 0;
    uint32_t slab_seq = 0;
    Tile t;
    for (int tile = pair_id; sched.get(tile, t); tile += num_pairs, ++local) {
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      if (kSwap) {
        // transposed tile: lane = weight row, columns = the tile's tokens
        const int nt = swap_cols(t.rows);
        const int n_local = static_cast<int>(rank) * kBM + row_in_cta;
        const bool n_ok = t.n0 + n_local < p.N;
        const float wsc = n_ok ? p.w_scale[t.ws0 + n_local] : 0.f;
        float *xs_s = S.w_scale[warp - 2];   // this warp's buffer: the row scales of the tile's tokens
        for (int c = lane; c < nt; c += 32) xs_s[c] = c < t.rows ? p.x_scale[t.row0 + c] : 0.f;
        __syncwarp();
        const bool got = mbar_wait(&S.tmem_full[acc], acc_phase, abort_flag, p.status, kStatusEpilogueTimeout);
        if (!__all_sync(0xffffffffu, got)) break;
        tc_fence_after();
        const uint32_t taddr =
            tmem_base + static_cast<uint32_t>(acc * kPairBN) + (static_cast<uint32_t>(quad * 32) << 16);
        __nv_bfloat16 *ycol = p.y + static_cast<size_t>(t.row0) * p.ldy + p.col0 + t.n0 + n_local;
        const int warp_n0 = t.n0 + static_cast<int>(rank) * kBM + quad * 32;   // first weight row of this warp
        uint8_t *bufs = out_stage + (warp - 2) * 2 * kOutSlabBytes;
#pragma unroll 1
        for (int c = 0; c * 32 < t.rows; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
          if (p.scatter_idx) {
            // fused combine: the block is transposed through shared memory, then lane l owns token
            // c*32 + l and ADDS its 32 columns (64 bytes) to row scatter_idx[token] of y
            uint8_t *buf = bufs + (slab_seq++ & 1) * kOutSlabBytes;
            __syncwarp();   // the lanes are done reading the block staged two chunks ago
#pragma unroll
            for (int j = 0; j < 32; ++j)
              *reinterpret_cast<__nv_bfloat16 *>(buf + j * 64 + lane * 2) =
                  __float2bfloat16_rn((__uint_as_float(r[j]) * xs_s[c * 32 + j]) * wsc);
            __syncwarp();
            const int token = c * 32 + lane;
            if (token < t.rows) {
              const long long dst = p.scatter_bits == 64
                                        ? static_cast<const long long *>(p.scatter_idx)[t.row0 + token]
                                        : static_cast<long long>(static_cast<const int *>(p.scatter_idx)[t.row0 + token]);
              if (dst < 0 || dst >= p.scatter_rows) {
                atomicOr(p.status, kStatusBadScatterIndex);   // reported, not followed
              } else {
                __nv_bfloat16 *yrow = p.y + static_cast<size_t>(dst) * p.ldy + p.col0 + warp_n0;
                if (p.tma_store && warp_n0 + 32 <= p.N) {   // 16-byte aligned destination, whole block in range
#pragma unroll
                  for (int q4 = 0; q4 < 4; ++q4) {
                    const uint4 v = *reinterpret_cast<const uint4 *>(buf + lane * 64 + q4 * 16);
                    asm volatile("red.relaxed.gpu.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(yrow + 8 * q4),
                                 "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                                 : "memory");
                  }
                } else {
                  for (int j = 0; j < 32 && warp_n0 + j < p.N; ++j)
                    atomicAdd(yrow + j, *reinterpret_cast<const __nv_bfloat16 *>(buf + lane * 64 + j * 2));
                }
              }
            }
          } else if (p.tma_store && c * 32 + 32 <= t.rows && warp_n0 + 32 <= p.N) {
            // whole 32-token x 32-column block: transpose through shared memory (row = token, 64 bytes),
            // one TMA store of 2 KB
            uint8_t *buf = bufs + (slab_seq++ & 1) * kOutSlabBytes;
            if (lane == 0) tma_store_wait_read<1>();  // the store that last read this buffer is done with it
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 32; ++j)
              *reinterpret_cast<__nv_bfloat16 *>(buf + j * 64 + lane * 2) =
                  __float2bfloat16_rn((__uint_as_float(r[j]) * xs_s[c * 32 + j]) * wsc);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&ymaps.m[1], buf, p.col0 + warp_n0, t.row0 + c * 32);
              tma_store_commit();
            }
          } else if (n_ok) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int token = c * 32 + j;
              if (token < t.rows)
                ycol[static_cast<size_t>(token) * p.ldy] = __float2bfloat16_rn((__uint_as_float(r[j]) * xs_s[token]) * wsc);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&S.tmem_empty[acc]), 0));
        continue;
      }
      float *ws_s = S.w_scale[warp - 2];
      float *bs_s = S.bias[warp - 2];
      for (int c = lane; c < kPairBN; c += 32) {
        const bool in = t.n0 + c < p.N;
        ws_s[c] = in ? p.w_scale[t.ws0 + c] : 0.f;
        float b = 0.f;
        if (in && p.bias_kind == MSLK_B200_BIAS_F32) b = static_cast<const float *>(p.bias)[t.ws0 + c];
        if (in && p.bias_kind == MSLK_B200_BIAS_BF16)
          b = __bfloat162float(static_cast<const __nv_bfloat16 *>(p.bias)[t.ws0 + c]);
        bs_s[c] = b;
      }
      __syncwarp();
      const bool row_ok = row_in_tile < t.rows;
      const float xs = row_ok ? p.x_scale[t.row0 + row_in_tile] : 0.f;
      const bool got = mbar_wait(&S.tmem_full[acc], acc_phase, abort_flag, p.status, kStatusEpilogueTimeout);
      if (!__all_sync(0xffffffffu, got)) break;
      tc_fence_after();
      const uint32_t taddr =
          tmem_base + static_cast<uint32_t>(acc * kPairBN) + (static_cast<uint32_t>(quad * 32) << 16);
      const int slab_row0 = static_cast<int>(rank) * kBM + quad * 32;   // first row of this warp's 32-row slab in the tile
      if (p.tma_store && slab_row0 + 32 <= t.rows) {
        // Full slab: scale in registers, stage 32 x 64 bf16 in shared memory (128-byte rows, 128-byte
        // swizzle), and let TMA write 128-byte row segments to every destination.
        uint8_t *bufs = out_stage + (warp - 2) * 2 * kOutSlabBytes;
#pragma unroll 1
        for (int c2 = 0; c2 < kPairBN / kOutCols; ++c2) {
          if (t.n0 + c2 * kOutCols >= p.N) break;
          uint8_t *buf = bufs + (slab_seq++ & 1) * kOutSlabBytes;  // alternates across tiles too
          if (lane == 0) tma_store_wait_read<1>();  // the store that last read this buffer is done with it
          __syncwarp();
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t r[32], packed[16];
            tmem_ld_32x32(taddr + c2 * kOutCols + h * 32, r);
            tmem_ld_wait();
            epilogue_pack_any(p.bias_kind, r, xs, ws_s + c2 * kOutCols + h * 32, bs_s + c2 * kOutCols + h * 32, packed);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int chunk = (h * 4 + q) ^ (lane & 7);
              *reinterpret_cast<uint4 *>(buf + lane * 128 + chunk * 16) =
                  make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            const int x = p.col0 + t.n0 + c2 * kOutCols;
            const int y = t.row0 + slab_row0;
            if (p.rs_rows > 0) {
              const int owner = y / p.rs_rows;
              tma_store_2d(&ymaps.m[owner], buf, x, p.rs_slot * p.rs_rows + (y - owner * p.rs_rows));
            } else {
              for (int d = 0; d <= p.n_extra; ++d) tma_store_2d(&ymaps.m[d], buf, x, y);
            }
            tma_store_commit();
          }
        }
      } else {
        const size_t yoff = static_cast<size_t>(t.row0 + row_in_tile) * p.ldy + p.col0 + t.n0;
#pragma unroll 1
        for (int c = 0; c < kPairBN / 32; ++c) {
          const int cols_left = p.N - (t.n0 + c * 32);
          if (cols_left <= 0) break;
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
          const float *ws = ws_s + c * 32;
          const float *bs = bs_s + c * 32;
          if (p.bias_kind == MSLK_B200_BIAS_NONE)
            epilogue_chunk<kPairBN, MSLK_B200_BIAS_NONE>(r, xs, ws, bs, p, yoff + c * 32, row_ok, cols_left, y_vec_ok);
          else if (p.bias_kind == MSLK_B200_BIAS_F32)
            epilogue_chunk<kPairBN, MSLK_B200_BIAS_F32>(r, xs, ws, bs, p, yoff + c * 32, row_ok, cols_left, y_vec_ok);
          else
            epilogue_chunk<kPairBN, MSLK_B200_BIAS_BF16>(r, xs, ws, bs, p, yoff + c * 32, row_ok, cols_left, y_vec_ok);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&S.tmem_empty[acc]), 0));
    }
    if (lane == 0) tma_store_wait<0>();  // every staged slab has been written out before the CTA leaves
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

}  // namespace

int launch_pair_kernel(const void *xq, const void *wq, const GemmParams &p, cudaStream_t st) {
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
  cfg.numAttrs = 1;   // the occupancy query below takes the cluster shape only

  if (max_pairs[dev] == 0) {
    for (const void *fn : {reinterpret_cast<const void *>(gemm_f8_rowwise_pair_kernel<false>),
                           reinterpret_cast<const void *>(gemm_f8_rowwise_pair_kernel<true>)})
      if (int rc = check_cuda(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   static_cast<int>(kSmemBytes)),
                              "cudaFuncSetAttribute(gemm_f8_rowwise_pair)"))
        return rc;
    // how many CTA pairs the device can hold at once: a persistent kernel must not launch more
    cfg.gridDim = dim3(2 * (sm_count() / 2), 1, 1);
    int n = 0;
    cudaError_t e = cudaOccupancyMaxActiveClusters(&n, gemm_f8_rowwise_pair_kernel<false>, &cfg);
    if (e != cudaSuccess || n <= 0) {
      cudaGetLastError();
      max_pairs[dev] = -1;
    } else {
      max_pairs[dev] = n;
    }
  }
  if (max_pairs[dev] < 0) return -1;

  const int64_t row_blocks_ub = p.m_sizes ? (static_cast<int64_t>(p.total_m) + kPairRows - 1) / kPairRows + p.G
                                          : static_cast<int64_t>(p.G) * ((p.group_m + kPairRows - 1) / kPairRows);
  const int64_t tiles_ub = row_blocks_ub *
                           ((p.N + kPairBN - 1) / kPairBN);
  const int64_t mp = max_pairs[dev].load();
  const int pairs = static_cast<int>(tiles_ub < mp ? tiles_ub : mp);

  CUtensorMap ta, tb, ta32, ta64;
  if (int rc = make_tmap_2d_bytes(&ta, xq, p.K, p.total_m, p.K, kBK, kBM, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  if (int rc = make_tmap_2d_bytes(&ta32, xq, p.K, p.total_m, p.K, kBK, 32, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  if (int rc = make_tmap_2d_bytes(&ta64, xq, p.K, p.total_m, p.K, kBK, 64, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  if (int rc = make_tmap_2d_bytes(&tb, wq, p.K, static_cast<uint64_t>(p.G) * p.N, p.K, kBK, kPairBN / 2,
                                  CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;

  // Output through shared memory + TMA stores when every destination allows it: 16-byte aligned
  // bases and row pitch, column window aligned to 8 and a multiple of the 64-column slab (a slab
  // must never spill into a neighbouring column block).
  GemmParams q = p;
  OutMaps ymaps;
  memset(&ymaps, 0, sizeof(ymaps));
  bool tma_ok = (q.ldy % 8 == 0) && (q.col0 % 8 == 0) && (q.N % kOutCols == 0);
  for (int d = 0; d <= q.n_extra && tma_ok; ++d) {
    const void *base = d == 0 ? static_cast<const void *>(q.y) : static_cast<const void *>(q.y_extra[d - 1]);
    tma_ok = (reinterpret_cast<uintptr_t>(base) & 15u) == 0;
  }
  if (tma_ok) {
    for (int d = 0; d <= q.n_extra; ++d) {
      const void *base = d == 0 ? static_cast<const void *>(q.y) : static_cast<const void *>(q.y_extra[d - 1]);
      if (int rc = make_tmap_2d_bf16(&ymaps.m[d], base, q.ldy, q.total_m, static_cast<uint64_t>(q.ldy) * 2, kOutCols, 32,
                                     CU_TENSOR_MAP_SWIZZLE_128B))
        return rc;
    }
  }
  q.tma_store = tma_ok ? 1 : 0;
  if (q.rs_rows > 0 && (!tma_ok || q.rs_rows % 32 != 0 || q.total_m % 32 != 0))
    return fail(1, "row-scatter GEMM needs 16-byte aligned buffers, N %% 64 == 0 and rows per rank %% 32 == 0");

  // Tile order of dense problems.  All pairs advance through K together, so one wave of P pairs working on b
  // blocks of one dimension and P / b of the other touches (b + P / b) 256-row slabs of K bytes each.  When that
  // working set fits the part of L2 a kernel can count on (about 45 MB measured: 8192^3 ran 368 us with bands of
  // 16, 402 us with bands of 32), the band's operand stays resident between waves and the other operand is read
  // once per band: take the tallest such band, along whichever dimension then moves fewer bytes.  When it cannot
  // fit (long K) nothing survives between waves anyway and the squarest wave (bands of 8) reads least.
  // (L2 eviction hints on the TMA copies were measured too: evict_last on the resident operand changed nothing,
  // evict_first on the streamed operand and the stores raised the DRAM reads by 15-20 %: lines were dropped before
  // every pair of the wave had fetched them.)
  if (q.G == 1 && !q.m_sizes && !q.end_offsets) {
    const int64_t m_tiles = (static_cast<int64_t>(q.total_m) + kPairRows - 1) / kPairRows;
    const int64_t n_tiles = (static_cast<int64_t>(q.N) + kPairBN - 1) / kPairBN;
    const double slab = static_cast<double>(kPairRows) * q.K, budget = 45.0 * (1 << 20), P = static_cast<double>(pairs);
    auto tallest = [&](int64_t tiles) {
      int64_t best = 0;
      for (int64_t b = std::min<int64_t>(8, tiles); b <= tiles; ++b)
        if ((b + P / b) * slab <= budget) best = b;
      return best;
    };
    const int64_t bm = tallest(m_tiles), bn = tallest(n_tiles);
    const double a_bytes = static_cast<double>(q.total_m) * q.K, b_bytes = static_cast<double>(q.N) * q.K;
    const double traffic_m = bm ? a_bytes + b_bytes * ((m_tiles + bm - 1) / bm) : 1e30;
    const double traffic_n = bn ? b_bytes + a_bytes * ((n_tiles + bn - 1) / bn) : 1e30;
    q.band_m = kPairBandM;
    if (bm && traffic_m <= traffic_n) q.band_m = static_cast<int>(bm);
    else if (bn) q.band_n = static_cast<int>(bn);
  }

  cfg.gridDim = dim3(2 * pairs, 1, 1);
  // grouped problems (ragged token counts) run with swapped operand roles
  // measured on E = 8 ... 128 experts: a gain of 16-19 % at a mean of 256 tokens per group, break-even near 1024,
  // a loss of 7 % at 4096 (the transposed epilogue costs more than the padding it saves); at a mean of 1024 (16 experts,
  // Zipf counts) normal roles were 2.6 % faster on (16384, 5120) and equal on (5120, 8192) once both ran with dependent launch
  bool swap = q.m_sizes != nullptr && q.bias_kind == MSLK_B200_BIAS_NONE && q.n_extra == 0 && q.rs_rows == 0;
  if (q.scatter_idx) {
    if (!swap) return -1;   // the scatter-add epilogue of this kernel exists for swapped roles only
  } else if (swap) {
    swap = q.total_m / q.G < 1024;
  }
  if (swap) {
    // its epilogue stores 32-token x 32-column blocks: box {32 columns = 64 bytes, 32 rows}, no swizzle, in map slot 1
    q.tma_store = (q.ldy % 8 == 0) && (q.col0 % 8 == 0) && (reinterpret_cast<uintptr_t>(q.y) & 15u) == 0;
    if (q.tma_store)
      if (int rc = make_tmap_2d_bf16(&ymaps.m[1], q.y, q.ldy, q.total_m, static_cast<uint64_t>(q.ldy) * 2, 32, 32,
                                     CU_TENSOR_MAP_SWIZZLE_NONE))
        return rc;
  }
  cfg.numAttrs = 1 + pdl_attribute(&attr[1]);   // the prologue may overlap the tail of the previous kernel of the stream
  if (swap)
    return check_cuda(cudaLaunchKernelEx(&cfg, gemm_f8_rowwise_pair_kernel<true>, ta, tb, ta32, ta64, ymaps, q),
                      "f8f8bf16_rowwise pair launch");
  return check_cuda(cudaLaunchKernelEx(&cfg, gemm_f8_rowwise_pair_kernel<false>, ta, tb, ta32, ta64, ymaps, q),
                    "f8f8bf16_rowwise pair launch");
}

}  // namespace gemm_f8
}  // namespace mslk_b200
