// Interface between the NVFP4 GEMM entry points (gemm_nvfp4.cu) and the CTA-pair kernel
// (gemm_nvfp4_2cta.cu).
#pragma once

#include "../../include/mslk_b200.h"
#include "host.h"

#include <cuda_bf16.h>

namespace mslk_b200 {
namespace nvfp4_pair {

constexpr int kPairMaxGroups = 255;

struct PairParams {
  const float *alpha;   // device scalar
  __nv_bfloat16 *y;
  int *status;
  int M, N, K;
  int ncb;              // scale atoms per 128-row block = ceil(K / 64); one scale per 32 elements: ceil(K / 128)
  int scale_mode;       // kScaleNvfp4 / kScaleMxfp4 / kScaleMxfp4_16 (common.cuh); alpha may be null for the MX formats
  int band;             // 256-row blocks per scheduling band (tiles of a band run column by column)
  int tma_store;        // set by the launcher: y is 16-byte aligned and N % 8 == 0, the epilogue may use TMA stores
  // Grouped (stacked) problems: G weight blocks of N rows, group g owning m_sizes[g] (or the rows up to
  // end_offsets[g]) consecutive rows of X / Y; the scale rows of every group start on a 128-row boundary,
  // sfa_row_start[g] when given, else the groups follow each other, each padded to 128 rows.  Dense: G = 1, all null.
  const int64_t *m_sizes;
  const int32_t *end_offsets;
  const int64_t *sfa_row_start;
  // K-grouped problems (the "2D-2D" form): X [M, K], W [N, K], group g contracting its own K range into y[g] of a
  // [G, M, N] output: int32 END offsets along K (multiples of 32), one scale block per group, and the 512-byte atoms the
  // two scale tensors hold.  Null / 0 for every other form.
  const int32_t *k_end_offsets;
  long long sfa_atoms, sfb_atoms;
  int G;
  int alpha_per_group;
  unsigned long long *timers;   // optional SM-cycle counters (sums over pairs): [0] the MMA lane waiting for operand stages,
                                // [1] for a free accumulator, [2] its whole loop, [3] the leader's producer waiting for free
                                // stages, [4] the leader's first epilogue warp from "accumulator ready" to handing it back
                                // (the chunks the next accumulator overlaps), [5] waiting for it, [6] reading the other chunks
};

// Dense problems and grouped ones with at most kPairMaxGroups groups.  Returns 0 on success, a non-zero code after recording an error, or -1 when
// the device cannot run CTA pairs (the caller then takes the one-CTA kernel).
int launch_pair_kernel(const void *xq, const void *wq, const void *x_scale, const void *w_scale, const PairParams &p,
                       cudaStream_t st);

// Diagnostics: device array of seven 64-bit counters the kernel adds its wait cycles to (nullptr = off).
void set_pipe_timers(unsigned long long *dev_counters);

}  // namespace nvfp4_pair
}  // namespace mslk_b200
