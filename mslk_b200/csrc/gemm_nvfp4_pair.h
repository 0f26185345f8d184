// Interface between the NVFP4 GEMM entry points (gemm_nvfp4.cu) and the CTA-pair kernel
// (gemm_nvfp4_2cta.cu).
#pragma once

#include "../../include/mslk_b200.h"
#include "host.h"

#include <cuda_bf16.h>

namespace mslk_b200 {
namespace nvfp4_pair {

struct PairParams {
  const float *alpha;   // device scalar
  __nv_bfloat16 *y;
  int *status;
  int M, N, K;
  int ncb;              // scale atoms per 128-row block = ceil(K / 64)
  int band;             // 256-row blocks per scheduling band (tiles of a band run column by column)
  int tma_store;        // set by the launcher: y is 16-byte aligned and N % 8 == 0, the epilogue may use TMA stores
  unsigned long long *timers;   // optional: [0] ns the MMA lane waited for operand stages, [1] for a free accumulator,
                                // [2] ns of its whole loop, [3] ns the producer of the leader waited for free stages (sums over pairs)
};

// Dense problems only.  Returns 0 on success, a non-zero code after recording an error, or -1 when
// the device cannot run CTA pairs (the caller then takes the one-CTA kernel).
int launch_pair_kernel(const void *xq, const void *wq, const void *x_scale, const void *w_scale, const PairParams &p,
                       cudaStream_t st);

// Diagnostics: device array of four 64-bit counters the kernel adds its wait cycles to (nullptr = off).
void set_pipe_timers(unsigned long long *dev_counters);

}  // namespace nvfp4_pair
}  // namespace mslk_b200
