// Interface between the NVFP4 GEMM entry points (gemm_nvfp4.cu) and the few-token
// weight-streaming kernel (gemm_nvfp4_decode.cu).
#pragma once

#include "../../include/mslk_b200.h"
#include "host.h"

#include <cuda_bf16.h>

namespace mslk_b200 {
namespace nvfp4_decode {

constexpr int kMaxTokens = 128;   // token rows the kernel takes (one UMMA N)

// Scratch needed for K splitting (0 when the shape runs unsplit or M is out of range).
size_t scratch_bytes(int64_t M, int64_t N, int64_t K, int sms);

// Dense problem with 1 <= M <= kMaxTokens, K % 32 == 0.  `scratch` (may be null) enables K splitting.
int launch_decode_kernel(const void *xq, const void *wq, const void *x_scale, const void *w_scale, const float *alpha,
                         void *y, int *status, int64_t M, int64_t N, int64_t K, void *scratch, size_t scratch_size,
                         cudaStream_t st, int scale_mode = 0);   // 0 = NVFP4 (kScaleNvfp4); MX modes: alpha is null

}  // namespace nvfp4_decode
}  // namespace mslk_b200
