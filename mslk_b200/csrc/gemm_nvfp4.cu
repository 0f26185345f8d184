// NVFP4 GEMM entry point (block-scaled tcgen05 kernel).
#include "../../include/mslk_b200.h"
#include "common.cuh"
#include "host.h"

MSLK_API int mslk_b200_f4f4bf16(const void *, const void *, const void *, const void *, const float *, void *, int64_t,
                                int64_t, int64_t, void *) {
  return mslk_b200::fail(3, "f4f4bf16: kernel not built yet");
}
