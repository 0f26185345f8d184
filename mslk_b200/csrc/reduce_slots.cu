// Sum of `slots` bf16 matrices [rows, cols] stored back to back -> bf16 [rows, cols], accumulated in
// fp32 in slot order (deterministic).  Second half of the fused K-sharded GEMM + reduce-scatter: every
// rank's GEMM epilogue has deposited its partial product for this rank's rows in slot <source rank>.
// HBM-bound: reads slots*rows*cols*2 bytes, writes rows*cols*2 bytes; 16-byte accesses.
#include "../../include/mslk_b200.h"
#include "common.cuh"
#include "host.h"

namespace mslk_b200 {
namespace {

__global__ void __launch_bounds__(256) reduce_slots_kernel(const uint4 *__restrict__ in, uint4 *__restrict__ out,
                                                           int slots, size_t vecs_per_slot) {
  for (size_t v = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < vecs_per_slot;
       v += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < slots; ++s) {
      const uint4 q = in[static_cast<size_t>(s) * vecs_per_slot + v];
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[2 * i] += __uint_as_float(w[i] << 16);
        acc[2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
      }
    }
    out[v] = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                        pack_bf16x2(acc[6], acc[7]));
  }
}

}  // namespace
}  // namespace mslk_b200

MSLK_API int mslk_b200_reduce_slots_bf16(const void *slots_base, int slots, int64_t rows, int64_t cols, void *out,
                                         void *stream) {
  using namespace mslk_b200;
  clear_error();
  if (slots < 1 || rows < 0 || cols < 0) return fail(1, "reduce_slots: bad shape");
  const size_t elems = static_cast<size_t>(rows) * cols;
  if (elems == 0) return 0;
  if (elems % 8 != 0) return fail(1, "reduce_slots: rows*cols must be a multiple of 8");
  if ((reinterpret_cast<uintptr_t>(slots_base) | reinterpret_cast<uintptr_t>(out)) & 15u)
    return fail(1, "reduce_slots: buffers must be 16-byte aligned");
  const size_t vecs = elems / 8;
  size_t blocks = (vecs + 255) / 256;
  const size_t cap = static_cast<size_t>(sm_count()) * 8;
  if (blocks > cap) blocks = cap;
  reduce_slots_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4 *>(slots_base), static_cast<uint4 *>(out), slots, vecs);
  return check_cuda(cudaGetLastError(), "reduce_slots launch");
}
