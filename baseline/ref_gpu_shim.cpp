// Torch-library shim around kernel instances of the reference (meta-pytorch/MSLK) compiled from the
// reference's own sources, for on-box comparison runs.  The instance functions are defined in the
// reference's csrc/gemm/cutlass/*/ *.cu files (declared in its *_manifest.cuh headers); this file only
// re-declares their signatures and registers them under the separate namespace `mslk_ref`, so that the
// library can live in one process with this repository's own `mslk::` operators.
#include <ATen/ATen.h>
#include <torch/library.h>

#include <optional>

namespace mslk::gemm {
// csrc/gemm/cutlass/f8f8bf16_rowwise/f8f8bf16_rowwise_manifest.cuh
at::Tensor f8f8bf16_rowwise_128_256_128_2_1_1_10_f_f(at::Tensor XQ, at::Tensor WQ, at::Tensor x_scale, at::Tensor w_scale,
                                                     bool use_fast_accum, std::optional<at::Tensor> bias,
                                                     std::optional<at::Tensor> output);
at::Tensor f8f8bf16_rowwise_128_64_128_1_1_1_10_f_f(at::Tensor XQ, at::Tensor WQ, at::Tensor x_scale, at::Tensor w_scale,
                                                    bool use_fast_accum, std::optional<at::Tensor> bias,
                                                    std::optional<at::Tensor> output);
// csrc/gemm/cutlass/f8f8bf16_rowwise_grouped_sm100/f8f8bf16_rowwise_grouped_manifest.cuh
at::Tensor f8f8bf16_rowwise_grouped_256_256_128_2_1_1_10_f(at::Tensor XQ, at::Tensor WQ, at::Tensor x_scale,
                                                           at::Tensor w_scale, at::Tensor output,
                                                           std::optional<at::Tensor> zero_start_index_M,
                                                           std::optional<at::Tensor> M_sizes);
// csrc/gemm/cutlass/f4f4bf16/f4f4bf16_manifest.cuh
// csrc/gemm/cutlass/f4f4bf16_grouped/f4f4bf16_grouped_manifest.cuh
at::Tensor f4f4bf16_grouped_256_256_256_2_1_1(at::Tensor XQ, at::Tensor WQ, at::Tensor x_scale, at::Tensor w_scale,
                                              at::Tensor output, std::optional<at::Tensor> offsets,
                                              std::optional<at::Tensor> M_sizes, std::optional<at::Tensor> global_scale,
                                              std::optional<at::Tensor> starting_row_after_padding);
at::Tensor f4f4bf16_256_256_2_1_1(at::Tensor XQ, at::Tensor WQ, at::Tensor x_scale, at::Tensor w_scale, at::Tensor output,
                                  std::optional<at::Tensor> global_scale, int64_t mxfp4_block_size);
at::Tensor f4f4bf16_256_128_4_1_1(at::Tensor XQ, at::Tensor WQ, at::Tensor x_scale, at::Tensor w_scale, at::Tensor output,
                                  std::optional<at::Tensor> global_scale, int64_t mxfp4_block_size);
}  // namespace mslk::gemm

namespace {

using at::Tensor;

// large-M instance the reference's heuristic picks on sm_100 for M > 1024 (csrc/gemm/cutlass/f8f8bf16_rowwise.cu:24-50)
Tensor rowwise_large(Tensor XQ, Tensor WQ, Tensor xs, Tensor ws, Tensor out) {
  return mslk::gemm::f8f8bf16_rowwise_128_256_128_2_1_1_10_f_f(XQ, WQ, xs, ws, true, std::nullopt, out);
}
// few-token instance (M <= 128, N > 1024)
Tensor rowwise_small(Tensor XQ, Tensor WQ, Tensor xs, Tensor ws, Tensor out) {
  return mslk::gemm::f8f8bf16_rowwise_128_64_128_1_1_1_10_f_f(XQ, WQ, xs, ws, true, std::nullopt, out);
}
// stacked grouped GEMM as f8f8bf16_rowwise_grouped_stacked calls its kernel (csrc/gemm/cutlass/f8f8bf16_rowwise_grouped.cu:342-368)
Tensor grouped_stacked(Tensor XQ, Tensor WQ, Tensor xs, Tensor ws, Tensor M_sizes, Tensor out_flat) {
  Tensor y = mslk::gemm::f8f8bf16_rowwise_grouped_256_256_128_2_1_1_10_f(XQ, WQ, xs, ws, out_flat, std::nullopt, M_sizes);
  return y.view({XQ.size(0), WQ.size(1)});
}
Tensor f4_large(Tensor XQ, Tensor WQ, Tensor xs, Tensor ws, Tensor out, Tensor gs) {
  return mslk::gemm::f4f4bf16_256_256_2_1_1(XQ, WQ, xs, ws, out, gs, 32);
}
// the same instance in its MXFP4 mode (e8m0 scales per 32 elements, no global scale)
Tensor f4_large_mx(Tensor XQ, Tensor WQ, Tensor xs, Tensor ws, Tensor out) {
  return mslk::gemm::f4f4bf16_256_256_2_1_1(XQ, WQ, xs, ws, out, std::nullopt, 32);
}
// grouped FP4 as f4f4bf16_grouped_stacked calls its kernel (csrc/gemm/cutlass/f4f4bf16_grouped.cu:321-374); no global
// scale = MXFP4
Tensor f4_grouped_stacked(Tensor XQ, Tensor WQ, Tensor xs, Tensor ws, Tensor M_sizes, std::optional<Tensor> gs,
                          Tensor starting_row_after_padding, Tensor out) {
  return mslk::gemm::f4f4bf16_grouped_256_256_256_2_1_1(XQ, WQ, xs, ws, out, std::nullopt, M_sizes, gs,
                                                        starting_row_after_padding);
}
// ... and as f4f4bf16_grouped_mm does (:376-475): WQ already transposed to [G, N, K/2] (2D-3D) or [N, total_K/2] (2D-2D)
Tensor f4_grouped_mm(Tensor XQ, Tensor WQ, Tensor xs, Tensor ws, Tensor offsets, std::optional<Tensor> gs, Tensor out) {
  return mslk::gemm::f4f4bf16_grouped_256_256_256_2_1_1(XQ, WQ, xs, ws, out, offsets, std::nullopt, gs, std::nullopt);
}
Tensor f4_small(Tensor XQ, Tensor WQ, Tensor xs, Tensor ws, Tensor out, Tensor gs) {
  return mslk::gemm::f4f4bf16_256_128_4_1_1(XQ, WQ, xs, ws, out, gs, 32);
}

}  // namespace

TORCH_LIBRARY(mslk_ref, m) {
  m.def("f8f8bf16_rowwise_large(Tensor XQ, Tensor WQ, Tensor x_scale, Tensor w_scale, Tensor(a!) output) -> Tensor(a!)", rowwise_large);
  m.def("f8f8bf16_rowwise_small(Tensor XQ, Tensor WQ, Tensor x_scale, Tensor w_scale, Tensor(a!) output) -> Tensor(a!)", rowwise_small);
  m.def("f8f8bf16_rowwise_grouped_stacked(Tensor XQ, Tensor WQ, Tensor x_scale, Tensor w_scale, Tensor M_sizes, Tensor(a!) output) -> Tensor", grouped_stacked);
  m.def("f4f4bf16_large(Tensor XQ, Tensor WQ, Tensor x_scale, Tensor w_scale, Tensor(a!) output, Tensor global_scale) -> Tensor(a!)", f4_large);
  m.def("f4f4bf16_large_mx(Tensor XQ, Tensor WQ, Tensor x_scale, Tensor w_scale, Tensor(a!) output) -> Tensor(a!)", f4_large_mx);
  m.def("f4f4bf16_grouped_stacked(Tensor XQ, Tensor WQ, Tensor x_scale, Tensor w_scale, Tensor M_sizes, Tensor? global_scale, Tensor starting_row_after_padding, Tensor(a!) output) -> Tensor(a!)", f4_grouped_stacked);
  m.def("f4f4bf16_grouped_mm(Tensor XQ, Tensor WQ, Tensor x_scale, Tensor w_scale, Tensor offsets, Tensor? global_scale, Tensor(a!) output) -> Tensor(a!)", f4_grouped_mm);
  m.def("f4f4bf16_small(Tensor XQ, Tensor WQ, Tensor x_scale, Tensor w_scale, Tensor(a!) output, Tensor global_scale) -> Tensor(a!)", f4_small);
}
