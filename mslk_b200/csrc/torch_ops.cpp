// Thin PyTorch extension over the C ABI (include/mslk_b200.h).
//
// Registers, in the `mslk` operator namespace and with the reference's own schema
// strings (csrc/gemm/gemm_ops.cpp:31-34,41-42,103-104 of meta-pytorch/MSLK):
//     f8f8bf16_rowwise, f8f8bf16_rowwise_out, f8f8bf16_rowwise_grouped_stacked, f4f4bf16
// plus three operators the Python layer builds on:
//     quantize_fp8_row      (backs the Python custom op triton::quantize_fp8_row)
//     quantize_fp8_per_row  (the historical CUDA op name for the same quantizer)
//     quantize_nvfp4
// Behaviour kept from the reference: CUDAGuard on XQ's device, launch on the current
// stream, outputs from the caching allocator, no host synchronisation (CUDA-graph
// capturable), failed pre-conditions raise through TORCH_CHECK.  CPU tensors are
// rejected: there is no fallback path in this library.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <optional>
#include <tuple>

#include "mslk_b200.h"

namespace {

void check_rc(int rc, const char *what) {
  TORCH_CHECK(rc == 0, what, " failed (code ", rc, "): ", mslk_b200_last_error());
}

void *stream_of(const at::Tensor &t) { return at::cuda::getCurrentCUDAStream(t.get_device()).stream(); }

// Every tensor whose raw pointer reaches a kernel must live on the device the kernel runs on: a CPU
// tensor or one on another GPU would make the kernel dereference a host or foreign address.
void same_device(const at::Tensor &t, const at::Tensor &ref, const char *op, const char *arg) {
  TORCH_CHECK(t.is_cuda(), op, ": ", arg, " must be a CUDA tensor (this library has no CPU path)");
  TORCH_CHECK(t.device() == ref.device(), op, ": ", arg, " must be on the same device as XQ (", t.device(), " vs ",
              ref.device(), ")");
}

int64_t round_up(int64_t v, int64_t to) { return (v + to - 1) / to * to; }

int64_t prod_leading(const at::Tensor &t) {
  int64_t p = 1;
  for (int64_t i = 0; i + 1 < t.dim(); ++i) p *= t.size(i);
  return p;
}

// ------------------------------------------------------------------ dense rowwise
void rowwise_impl(const at::Tensor &XQ, const at::Tensor &WQ, const at::Tensor &x_scale, const at::Tensor &w_scale,
                  const std::optional<at::Tensor> &bias, at::Tensor &out) {
  TORCH_CHECK(XQ.is_cuda() && XQ.is_contiguous(), "f8f8bf16_rowwise: XQ must be a contiguous CUDA tensor");
  TORCH_CHECK(WQ.is_cuda() && WQ.is_contiguous(), "f8f8bf16_rowwise: WQ must be a contiguous CUDA tensor");
  TORCH_CHECK(XQ.dtype() == at::kFloat8_e4m3fn && WQ.dtype() == at::kFloat8_e4m3fn,
              "f8f8bf16_rowwise: XQ and WQ must be float8_e4m3fn");
  TORCH_CHECK(x_scale.dtype() == at::kFloat && w_scale.dtype() == at::kFloat,
              "f8f8bf16_rowwise: x_scale and w_scale must be float32");
  same_device(WQ, XQ, "f8f8bf16_rowwise", "WQ");
  same_device(x_scale, XQ, "f8f8bf16_rowwise", "x_scale");
  same_device(w_scale, XQ, "f8f8bf16_rowwise", "w_scale");
  same_device(out, XQ, "f8f8bf16_rowwise", "output");
  TORCH_CHECK(XQ.dim() >= 1 && WQ.dim() >= 1, "f8f8bf16_rowwise: XQ and WQ need at least one dimension");
  const int64_t K = XQ.size(-1);
  const int64_t M = prod_leading(XQ);
  const int64_t N = prod_leading(WQ);
  TORCH_CHECK(WQ.size(-1) == K, "f8f8bf16_rowwise: XQ and WQ disagree on K (", K, " vs ", WQ.size(-1), ")");
  TORCH_CHECK(x_scale.numel() == M && w_scale.numel() == N, "f8f8bf16_rowwise: scale sizes must equal M and N");
  TORCH_CHECK(out.dtype() == at::kBFloat16 && out.is_contiguous() && out.numel() == M * N,
              "f8f8bf16_rowwise: output must be a contiguous bfloat16 tensor of M*N elements");
  int kind = MSLK_B200_BIAS_NONE;
  at::Tensor b;
  if (bias.has_value()) {
    b = bias->contiguous();
    same_device(b, XQ, "f8f8bf16_rowwise", "bias");
    TORCH_CHECK(b.numel() == N, "f8f8bf16_rowwise: bias must have N elements");
    TORCH_CHECK(b.dtype() == at::kFloat || b.dtype() == at::kBFloat16,
                "f8f8bf16_rowwise: bias must be float32 or bfloat16");
    kind = b.dtype() == at::kFloat ? MSLK_B200_BIAS_F32 : MSLK_B200_BIAS_BF16;
  }
  c10::cuda::CUDAGuard guard(XQ.device());
  const at::Tensor xs = x_scale.contiguous(), ws = w_scale.contiguous();
  check_rc(mslk_b200_f8f8bf16_rowwise(XQ.data_ptr(), WQ.data_ptr(), xs.data_ptr<float>(), ws.data_ptr<float>(),
                                      kind ? b.data_ptr() : nullptr, kind, out.data_ptr(), M, N, K, stream_of(XQ)),
           "f8f8bf16_rowwise");
}

at::Tensor f8f8bf16_rowwise(at::Tensor XQ, at::Tensor WQ, at::Tensor x_scale, at::Tensor w_scale,
                            std::optional<at::Tensor> bias, bool /*use_fast_accum*/) {
  TORCH_CHECK(XQ.dim() >= 1 && WQ.dim() >= 1, "f8f8bf16_rowwise: XQ and WQ need at least one dimension");
  std::vector<int64_t> shape(XQ.sizes().begin(), XQ.sizes().end() - 1);
  shape.push_back(prod_leading(WQ));
  at::Tensor out = at::empty(shape, XQ.options().dtype(at::kBFloat16));
  rowwise_impl(XQ, WQ, x_scale, w_scale, bias, out);
  return out;
}

void f8f8bf16_rowwise_out(at::Tensor XQ, at::Tensor WQ, at::Tensor x_scale, at::Tensor w_scale, at::Tensor output,
                          std::optional<at::Tensor> bias, bool /*use_fast_accum*/) {
  rowwise_impl(XQ, WQ, x_scale, w_scale, bias, output);
}

// ------------------------------------------------------------------ grouped stacked
at::Tensor f8f8bf16_rowwise_grouped_stacked(at::Tensor XQ, at::Tensor WQ, at::Tensor x_scale, at::Tensor w_scale,
                                            at::Tensor M_sizes) {
  const char *n = "f8f8bf16_rowwise_grouped_stacked";
  TORCH_CHECK(XQ.is_cuda() && XQ.is_contiguous() && WQ.is_cuda() && WQ.is_contiguous(), n,
              ": XQ and WQ must be contiguous CUDA tensors");
  TORCH_CHECK(XQ.dtype() == at::kFloat8_e4m3fn && WQ.dtype() == at::kFloat8_e4m3fn, n,
              ": XQ and WQ must be float8_e4m3fn");
  TORCH_CHECK(M_sizes.device() == XQ.device(), n, ": M_sizes must be on same device as inputs.");
  TORCH_CHECK(M_sizes.dtype() == at::kLong, n, ": M_sizes must be int64.");
  TORCH_CHECK(WQ.dim() == 3 && WQ.size(0) == M_sizes.numel(), n, ": WQ must be [G,N,K] with G == M_sizes.numel()");
  TORCH_CHECK(XQ.dim() == 2 && XQ.size(1) == WQ.size(2), n, ": XQ must be [total_M,K] with the K of WQ");
  TORCH_CHECK(x_scale.dtype() == at::kFloat && w_scale.dtype() == at::kFloat, n, ": scales must be float32");
  same_device(WQ, XQ, n, "WQ");
  same_device(x_scale, XQ, n, "x_scale");
  same_device(w_scale, XQ, n, "w_scale");
  const int64_t G = WQ.size(0), N = WQ.size(1), K = WQ.size(2), total_M = XQ.size(0);
  TORCH_CHECK(x_scale.numel() == total_M && w_scale.numel() == G * N, n, ": scale sizes must equal total_M and G*N");
  at::Tensor Y = at::empty({total_M, N}, XQ.options().dtype(at::kBFloat16));
  if (total_M == 0) return Y;
  c10::cuda::CUDAGuard guard(XQ.device());
  const at::Tensor xs = x_scale.contiguous(), ws = w_scale.contiguous(), ms = M_sizes.contiguous();
  check_rc(mslk_b200_f8f8bf16_rowwise_grouped_stacked(XQ.data_ptr(), WQ.data_ptr(), xs.data_ptr<float>(),
                                                      ws.data_ptr<float>(), ms.data_ptr<int64_t>(), G, total_M, N, K,
                                                      Y.data_ptr(), stream_of(XQ)),
           n);
  return Y;
}

// ------------------------------------------------------------------ batched
// csrc/gemm/cutlass/f8f8bf16_rowwise_batched.cu:20-139: 3-D inputs only, fp32 bias, optional output.
at::Tensor f8f8bf16_rowwise_batched(at::Tensor XQ, at::Tensor WQ, at::Tensor x_scale, at::Tensor w_scale,
                                    std::optional<at::Tensor> bias, bool use_fast_accum,
                                    std::optional<at::Tensor> output) {
  const char *n = "f8f8bf16_rowwise_batched";
  TORCH_CHECK(use_fast_accum, "f8f8bf16_rowwise_batched only supports fast_accum=True");
  TORCH_CHECK(XQ.dim() == 3 && WQ.dim() == 3, "FP8 rowwise batched GEMM only supports 3D inputs");
  TORCH_CHECK(XQ.is_cuda() && XQ.is_contiguous() && WQ.is_cuda() && WQ.is_contiguous(), n,
              ": XQ and WQ must be contiguous CUDA tensors");
  TORCH_CHECK(XQ.dtype() == at::kFloat8_e4m3fn, "XQ must be FP8 e4m3fn");
  TORCH_CHECK(WQ.dtype() == at::kFloat8_e4m3fn, "WQ must be FP8 e4m3fn");
  TORCH_CHECK(x_scale.dtype() == at::kFloat && w_scale.dtype() == at::kFloat, "Scale tensors must be float32.");
  const int64_t B = XQ.size(0), M = XQ.size(1), N = WQ.size(1), K = WQ.size(2);
  TORCH_CHECK(WQ.size(0) == B, n, ": XQ and WQ disagree on the batch count");
  if (M == 0 || N == 0 || K == 0) return at::zeros({B, M, N}, XQ.options().dtype(at::kBFloat16));
  TORCH_CHECK(XQ.size(2) == K, n, ": XQ and WQ disagree on K");
  same_device(WQ, XQ, n, "WQ");
  same_device(x_scale, XQ, n, "x_scale");
  same_device(w_scale, XQ, n, "w_scale");
  TORCH_CHECK(x_scale.numel() == B * M && w_scale.numel() == B * N, n, ": scales must have B*M and B*N elements");
  at::Tensor b;
  int kind = MSLK_B200_BIAS_NONE;
  if (bias.has_value()) {
    b = bias->contiguous();
    TORCH_CHECK(b.dtype() == at::kFloat, "Bias type must be float32 if provided.");
    same_device(b, XQ, n, "bias");
    TORCH_CHECK(b.numel() == B * N, n, ": bias must have B*N elements");
    kind = MSLK_B200_BIAS_F32;
  }
  at::Tensor Y;
  if (output.has_value()) {
    Y = *output;
    TORCH_CHECK(Y.dtype() == at::kBFloat16);
    same_device(Y, XQ, n, "output");
    TORCH_CHECK(Y.is_contiguous() && Y.numel() == B * M * N, n, ": output must be a contiguous tensor of B*M*N elements");
  } else {
    Y = at::empty({B, M, N}, XQ.options().dtype(at::kBFloat16));
  }
  c10::cuda::CUDAGuard guard(XQ.device());
  const at::Tensor xs = x_scale.contiguous(), ws = w_scale.contiguous();
  check_rc(mslk_b200_f8f8bf16_rowwise_batched(XQ.data_ptr(), WQ.data_ptr(), xs.data_ptr<float>(), ws.data_ptr<float>(),
                                              kind ? b.data_ptr() : nullptr, kind, Y.data_ptr(), B, M, N, K,
                                              stream_of(XQ)),
           n);
  return Y;
}

// ------------------------------------------------------------------ NVFP4 GEMM
at::Tensor f4f4bf16(at::Tensor XQ, at::Tensor WQ, at::Tensor x_scale, at::Tensor w_scale,
                    std::optional<at::Tensor> output, std::optional<at::Tensor> global_scale,
                    int64_t mxfp4_block_size) {
  TORCH_CHECK(XQ.is_cuda() && XQ.is_contiguous(), "f4f4bf16: XQ must be a contiguous CUDA tensor");
  TORCH_CHECK(WQ.is_cuda() && WQ.is_contiguous(), "f4f4bf16: WQ must be a contiguous CUDA tensor");
  TORCH_CHECK(x_scale.is_cuda() && x_scale.is_contiguous() && w_scale.is_cuda() && w_scale.is_contiguous(),
              "f4f4bf16: scales must be contiguous CUDA tensors");
  TORCH_CHECK(mxfp4_block_size == 16 || mxfp4_block_size == 32, "f4f4bf16: mxfp4_block_size must be 16 or 32");
  TORCH_CHECK(XQ.dim() == 2 && WQ.dim() == 2, "f4f4bf16: XQ and WQ must be 2-D");
  const int64_t M = XQ.size(0), K = XQ.size(1) * 2, N = WQ.size(0);
  TORCH_CHECK(WQ.size(1) * 2 == K, "f4f4bf16: XQ and WQ disagree on K");
  TORCH_CHECK(N % 16 == 0 && K % 16 == 0, "f4f4bf16: N and K must be multiples of 16");
  same_device(WQ, XQ, "f4f4bf16", "WQ");
  same_device(x_scale, XQ, "f4f4bf16", "x_scale");
  same_device(w_scale, XQ, "f4f4bf16", "w_scale");
  if (global_scale.has_value()) same_device(*global_scale, XQ, "f4f4bf16", "global_scale");
  // NVFP4 (global_scale given): one e4m3 scale per 16 elements; else MXFP4: one e8m0 scale per mxfp4_block_size
  const int64_t block = global_scale.has_value() ? 16 : mxfp4_block_size;
  // the kernels copy whole 512-byte scale atoms of the swizzled layout padded to [roundup(rows,128), roundup(K/block,4)]
  TORCH_CHECK(x_scale.element_size() == 1 && w_scale.element_size() == 1, "f4f4bf16: scales must be 1-byte tensors");
  TORCH_CHECK(x_scale.numel() >= round_up(M, 128) * round_up(K / block, 4),
              "f4f4bf16: x_scale holds ", x_scale.numel(), " scales, the padded swizzled layout of [", M, ", ", K / block,
              "] needs ", round_up(M, 128) * round_up(K / block, 4));
  TORCH_CHECK(w_scale.numel() >= round_up(N, 128) * round_up(K / block, 4),
              "f4f4bf16: w_scale holds ", w_scale.numel(), " scales, the padded swizzled layout of [", N, ", ", K / block,
              "] needs ", round_up(N, 128) * round_up(K / block, 4));
  at::Tensor Y;
  if (output.has_value()) {
    Y = *output;
    same_device(Y, XQ, "f4f4bf16", "output");
    TORCH_CHECK(Y.dtype() == at::kBFloat16 && Y.is_contiguous() && Y.dim() == 2 && Y.size(0) == M && Y.size(1) == N,
                "f4f4bf16: output must be a contiguous bfloat16 [M,N] tensor");
  } else {
    Y = at::empty({M, N}, XQ.options().dtype(at::kBFloat16));
  }
  if (M == 0 || N == 0 || K == 0) return Y.zero_();
  c10::cuda::CUDAGuard guard(XQ.device());
  if (!global_scale.has_value()) {
    check_rc(mslk_b200_f4f4bf16_mx(XQ.data_ptr(), WQ.data_ptr(), x_scale.data_ptr(), w_scale.data_ptr(), Y.data_ptr(), M, N,
                                   K, static_cast<int>(mxfp4_block_size), stream_of(XQ)),
             "f4f4bf16");
    return Y;
  }
  const at::Tensor gs = global_scale->reshape({-1}).to(at::kFloat);
  // few-token shapes may split K over CTAs: scratch for the partial tiles comes from the caching allocator
  const size_t wsz = mslk_b200_f4f4bf16_workspace_bytes(M, N, K);
  at::Tensor ws;
  if (wsz) ws = at::empty({static_cast<int64_t>(wsz)}, XQ.options().dtype(at::kByte));
  check_rc(mslk_b200_f4f4bf16_ws(XQ.data_ptr(), WQ.data_ptr(), x_scale.data_ptr(), w_scale.data_ptr(),
                                 gs.data_ptr<float>(), Y.data_ptr(), M, N, K, wsz ? ws.data_ptr() : nullptr, wsz,
                                 stream_of(XQ)),
           "f4f4bf16");
  return Y;
}

// ------------------------------------------------------------------ quantizers
std::tuple<at::Tensor, at::Tensor> quantize_fp8_row(at::Tensor a, std::optional<at::Tensor> scale_ub,
                                                    std::optional<at::Tensor> zero_start_index_M,
                                                    std::optional<int64_t> align_rows_to, double eps) {
  TORCH_CHECK(a.is_cuda(), "quantize_fp8_row: expected a CUDA tensor (this library has no CPU path)");
  TORCH_CHECK(a.dim() >= 1 && a.dim() <= 4, "quantize_fp8_row: only up to 4 dimension input tensor is supported");
  int dt;
  if (a.dtype() == at::kFloat) dt = MSLK_B200_F32;
  else if (a.dtype() == at::kBFloat16) dt = MSLK_B200_BF16;
  else if (a.dtype() == at::kHalf) dt = MSLK_B200_F16;
  else TORCH_CHECK(false, "quantize_fp8_row: unsupported input dtype ", a.dtype());
  if (scale_ub.has_value()) TORCH_CHECK(scale_ub->device() == a.device(), "'scale_ub' must be on the same device as 'a'");
  if (zero_start_index_M.has_value())
    TORCH_CHECK(zero_start_index_M->device() == a.device(), "'zero_start_index_M' must be on the same device as 'a'");
  std::vector<int64_t> out_shape(a.sizes().begin(), a.sizes().end());
  at::Tensor a4 = a;
  while (a4.dim() < 4) a4 = a4.unsqueeze(0);
  const int64_t B = a4.size(0), M = a4.size(1), N = a4.size(2), K = a4.size(3);
  int64_t K_out = K;
  if (align_rows_to.has_value()) {
    TORCH_CHECK(*align_rows_to > 0, "quantize_fp8_row: align_rows_to must be positive");
    K_out = (K + *align_rows_to - 1) / *align_rows_to * *align_rows_to;
    out_shape.back() = K_out;
  }
  at::Tensor q = at::empty(out_shape, a.options().dtype(at::kFloat8_e4m3fn));
  out_shape.pop_back();
  at::Tensor s = at::empty(out_shape, a.options().dtype(at::kFloat));
  at::Tensor ub, zs;
  if (scale_ub.has_value()) ub = scale_ub->to(at::kFloat).contiguous();
  if (zero_start_index_M.has_value()) zs = zero_start_index_M->reshape({B, M}).to(at::kLong).contiguous();
  c10::cuda::CUDAGuard guard(a.device());
  check_rc(mslk_b200_quantize_fp8_row(a4.data_ptr(), dt, B, M, N, K, K_out, a4.stride(0), a4.stride(1), a4.stride(2),
                                      a4.stride(3), ub.defined() ? ub.data_ptr<float>() : nullptr,
                                      zs.defined() ? zs.data_ptr<int64_t>() : nullptr, static_cast<float>(eps),
                                      q.data_ptr(), s.data_ptr<float>(), stream_of(a)),
           "quantize_fp8_row");
  return {q, s};
}

std::tuple<at::Tensor, at::Tensor> quantize_fp8_per_row(at::Tensor a, std::optional<at::Tensor> scale_ub) {
  return quantize_fp8_row(a, scale_ub, std::nullopt, std::nullopt, 1.0 / 512.0);
}

std::tuple<at::Tensor, at::Tensor> quantize_nvfp4(at::Tensor x, std::optional<at::Tensor> global_scale) {
  TORCH_CHECK(x.is_cuda() && (x.dtype() == at::kBFloat16 || x.dtype() == at::kHalf),
              "quantize_nvfp4: expected a bfloat16 or float16 CUDA tensor");
  TORCH_CHECK(x.dim() >= 2, "quantize_nvfp4: expected at least 2 dimensions");
  const int64_t K = x.size(-1);
  TORCH_CHECK(K % 16 == 0, "N must be divisible by 16 for NVFP4 quantization");
  at::Tensor x2 = x.reshape({-1, K});
  if (x2.stride(1) != 1) x2 = x2.contiguous();
  const int64_t M = x2.size(0);
  const int64_t pr = (M + 127) / 128 * 128, pc = (K / 16 + 3) / 4 * 4;
  at::Tensor q = at::empty({M, K / 2}, x.options().dtype(at::kByte));
  at::Tensor s = at::empty({pr, pc}, x.options().dtype(at::kFloat8_e4m3fn));
  at::Tensor gs;
  if (global_scale.has_value()) {
    TORCH_CHECK(global_scale->is_cuda() && global_scale->device() == x.device(),
                "quantize_nvfp4: global_scale must be on the same device as x");
    gs = global_scale->reshape({-1}).to(at::kFloat);
  }
  c10::cuda::CUDAGuard guard(x.device());
  check_rc(mslk_b200_quantize_nvfp4_dt(x2.data_ptr(), x.dtype() == at::kHalf ? MSLK_B200_F16 : MSLK_B200_BF16, M, K, x2.stride(0),
                                       gs.defined() ? gs.data_ptr<float>() : nullptr,
                                    q.data_ptr(), s.data_ptr(), stream_of(x)),
           "quantize_nvfp4");
  std::vector<int64_t> qshape(x.sizes().begin(), x.sizes().end() - 2), sshape = qshape;
  qshape.push_back(-1);
  qshape.push_back(K / 2);
  sshape.push_back(-1);
  sshape.push_back(pc);
  return {q.view(qshape), s.view(sshape)};
}

// Status word of the current device: 0, or the code left by a kernel whose bounded pipeline wait expired /
// that skipped an out-of-range index.  Synchronises the device and clears the word; not for use under capture.
int64_t device_status() {
  int st = 0;
  check_rc(mslk_b200_device_status(&st), "device_status");
  return st;
}

}  // namespace

TORCH_LIBRARY_FRAGMENT(mslk, m) {
  m.def("device_status() -> int", device_status);
  m.def(
      "f8f8bf16_rowwise(Tensor XQ, Tensor WQ, Tensor x_scale, Tensor w_scale, Tensor? bias=None, bool "
      "use_fast_accum=True) -> Tensor");
  m.def(
      "f8f8bf16_rowwise_out(Tensor XQ, Tensor WQ, Tensor x_scale, Tensor w_scale, Tensor(a!) output, Tensor? "
      "bias=None, bool use_fast_accum=True) -> ()");
  m.def(
      "f8f8bf16_rowwise_batched(Tensor XQ, Tensor WQ, Tensor x_scale, Tensor w_scale, Tensor? bias=None, bool "
      "use_fast_accum=True, Tensor(a!)? output=None) -> Tensor");
  m.def(
      "f8f8bf16_rowwise_grouped_stacked(Tensor XQ, Tensor WQ, Tensor x_scale, Tensor w_scale, Tensor M_sizes) -> "
      "Tensor");
  m.def(
      "f4f4bf16(Tensor XQ, Tensor WQ, Tensor x_scale, Tensor w_scale, Tensor? output=None, Tensor? global_scale=None, "
      "int mxfp4_block_size=32) -> Tensor");
  m.def(
      "quantize_fp8_row(Tensor a, Tensor? scale_ub=None, Tensor? zero_start_index_M=None, int? align_rows_to=None, "
      "float eps=0.001953125) -> (Tensor, Tensor)");
  m.def("quantize_fp8_per_row(Tensor a, Tensor? scale_ub=None) -> (Tensor, Tensor)");
  m.def("quantize_nvfp4(Tensor x, Tensor? global_scale=None) -> (Tensor, Tensor)");
}

// The same functions under the CPU key, as the reference does (csrc/gemm/gemm_ops.cpp:187-233),
// so that a call with CPU tensors reaches the checks above and fails with their message.
TORCH_LIBRARY_IMPL(mslk, CPU, m) {
  m.impl("f8f8bf16_rowwise", f8f8bf16_rowwise);
  m.impl("f8f8bf16_rowwise_out", f8f8bf16_rowwise_out);
  m.impl("f8f8bf16_rowwise_batched", f8f8bf16_rowwise_batched);
  m.impl("f8f8bf16_rowwise_grouped_stacked", f8f8bf16_rowwise_grouped_stacked);
  m.impl("f4f4bf16", f4f4bf16);
  m.impl("quantize_fp8_row", quantize_fp8_row);
  m.impl("quantize_fp8_per_row", quantize_fp8_per_row);
  m.impl("quantize_nvfp4", quantize_nvfp4);
}

TORCH_LIBRARY_IMPL(mslk, CUDA, m) {
  m.impl("f8f8bf16_rowwise", f8f8bf16_rowwise);
  m.impl("f8f8bf16_rowwise_out", f8f8bf16_rowwise_out);
  m.impl("f8f8bf16_rowwise_batched", f8f8bf16_rowwise_batched);
  m.impl("f8f8bf16_rowwise_grouped_stacked", f8f8bf16_rowwise_grouped_stacked);
  m.impl("f4f4bf16", f4f4bf16);
  m.impl("quantize_fp8_row", quantize_fp8_row);
  m.impl("quantize_fp8_per_row", quantize_fp8_per_row);
  m.impl("quantize_nvfp4", quantize_nvfp4);
}
