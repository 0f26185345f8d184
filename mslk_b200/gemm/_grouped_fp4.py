"""``mslk::f4f4bf16_grouped_stacked`` and ``mslk::f4f4bf16_grouped_mm`` with the reference's schemas
(``csrc/gemm/gemm_ops.cpp:109-112``), implemented over the C ABI; NVFP4 mode only."""

from typing import Optional

import torch

from .. import ops as _ops

torch.library.define(
    "mslk::f4f4bf16_grouped_stacked",
    "(Tensor XQ, Tensor WQ, Tensor x_scale, Tensor w_scale, Tensor M_sizes, Tensor? global_scale=None, "
    "Tensor? starting_row_after_padding=None, bool use_mx=True) -> Tensor",
)
torch.library.define(
    "mslk::f4f4bf16_grouped_mm",
    "(Tensor XQ, Tensor WQ, Tensor x_scale, Tensor w_scale, Tensor offsets, Tensor(a!)? output=None, "
    "Tensor(a!)? global_scale=None) -> Tensor",
)


@torch.library.impl("mslk::f4f4bf16_grouped_stacked", "CUDA")
def _grouped_stacked_cuda(XQ, WQ, x_scale, w_scale, M_sizes, global_scale=None, starting_row_after_padding=None,
                          use_mx=True):
    return _ops.f4f4bf16_grouped_stacked(XQ, WQ, x_scale, w_scale, M_sizes, global_scale, starting_row_after_padding,
                                         use_mx)


@torch.library.impl("mslk::f4f4bf16_grouped_stacked", "Meta")
def _grouped_stacked_meta(XQ, WQ, x_scale, w_scale, M_sizes, global_scale=None, starting_row_after_padding=None,
                          use_mx=True):
    return torch.empty((XQ.shape[0], WQ.shape[1]), dtype=torch.bfloat16, device=XQ.device)


@torch.library.impl("mslk::f4f4bf16_grouped_mm", "CUDA")
def _grouped_mm_cuda(XQ, WQ, x_scale, w_scale, offsets, output=None, global_scale=None):
    return _ops.f4f4bf16_grouped_mm(XQ, WQ, x_scale, w_scale, offsets, output, global_scale)


@torch.library.impl("mslk::f4f4bf16_grouped_mm", "Meta")
def _grouped_mm_meta(XQ, WQ, x_scale, w_scale, offsets, output=None, global_scale: Optional[torch.Tensor] = None):
    if WQ.dim() == 2:   # 2D-2D: groups along K, one [M, N] product per group
        return torch.empty((offsets.shape[0], XQ.shape[0], WQ.shape[-1]), dtype=torch.bfloat16, device=XQ.device)
    return torch.empty((XQ.shape[0], WQ.shape[-1]), dtype=torch.bfloat16, device=XQ.device)
