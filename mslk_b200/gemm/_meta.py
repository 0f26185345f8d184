"""Fake (meta) kernels: output shapes and dtypes for ``torch.compile`` / ``torch.export``.

Shape rules follow the reference's ``mslk/gemm/_meta.py:28-67,68-83,116-128,234-247``.
"""

from typing import Optional

import torch


@torch.library.register_fake("mslk::f8f8bf16_rowwise")
def _f8f8bf16_rowwise_fake(XQ, WQ, x_scale, w_scale, bias: Optional[torch.Tensor] = None, use_fast_accum: bool = True):
    assert XQ.dim() in (2, 3) and WQ.dim() == 2, "The dim of XQ must be 2 or 3, and dim of WQ must be 2"
    return torch.empty((*XQ.shape[:-1], WQ.shape[0]), dtype=torch.bfloat16, device=XQ.device)


@torch.library.register_fake("mslk::f8f8bf16_rowwise_out")
def _f8f8bf16_rowwise_out_fake(XQ, WQ, x_scale, w_scale, output, bias: Optional[torch.Tensor] = None,
                               use_fast_accum: bool = True) -> None:
    return None


@torch.library.register_fake("mslk::f8f8bf16_rowwise_batched")
def _f8f8bf16_rowwise_batched_fake(XQ, WQ, x_scale, w_scale, bias: Optional[torch.Tensor] = None,
                                   use_fast_accum: bool = True, output: Optional[torch.Tensor] = None):
    return torch.empty((XQ.shape[0], XQ.shape[1], WQ.shape[1]), dtype=torch.bfloat16, device=XQ.device)


@torch.library.register_fake("mslk::f8f8bf16_rowwise_grouped_stacked")
def _f8f8bf16_rowwise_grouped_stacked_fake(XQ, WQ, x_scale, w_scale, M_sizes):
    return torch.empty((XQ.shape[0], WQ.shape[1]), dtype=torch.bfloat16, device=XQ.device)


@torch.library.register_fake("mslk::f4f4bf16")
def _f4f4bf16_fake(XQ, WQ, x_scale, w_scale, output: Optional[torch.Tensor] = None,
                   global_scale: Optional[torch.Tensor] = None, mxfp4_block_size: int = 32):
    return torch.empty((XQ.shape[0], WQ.shape[0]), dtype=torch.bfloat16, device=XQ.device)


def _quant_shapes(a, align_rows_to):
    shape = list(a.shape)
    if align_rows_to is not None:
        shape[-1] = (shape[-1] + align_rows_to - 1) // align_rows_to * align_rows_to
    return shape


@torch.library.register_fake("mslk::quantize_fp8_row")
def _quantize_fp8_row_fake(a, scale_ub=None, zero_start_index_M=None, align_rows_to=None, eps=1.0 / 512.0):
    shape = _quant_shapes(a, align_rows_to)
    return (torch.empty(shape, dtype=torch.float8_e4m3fn, device=a.device),
            torch.empty(shape[:-1], dtype=torch.float32, device=a.device))


@torch.library.register_fake("mslk::quantize_fp8_per_row")
def _quantize_fp8_per_row_fake(a, scale_ub=None):
    return (torch.empty(a.shape, dtype=torch.float8_e4m3fn, device=a.device),
            torch.empty(a.shape[:-1], dtype=torch.float32, device=a.device))


@torch.library.register_fake("mslk::quantize_nvfp4")
def _quantize_nvfp4_fake(x, global_scale=None):
    K = x.shape[-1]
    rows = x.numel() // K if K else 0
    lead = list(x.shape[:-2])
    n_lead = 1
    for d in lead:
        n_lead *= d
    pr = (rows + 127) // 128 * 128
    pc = (K // 16 + 3) // 4 * 4
    return (torch.empty((*lead, x.shape[-2], K // 2), dtype=torch.uint8, device=x.device),
            torch.empty((*lead, pr // max(1, n_lead), pc), dtype=torch.float8_e4m3fn, device=x.device))
