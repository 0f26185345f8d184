"""Per-row FP8 quantization with the reference's Python symbols.

Mirrors ``mslk/quantize/triton/fp8_quantize.py:210-407``: ``triton_quantize_fp8_row``,
the custom op ``quantize_fp8_row`` (registered as ``triton::quantize_fp8_row``) and its
shape function ``quantize_fp8_row_meta``.  The work is done by the sm_100a kernel behind
``torch.ops.mslk.quantize_fp8_row``.  Deliberate differences: ``use_triton`` is accepted
and ignored, and CPU tensors raise instead of taking a torch fallback.
"""

from typing import Optional

import torch

from ... import gemm as _gemm  # noqa: F401  loads the operator library


def triton_quantize_fp8_row(
    a: torch.Tensor,
    scale_ub: Optional[torch.Tensor] = None,
    zero_start_index_M: Optional[torch.Tensor] = None,
    align_rows_to: Optional[int] = None,
    eps_opt: Optional[float] = 1.0 / 512.0,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Quantize ``a`` (<= 4-D, last dim = row) to float8_e4m3fn with one scale per row.

    Returns ``(a_fp8, a_scale)`` with ``a_scale = max(amax, eps) / 448`` (clamped by
    ``scale_ub`` when given) and ``a_fp8 = a / a_scale``.  ``align_rows_to`` zero-pads the
    row length to a multiple; ``zero_start_index_M`` marks trailing rows of each group empty.
    """
    if scale_ub is not None and scale_ub.device != a.device:
        raise Exception("'scale_ub' must be on the same device as 'a'")
    if zero_start_index_M is not None and zero_start_index_M.device != a.device:
        raise Exception("'zero_start_index_M' must be on the same device as 'a'")
    assert a.dim() <= 4, "Triton only supports up to 4 dimension input tensor."
    eps = 1e-12 if eps_opt is None else float(eps_opt)
    return torch.ops.mslk.quantize_fp8_row(a, scale_ub, zero_start_index_M, align_rows_to, eps)


@torch.library.custom_op("triton::quantize_fp8_row", mutates_args=())
def quantize_fp8_row(
    a: torch.Tensor,
    scale_ub: Optional[torch.Tensor] = None,
    zero_start_index_M: Optional[torch.Tensor] = None,
    use_triton: bool = True,
    output_device: Optional[torch.device] = None,
    align_rows_to: Optional[int] = None,
    eps_opt: Optional[float] = 1.0 / 512.0,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Quantize ``a`` to fp8 with row-wise scalings and optionally move to ``output_device``."""
    a_fp8, a_scale = triton_quantize_fp8_row(a, scale_ub, zero_start_index_M, align_rows_to=align_rows_to,
                                             eps_opt=eps_opt)
    if output_device is not None and torch.device(output_device) != a.device:
        a_fp8, a_scale = a_fp8.to(output_device), a_scale.to(output_device)
    return a_fp8, a_scale


@quantize_fp8_row.register_fake
def quantize_fp8_row_meta(
    a: torch.Tensor,
    scale_ub: Optional[torch.Tensor] = None,
    zero_start_index_M: Optional[torch.Tensor] = None,
    use_triton: bool = True,
    output_device: Optional[torch.device] = None,
    align_rows_to: Optional[int] = None,
    eps_opt: Optional[float] = 1.0 / 512.0,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Shape function for torch compile."""
    if output_device is None:
        output_device = a.device
    shape = list(a.shape)
    if align_rows_to is not None:
        shape[-1] = (shape[-1] + align_rows_to - 1) // align_rows_to * align_rows_to
    return (torch.empty(shape, device=output_device, dtype=torch.float8_e4m3fn),
            torch.empty(shape[:-1], device=output_device, dtype=torch.float32))
