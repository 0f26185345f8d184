"""NVFP4 quantization with the reference's Python symbols
(``mslk/quantize/triton/fp4_quantize.py:40-43`` re-exporting ``quantize_kernels/nvfp4.py:62-149``)."""

from typing import Optional

import torch

from ... import gemm as _gemm  # noqa: F401  loads the operator library
from .fp4_utils import _from_blocked, _to_blocked, global_scale_nvfp4  # noqa: F401


def triton_quantize_nvfp4(
    x: torch.Tensor,
    global_scale: Optional[torch.Tensor],
    use_e8m0_scale: bool = False,
    use_precise_math: bool = True,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Quantize a bf16 tensor to NVFP4: packed e2m1 bytes (viewed as float4_e2m1fn_x2) and
    e4m3 block scales in the 128x4 swizzled layout.  Only the e4m3-scale, precise-math mode of
    the reference is implemented (its defaults)."""
    if use_e8m0_scale or not use_precise_math:
        raise NotImplementedError("only use_e8m0_scale=False, use_precise_math=True is implemented")
    assert x.shape[-1] % 16 == 0, "N must be divisible by 16 for NVFP4 quantization"
    xq, scales = torch.ops.mslk.quantize_nvfp4(x, global_scale)
    if hasattr(torch, "float4_e2m1fn_x2"):
        xq = xq.view(torch.float4_e2m1fn_x2)
    return xq, scales


from .fp4_primitives import RoundingMode  # noqa: E402,F401  (the reference re-exports it here)


def triton_quantize_mx4_unpack(input: torch.Tensor, group_size: int = 32, ebits: int = 2, mbits: int = 1,
                               rounding_mode: int = 4, stochastic_casting: bool = False, *, seed=None):
    """MXFP4 quantize with the reference's symbol (``mslk/quantize/triton/fp4_quantize.py:46-90``): packed e2m1 bytes
    ``[..., K // 2]`` and flattened swizzled e8m0 scales (int8).  Rounding modes nearest (0), floor (1), even (2) and
    ceil (4, the default) are implemented; stochastic raises."""
    from ... import ops as _ops
    if ebits != 2 or mbits != 1:
        raise NotImplementedError(f"triton_quantize_mx4_unpack: only E2M1 (ebits=2, mbits=1) is supported, got ebits={ebits}, mbits={mbits}.")
    if stochastic_casting:
        raise NotImplementedError("stochastic rounding is not implemented by this library")
    xq, scale = _ops.quantize_mx4(input, group_size, int(rounding_mode))
    return xq.reshape(list(input.shape[:-1]) + [-1]), scale


def triton_quantize_mx4(input: torch.Tensor, *, rounding_mode: int = 4, seed=None):
    """``mslk/quantize/triton/fp4_quantize.py:93-120``: group size 32."""
    return triton_quantize_mx4_unpack(input, 32, rounding_mode=rounding_mode)


def calculate_group_max(input: torch.Tensor, m_sizes: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-group NVFP4 global scales for stacked MoE activations
    (``mslk/quantize/triton/legacy/global_scale.py:156-230``): ``(global_scale [G] fp32, group of each row [M] int64)``."""
    from ... import ops as _ops
    return _ops.calculate_group_max(input, m_sizes)


def nvfp4_quantize_stacked(
    m_sizes: torch.Tensor,
    input: torch.Tensor,
    global_scale: torch.Tensor,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Quantize concatenated MoE activations to NVFP4 with per-expert global scales
    (``mslk/quantize/triton/legacy/quantize_stacked.py:315-400``).  Returns the packed data ``[M, K // 2]`` and the
    padded + swizzled scale buffer in which every group starts on a 128-row boundary."""
    from ... import ops as _ops
    return _ops.nvfp4_quantize_stacked(m_sizes, input, global_scale)
