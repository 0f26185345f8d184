"""``quantize_mx4`` with the reference's signature (``mslk/quantize/triton/quantize_kernels/mx4.py:217-355``)."""
from typing import Optional, Union

import torch

from ..fp4_primitives import RoundingMode


def quantize_mx4(x: torch.Tensor, group_size: int = 32, rounding_mode: Union[RoundingMode, int] = RoundingMode.ceil, *,
                 seed: Optional[int] = None) -> tuple[torch.Tensor, torch.Tensor]:
    """bf16 / fp16 ``[..., N]`` -> packed e2m1 ``[..., N // 2]`` (uint8) and flattened swizzled e8m0 scales (int8,
    ``roundup(M, 128) * roundup(N / group_size, 4)`` bytes).  Rounding modes nearest, floor, even, stochastic (``seed``, by
    default the CUDA generator's initial seed) and ceil."""
    from .... import ops as _ops
    return _ops.quantize_mx4(x, group_size, int(rounding_mode), seed)
