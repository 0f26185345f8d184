"""``quantize_mx4_stacked`` with the reference's signature
(``mslk/quantize/triton/quantize_kernels/mx4_stacked.py:221-360``)."""
from typing import Optional, Union

import torch

from ..fp4_primitives import RoundingMode


def quantize_mx4_stacked(m_sizes: torch.Tensor, x: torch.Tensor, group_size: int = 32,
                         rounding_mode: Union[RoundingMode, int] = RoundingMode.ceil, *,
                         seed: Optional[int] = None) -> tuple[torch.Tensor, torch.Tensor]:
    """Stacked MoE activations ``[M, N]`` with ``m_sizes`` rows per segment -> packed e2m1 ``[M, N // 2]`` and the
    flattened scale buffer of ``(M + 127 * num_segments) * roundup(N / group_size, 4)`` bytes in which every segment
    starts on a 128-row boundary (padding is zero)."""
    from .... import ops as _ops
    return _ops.quantize_mx4_stacked(m_sizes, x, group_size, int(rounding_mode), seed)
