"""NVFP4 helpers with the reference's names (``mslk/quantize/triton/legacy/fp4_utils.py``,
``legacy/primitives.py``): global scale, blocked-scale layout conversion, dequantization.
Plain torch tensor code (layout and test helpers, not the hot path)."""

import math
from typing import Tuple

import torch

FP8_E4M3_MAX = 448.0
FP4_E2M1_MAX = 6.0


def global_scale_nvfp4(x: torch.Tensor) -> torch.Tensor:
    """``(448 * 6) / amax(|x|)`` as an fp32 tensor (reference: ``legacy/fp4_utils.py:78-92``)."""
    assert x.dtype == torch.bfloat16
    amax = torch.amax(torch.abs(x)).to(torch.float32)
    return (FP8_E4M3_MAX * FP4_E2M1_MAX) / amax


def _to_blocked(x: torch.Tensor) -> torch.Tensor:
    """[rows, cols] scale matrix -> flattened 128x4-tile swizzled layout (``legacy/primitives.py:51-86``)."""
    rows, cols = x.shape
    rb, cb = (rows + 127) // 128, (cols + 3) // 4
    padded = x
    if (rows, cols) != (rb * 128, cb * 4):
        padded = torch.zeros((rb * 128, cb * 4), device=x.device, dtype=x.dtype)
        padded[:rows, :cols] = x
    return padded.view(rb, 4, 32, cb, 4).permute(0, 3, 2, 1, 4).reshape(-1, 32, 16).flatten()


def _from_blocked(x: torch.Tensor, original_shape: Tuple[int, int]) -> torch.Tensor:
    """Inverse of :func:`_to_blocked` (``legacy/primitives.py:89-119``)."""
    rows, cols = original_shape
    rb, cb = (rows + 127) // 128, (cols + 3) // 4
    padded = x.reshape(rb, cb, 32, 4, 4).permute(0, 3, 2, 1, 4).reshape(rb * 128, cb * 4)
    return padded[:rows, :cols].contiguous()


def fp4_to_float(x: torch.Tensor) -> torch.Tensor:
    """Packed e2m1 bytes -> fp32 (element 2j in the low nibble), ``legacy/fp4_utils.py:19-45``."""
    lut = torch.tensor([0, 0.5, 1, 1.5, 2, 3, 4, 6, 0, -0.5, -1, -1.5, -2, -3, -4, -6],
                       dtype=torch.float32, device=x.device)
    p = x.view(torch.uint8).to(torch.int64)
    idx = torch.stack([p & 0xF, (p >> 4) & 0xF], dim=-1).reshape(*p.shape[:-1], p.shape[-1] * 2)
    return lut[idx]


def dequantize_nvfp4(input_quantized: torch.Tensor, scale: torch.Tensor, global_scale: torch.Tensor,
                     group_size: int = 16) -> torch.Tensor:
    """Packed NVFP4 + blocked scales + global scale -> bfloat16 (``legacy/fp4_utils.py:95-120``)."""
    M = input_quantized.shape[0]
    N = input_quantized.shape[1] * 2
    s = _from_blocked(scale.reshape(-1), (M, math.ceil(N / group_size)))
    true_scale = s.view(torch.float8_e4m3fn).to(torch.float) / global_scale
    x = fp4_to_float(input_quantized)
    num_groups = N // group_size
    out = x.view(-1, num_groups, group_size) * true_scale.view(M, -1)[:, :num_groups, None]
    return out.view(x.shape).to(torch.bfloat16)
