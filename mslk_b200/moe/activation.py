"""SwiGLU activation, optionally fused with per-row FP8 quantization, with the reference's symbols.

Mirrors ``mslk/moe/activation.py``: ``silu_mul`` (:25-69), ``silu_mul_quant`` (:72-133) and the
operators ``mslk::silu_mul`` / ``mslk::silu_mul_quant`` (:137-176) with the same schemas.  The work is
done by the sm_100a kernels behind ``mslk_b200_silu_mul`` / ``mslk_b200_silu_mul_quant``.  CPU tensors
raise: there is no fallback path (the reference has none either).
"""

from typing import Optional

import torch

from .. import ops as _ops

FP8_DTYPE = torch.float8_e4m3fn


def silu_mul(x0: torch.Tensor, x1: torch.Tensor, valid_token_count: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``y = x0 * sigmoid(x0) * x1`` for ``(T, D)`` inputs; ``valid_token_count`` (shape ``(1,)``) bounds the rows."""
    return _ops.silu_mul(x0, x1, valid_token_count)


def silu_mul_quant(
    x0: torch.Tensor,
    x1: torch.Tensor,
    scale_ub: Optional[torch.Tensor] = None,
    valid_token_count: Optional[torch.Tensor] = None,
) -> tuple[torch.Tensor, torch.Tensor]:
    """``y, y_scale = quantize(x0 * sigmoid(x0) * x1)``: fp8 ``(T, D)`` and its inverse scale ``(T,)``."""
    return _ops.silu_mul_quant(x0, x1, scale_ub, valid_token_count)


torch.library.define("mslk::silu_mul", "(Tensor x0, Tensor x1, Tensor? valid_token_count=None) -> Tensor")
torch.library.define(
    "mslk::silu_mul_quant",
    "(Tensor x0, Tensor x1, Tensor? scale_ub=None, Tensor? valid_token_count=None) -> (Tensor, Tensor)",
)


@torch.library.impl("mslk::silu_mul", "Meta")
def silu_mul_meta(x0, x1, valid_token_count=None):
    return x0.new_empty(x0.shape)


@torch.library.impl("mslk::silu_mul", "CUDA")
def silu_mul_cuda(x0, x1, valid_token_count=None):
    return silu_mul(x0, x1, valid_token_count)


@torch.library.impl("mslk::silu_mul_quant", "Meta")
def silu_mul_quant_meta(x0, x1, scale_ub=None, valid_token_count=None):
    # Two outputs, as the schema declares (the reference's shape function returns the first only).
    return (torch.empty(x0.shape, device=x0.device, dtype=FP8_DTYPE),
            torch.empty((x0.shape[0],), device=x0.device, dtype=torch.float32))


@torch.library.impl("mslk::silu_mul_quant", "CUDA")
def silu_mul_quant_cuda(x0, x1, scale_ub=None, valid_token_count=None):
    return silu_mul_quant(x0, x1, scale_ub, valid_token_count)
