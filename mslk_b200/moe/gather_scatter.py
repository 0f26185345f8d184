"""MoE token gather / scatter with the reference's symbols.

Mirrors ``mslk/moe/gather_scatter.py``: ``gather_scale_dense_tokens`` (:18-93),
``gather_scale_quant_dense_tokens`` (:96-169), ``scatter_add_dense_tokens`` (:172-226),
``scatter_add_padded_tokens`` (:229-282) and the four ``mslk::`` operators (:285-428) with the same
schemas.  The work is done by the sm_100a kernels of ``moe_gather_scatter.cu``; CPU tensors raise.
"""

from typing import Optional

import torch

from .. import ops as _ops

FP8_DTYPE = torch.float8_e4m3fn


def gather_scale_dense_tokens(
    x: torch.Tensor,
    token_indices: torch.Tensor,
    expert_indices: torch.Tensor,
    scores: torch.Tensor,
    valid_token_count: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Gather rows of ``x`` (T, D) along ``token_indices`` (a,) and scale each by its routing score."""
    return _ops.gather_scale_dense_tokens(x, token_indices, expert_indices, scores, valid_token_count)


def gather_scale_quant_dense_tokens(
    x: torch.Tensor,
    token_indices: torch.Tensor,
    expert_indices: torch.Tensor,
    scores: torch.Tensor,
    scale_ub: Optional[torch.Tensor] = None,
    valid_token_count: Optional[torch.Tensor] = None,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Gather, scale and quantize to FP8 with one inverse scale per output row."""
    return _ops.gather_scale_quant_dense_tokens(x, token_indices, expert_indices, scores, scale_ub, valid_token_count)


def scatter_add_dense_tokens(
    out_tokens: torch.Tensor,
    in_tokens: torch.Tensor,
    token_indices: torch.Tensor,
    valid_token_count: Optional[torch.Tensor] = None,
) -> None:
    """``out_tokens[token_indices[i]] += in_tokens[i]``."""
    _ops.scatter_add_dense_tokens(out_tokens, in_tokens, token_indices, valid_token_count)


def scatter_add_padded_tokens(
    in_tokens: torch.Tensor,
    token_counts: torch.Tensor,
    token_indices: torch.Tensor,
    out_tokens: torch.Tensor,
) -> None:
    """Scatter-add the valid rows of expert-parallel padded buffers ``in_tokens`` (EP, T_K, D)."""
    _ops.scatter_add_padded_tokens(in_tokens, token_counts, token_indices, out_tokens)


torch.library.define(
    "mslk::gather_scale_dense_tokens",
    "(Tensor x, Tensor token_indices, Tensor expert_indices, Tensor scores, Tensor? valid_token_count=None) -> Tensor",
)
torch.library.define(
    "mslk::gather_scale_quant_dense_tokens",
    "(Tensor x, Tensor token_indices, Tensor expert_indices, Tensor scores, Tensor? scale_ub=None, Tensor? valid_token_count=None) -> Tensor",
)
torch.library.define(
    "mslk::scatter_add_dense_tokens",
    "(Tensor out_tokens, Tensor in_tokens, Tensor token_indices, Tensor? valid_token_count=None) -> None",
)
torch.library.define(
    "mslk::scatter_add_padded_tokens",
    "(Tensor in_tokens, Tensor token_counts, Tensor token_indices, Tensor out_tokens) -> None",
)


@torch.library.impl("mslk::gather_scale_dense_tokens", "Meta")
def gather_scale_dense_tokens_meta(x, token_indices, expert_indices, scores, valid_token_count=None):
    return x.new_empty((token_indices.shape[0], x.shape[1]))


@torch.library.impl("mslk::gather_scale_dense_tokens", "CUDA")
def gather_scale_dense_tokens_cuda(x, token_indices, expert_indices, scores, valid_token_count=None):
    return gather_scale_dense_tokens(x, token_indices, expert_indices, scores, valid_token_count)


# The reference's schema declares ONE tensor for this operator although its implementation returns
# (fp8, scale) (mslk/moe/gather_scatter.py:325-364); the operator form here returns the fp8 tensor,
# the function form above returns both.
@torch.library.impl("mslk::gather_scale_quant_dense_tokens", "Meta")
def gather_scale_quant_dense_tokens_meta(x, token_indices, expert_indices, scores, scale_ub=None,
                                         valid_token_count=None):
    return torch.empty((token_indices.shape[0], x.shape[1]), device=x.device, dtype=FP8_DTYPE)


@torch.library.impl("mslk::gather_scale_quant_dense_tokens", "CUDA")
def gather_scale_quant_dense_tokens_cuda(x, token_indices, expert_indices, scores, scale_ub=None,
                                         valid_token_count=None):
    return gather_scale_quant_dense_tokens(x, token_indices, expert_indices, scores, scale_ub, valid_token_count)[0]


@torch.library.impl("mslk::scatter_add_dense_tokens", "Meta")
def scatter_add_dense_tokens_meta(out_tokens, in_tokens, token_indices, valid_token_count=None):
    return None


@torch.library.impl("mslk::scatter_add_dense_tokens", "CUDA")
def scatter_add_dense_tokens_cuda(out_tokens, in_tokens, token_indices, valid_token_count=None):
    return scatter_add_dense_tokens(out_tokens, in_tokens, token_indices, valid_token_count)


@torch.library.impl("mslk::scatter_add_padded_tokens", "Meta")
def scatter_add_padded_tokens_meta(in_tokens, token_counts, token_indices, out_tokens):
    return None


@torch.library.impl("mslk::scatter_add_padded_tokens", "CUDA")
def scatter_add_padded_tokens_cuda(in_tokens, token_counts, token_indices, out_tokens):
    return scatter_add_padded_tokens(in_tokens, token_counts, token_indices, out_tokens)
