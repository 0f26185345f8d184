"""``grouped_gemm_fp8_rowwise`` with the reference's Python signature
(``mslk/gemm/triton/grouped_gemm.py:1112-1137``), served by the sm_100a grouped kernel.

``x [M, K]`` and ``w [G * N, K]`` are float8_e4m3fn, ``m_sizes [G]`` the rows per group (any integer dtype,
on the device), ``x_scale [M]`` / ``w_scale [G * N]`` fp32.  With ``_output_tensor`` and
``_scatter_add_indices`` the product rows are added to ``_output_tensor[_scatter_add_indices[r]]``
instead of being returned stacked (the fused MoE combine)."""

from typing import Optional

import torch

from ... import ops as _ops


def grouped_gemm_fp8_rowwise(
    x: torch.Tensor,
    w: torch.Tensor,
    m_sizes: torch.Tensor,
    x_scale: torch.Tensor,
    w_scale: torch.Tensor,
    use_fast_accum: bool = True,
    *,
    _use_warp_specialization: bool = True,
    _output_tensor: Optional[torch.Tensor] = None,
    _scatter_add_indices: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    G = m_sizes.shape[0]
    assert x.is_contiguous()
    assert w.is_contiguous()
    assert m_sizes.is_contiguous()
    M, K = x.shape
    N = w.shape[0] // G
    assert K == w.shape[1]
    ms = m_sizes if m_sizes.dtype == torch.int64 else m_sizes.to(torch.int64)
    w3 = w.view(G, N, K)
    if _output_tensor is None:
        assert _scatter_add_indices is None
        return _ops.f8f8bf16_rowwise_grouped_stacked(x, w3, x_scale, w_scale, ms)
    assert _scatter_add_indices is not None
    return _ops.f8f8bf16_rowwise_grouped_stacked_scatter_add(x, w3, x_scale, w_scale, ms, _output_tensor,
                                                             _scatter_add_indices)
