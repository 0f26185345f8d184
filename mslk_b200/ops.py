"""Tensor-level wrappers over the C ABI (ctypes).

These functions take CUDA tensors, allocate outputs with torch's caching
allocator, and enqueue the kernels on torch's current stream of the tensors'
device.  They keep the argument meaning and error behaviour of the reference
operators they stand for:

* ``quantize_fp8_row``       -- ``mslk/quantize/triton/fp8_quantize.py:210-316,319-378``
* ``f8f8bf16_rowwise``       -- ``csrc/gemm/cutlass/f8f8bf16_rowwise.cu:183-206``
* ``f8f8bf16_rowwise_batched`` -- ``csrc/gemm/cutlass/f8f8bf16_rowwise_batched.cu:20-139``
* ``f8f8bf16_rowwise_grouped_stacked`` -- ``csrc/gemm/cutlass/f8f8bf16_rowwise_grouped.cu:342-368``
* ``quantize_nvfp4``         -- ``mslk/quantize/triton/quantize_kernels/nvfp4.py:62-149``
* ``f4f4bf16``               -- ``csrc/gemm/cutlass/f4f4bf16.cu:6413-6473``
* ``f4f4bf16_grouped_stacked`` / ``f4f4bf16_grouped_mm`` -- ``csrc/gemm/cutlass/f4f4bf16_grouped.cu:321-475``
* ``calculate_group_max`` / ``nvfp4_quantize_stacked`` -- ``mslk/quantize/triton/legacy/global_scale.py:156-230``,
  ``legacy/quantize_stacked.py:315-400``
* ``silu_mul`` / ``silu_mul_quant`` -- ``mslk/moe/activation.py:25-69,72-133``
* ``gather_scale_dense_tokens``, ``gather_scale_quant_dense_tokens``, ``scatter_add_dense_tokens``,
  ``scatter_add_padded_tokens`` -- ``mslk/moe/gather_scatter.py:18-282``

CPU tensors are rejected: there is no fallback path.
"""

from __future__ import annotations

import math
from typing import Optional

import torch

from ._lib import check, lib

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
FP8_DTYPE = torch.float8_e4m3fn


def _require_cuda(name: str, *tensors: Optional[torch.Tensor]) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError(f"{name}: expected CUDA tensors (mslk_b200 has no CPU path), got {t.device}")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"{name}: all tensors must be on the same device ({dev} vs {t.device})")
    assert dev is not None
    return dev


def _stream(dev: torch.device) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


# --------------------------------------------------------------------------- FP8 row quantize

def quantize_fp8_row(
    a: torch.Tensor,
    scale_ub: Optional[torch.Tensor] = None,
    zero_start_index_M: Optional[torch.Tensor] = None,
    align_rows_to: Optional[int] = None,
    eps_opt: Optional[float] = 1.0 / 512.0,
):
    """Per-row e4m3 quantization; returns ``(a_fp8 [..., K_out], a_scale [...] fp32)``."""
    if scale_ub is not None and scale_ub.device != a.device:
        raise Exception("'scale_ub' must be on the same device as 'a'")
    if zero_start_index_M is not None and zero_start_index_M.device != a.device:
        raise Exception("'zero_start_index_M' must be on the same device as 'a'")
    assert a.dim() <= 4, "Only up to 4 dimension input tensor is supported."
    dev = _require_cuda("quantize_fp8_row", a, scale_ub, zero_start_index_M)
    if a.dtype not in _DTYPE_CODE:
        raise RuntimeError(f"quantize_fp8_row: unsupported input dtype {a.dtype}")
    out_shape = list(a.shape)
    a4 = a
    while a4.dim() < 4:
        a4 = a4.unsqueeze(0)
    B, M, N, K = a4.shape
    K_out = K
    if align_rows_to is not None:
        K_out = (K + align_rows_to - 1) // align_rows_to * align_rows_to
        out_shape[-1] = K_out
    zs = None
    if zero_start_index_M is not None:
        zs = zero_start_index_M.reshape(B, M).to(torch.int64).contiguous()
    ub = None
    if scale_ub is not None:
        ub = scale_ub if scale_ub.dtype == torch.float32 else scale_ub.to(torch.float32)
    eps = 1e-12 if eps_opt is None else float(eps_opt)
    q = torch.empty(out_shape, dtype=FP8_DTYPE, device=dev)
    s = torch.empty(out_shape[:-1], dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        check(lib.mslk_b200_quantize_fp8_row(
            _ptr(a4), _DTYPE_CODE[a.dtype], B, M, N, K, K_out,
            a4.stride(0), a4.stride(1), a4.stride(2), a4.stride(3),
            _ptr(ub), _ptr(zs), eps, _ptr(q), _ptr(s), _stream(dev)), "quantize_fp8_row")
    return q, s


# --------------------------------------------------------------------------- FP8 rowwise GEMM

def _check_rowwise_args(name, XQ, WQ, x_scale, w_scale):
    dev = _require_cuda(name, XQ, WQ, x_scale, w_scale)
    if XQ.dtype != FP8_DTYPE or WQ.dtype != FP8_DTYPE:
        raise RuntimeError(f"{name}: XQ and WQ must be float8_e4m3fn")
    if not (XQ.is_contiguous() and WQ.is_contiguous()):
        raise RuntimeError(f"{name}: XQ and WQ must be contiguous")
    if x_scale.dtype != torch.float32 or w_scale.dtype != torch.float32:
        raise RuntimeError(f"{name}: x_scale and w_scale must be float32")
    return dev


def f8f8bf16_rowwise_out(XQ, WQ, x_scale, w_scale, output, bias=None, use_fast_accum: bool = True) -> None:
    """``output[M,N] = bf16((XQ @ WQ.T) * x_scale[:,None] * w_scale[None,:] + bias)``.
    ``use_fast_accum`` is accepted for signature parity and has no effect (as on the
    reference's sm_100 path)."""
    dev = _check_rowwise_args("f8f8bf16_rowwise", XQ, WQ, x_scale, w_scale)
    _require_cuda("f8f8bf16_rowwise", XQ, output)
    K = XQ.shape[-1]
    M = math.prod(XQ.shape[:-1])
    N = math.prod(WQ.shape[:-1])
    if WQ.shape[-1] != K:
        raise RuntimeError(f"f8f8bf16_rowwise: K mismatch ({K} vs {WQ.shape[-1]})")
    if x_scale.numel() != M or w_scale.numel() != N:
        raise RuntimeError("f8f8bf16_rowwise: scale sizes must match M and N")
    if output.dtype != torch.bfloat16 or output.numel() != M * N or not output.is_contiguous():
        raise RuntimeError("f8f8bf16_rowwise: output must be a contiguous bfloat16 tensor of M*N elements")
    kind = 0
    if bias is not None:
        _require_cuda("f8f8bf16_rowwise", XQ, bias)
        if bias.dtype == torch.float32:
            kind = 1
        elif bias.dtype == torch.bfloat16:
            kind = 2
        else:
            raise RuntimeError("f8f8bf16_rowwise: bias must be float32 or bfloat16")
        if bias.numel() != N:
            raise RuntimeError("f8f8bf16_rowwise: bias must have N elements")
        bias = bias.contiguous()
    xs, ws = x_scale.contiguous(), w_scale.contiguous()
    with torch.cuda.device(dev):
        check(lib.mslk_b200_f8f8bf16_rowwise(
            _ptr(XQ), _ptr(WQ), _ptr(xs), _ptr(ws), _ptr(bias), kind, _ptr(output), M, N, K, _stream(dev)),
            "f8f8bf16_rowwise")


def f8f8bf16_rowwise(XQ, WQ, x_scale, w_scale, bias=None, use_fast_accum: bool = True) -> torch.Tensor:
    dev = _check_rowwise_args("f8f8bf16_rowwise", XQ, WQ, x_scale, w_scale)
    N = math.prod(WQ.shape[:-1])
    out = torch.empty((*XQ.shape[:-1], N), dtype=torch.bfloat16, device=dev)
    f8f8bf16_rowwise_out(XQ, WQ, x_scale, w_scale, out, bias, use_fast_accum)
    return out


def f8f8bf16_rowwise_batched(XQ, WQ, x_scale, w_scale, bias=None, use_fast_accum: bool = True,
                             output: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``y[b] = f8f8bf16_rowwise(XQ[b], WQ[b], x_scale[b], w_scale[b], bias[b])`` in one launch.
    ``XQ [B,M,K]``, ``WQ [B,N,K]``, ``x_scale [B,M]``, ``w_scale [B,N]``, fp32 ``bias [B,N]``."""
    name = "f8f8bf16_rowwise_batched"
    if not use_fast_accum:
        raise RuntimeError("f8f8bf16_rowwise_batched only supports fast_accum=True")
    if XQ.dim() != 3 or WQ.dim() != 3:
        raise RuntimeError("FP8 rowwise batched GEMM only supports 3D inputs")
    dev = _check_rowwise_args(name, XQ, WQ, x_scale, w_scale)
    B, M, K = XQ.shape
    N = WQ.shape[1]
    if WQ.shape[0] != B:
        raise RuntimeError(f"{name}: XQ and WQ disagree on the batch count")
    if M == 0 or N == 0 or K == 0:
        return torch.zeros((B, M, N), dtype=torch.bfloat16, device=dev)
    if WQ.shape[2] != K:
        raise RuntimeError(f"{name}: XQ and WQ disagree on K")
    if x_scale.numel() != B * M or w_scale.numel() != B * N:
        raise RuntimeError(f"{name}: scale sizes must match B*M and B*N")
    kind = 0
    if bias is not None:
        _require_cuda(name, XQ, bias)
        if bias.dtype != torch.float32:
            raise RuntimeError("Bias type must be float32 if provided.")
        if bias.numel() != B * N:
            raise RuntimeError(f"{name}: bias must have B*N elements")
        bias = bias.contiguous()
        kind = 1
    _require_cuda(name, XQ, output)
    if output is None:
        output = torch.empty((B, M, N), dtype=torch.bfloat16, device=dev)
    elif output.dtype != torch.bfloat16 or output.numel() != B * M * N or not output.is_contiguous():
        raise RuntimeError(f"{name}: output must be a contiguous bfloat16 tensor of B*M*N elements")
    xs, ws = x_scale.contiguous(), w_scale.contiguous()
    with torch.cuda.device(dev):
        check(lib.mslk_b200_f8f8bf16_rowwise_batched(
            _ptr(XQ), _ptr(WQ), _ptr(xs), _ptr(ws), _ptr(bias), kind, _ptr(output), B, M, N, K, _stream(dev)), name)
    return output


def f8f8bf16_rowwise_grouped_stacked(XQ, WQ, x_scale, w_scale, M_sizes) -> torch.Tensor:
    """Stacked grouped GEMM: ``XQ [total_M,K]``, ``WQ [G,N,K]``, ``M_sizes`` int64 [G] on the device."""
    name = "f8f8bf16_rowwise_grouped_stacked"
    dev = _check_rowwise_args(name, XQ, WQ, x_scale, w_scale)
    if M_sizes.device != XQ.device:
        raise RuntimeError(f"{name}: M_sizes must be on same device as inputs.")
    if M_sizes.dtype != torch.int64:
        raise RuntimeError(f"{name}: M_sizes must be int64.")
    if WQ.dim() != 3 or WQ.shape[0] != M_sizes.numel():
        raise RuntimeError(f"{name}: WQ must be [G,N,K] with G == M_sizes.numel()")
    if XQ.dim() != 2 or XQ.shape[1] != WQ.shape[2]:
        raise RuntimeError(f"{name}: XQ must be [total_M,K] with the K of WQ")
    G, N, K = WQ.shape
    total_M = XQ.shape[0]
    if x_scale.numel() != total_M or w_scale.numel() != G * N:
        raise RuntimeError(f"{name}: scale sizes must match total_M and G*N")
    y = torch.empty((total_M, N), dtype=torch.bfloat16, device=dev)
    if total_M == 0:
        return y
    xs, ws, ms = x_scale.contiguous(), w_scale.contiguous(), M_sizes.contiguous()
    with torch.cuda.device(dev):
        check(lib.mslk_b200_f8f8bf16_rowwise_grouped_stacked(
            _ptr(XQ), _ptr(WQ), _ptr(xs), _ptr(ws), _ptr(ms), G, total_M, N, K, _ptr(y), _stream(dev)), name)
    return y


def f8f8bf16_rowwise_grouped_stacked_scatter_add(XQ, WQ, x_scale, w_scale, M_sizes, output, scatter_add_indices) -> torch.Tensor:
    """The stacked grouped GEMM with the combine fused in: ``output[scatter_add_indices[r]] += product[r]`` (atomic, bf16)."""
    name = "f8f8bf16_rowwise_grouped_stacked_scatter_add"
    dev = _check_rowwise_args(name, XQ, WQ, x_scale, w_scale)
    _require_cuda(name, XQ, M_sizes, output, scatter_add_indices)
    if M_sizes.dtype != torch.int64:
        raise RuntimeError(f"{name}: M_sizes must be int64.")
    if WQ.dim() != 3 or WQ.shape[0] != M_sizes.numel():
        raise RuntimeError(f"{name}: WQ must be [G,N,K] with G == M_sizes.numel()")
    if XQ.dim() != 2 or XQ.shape[1] != WQ.shape[2]:
        raise RuntimeError(f"{name}: XQ must be [total_M,K] with the K of WQ")
    G, N, K = WQ.shape
    total_M = XQ.shape[0]
    if x_scale.numel() != total_M or w_scale.numel() != G * N:
        raise RuntimeError(f"{name}: scale sizes must match total_M and G*N")
    assert scatter_add_indices.is_contiguous()
    assert scatter_add_indices.shape == (total_M,)
    if output.dtype != torch.bfloat16 or output.dim() != 2 or output.shape[1] != N or not output.is_contiguous():
        raise RuntimeError(f"{name}: output must be a contiguous bfloat16 [rows, N] tensor")
    if total_M == 0 or N == 0:
        return output
    xs, ws, ms = x_scale.contiguous(), w_scale.contiguous(), M_sizes.contiguous()
    with torch.cuda.device(dev):
        check(lib.mslk_b200_f8f8bf16_rowwise_grouped_stacked_scatter_add(
            _ptr(XQ), _ptr(WQ), _ptr(xs), _ptr(ws), _ptr(ms), G, total_M, N, K, _ptr(scatter_add_indices),
            _index_bits(name, scatter_add_indices), _ptr(output), output.shape[0], _stream(dev)), name)
    return output


# --------------------------------------------------------------------------- NVFP4

def nvfp4_scale_shape(rows: int, K: int):
    return ((rows + 127) // 128 * 128, (K // 16 + 3) // 4 * 4)


def _check_nvfp4_scale_extent(name: str, arg: str, scale: torch.Tensor, rows: int, K: int, groups: int = 1,
                              block: int = 16) -> None:
    """The kernels bulk-copy whole 512-byte atoms of the swizzled scale layout, padded to
    ``[roundup(rows, 128), roundup(K/block, 4)]`` per group: a shorter tensor would be read past its end."""
    if scale.element_size() != 1:
        raise RuntimeError(f"{name}: {arg} must be a 1-byte (e4m3 / e8m0) tensor, got {scale.dtype}")
    pr, pc = (rows + 127) // 128 * 128, (K // block + 3) // 4 * 4
    need = groups * pr * pc
    if scale.numel() < need:
        raise RuntimeError(f"{name}: {arg} holds {scale.numel()} scales; the padded swizzled layout needs {need}")


def quantize_nvfp4(x: torch.Tensor, global_scale: Optional[torch.Tensor]):
    """Returns ``(xq uint8 [..., K/2], scales float8_e4m3fn [rows_pad, cols_pad] swizzled)``."""
    dev = _require_cuda("quantize_nvfp4", x, global_scale)
    if x.dtype not in (torch.bfloat16, torch.float16):
        raise RuntimeError(f"quantize_nvfp4: input must be bfloat16 or float16, got {x.dtype}")
    lead, K = x.shape[:-2], x.shape[-1]
    x2 = x.reshape(-1, K)
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    M = x2.shape[0]
    assert K % 16 == 0, "N must be divisible by 16 for NVFP4 quantization"
    pr, pc = nvfp4_scale_shape(M, K)
    q = torch.empty((M, K // 2), dtype=torch.uint8, device=dev)
    s = torch.empty((pr, pc), dtype=FP8_DTYPE, device=dev)
    gs = None
    if global_scale is not None:
        gs = global_scale.reshape(-1).to(torch.float32)
    with torch.cuda.device(dev):
        check(lib.mslk_b200_quantize_nvfp4_dt(_ptr(x2), _DTYPE_CODE[x2.dtype], M, K, x2.stride(0), _ptr(gs), _ptr(q), _ptr(s), _stream(dev)),
              "quantize_nvfp4")
    return q.view(*lead, -1, K // 2), s.view(*lead, -1, pc)


def _mx4_seed(seed, rounding_mode: int, dev) -> int:
    """The seed the reference hands its kernel (``mslk/quantize/triton/quantize_kernels/__init__.py:20-44``): 0 unless
    the mode is stochastic; else the caller's seed, or the CUDA generator's initial seed, masked to 63 bits."""
    if int(rounding_mode) != 3:
        return 0
    if seed is None:
        seed = torch.cuda.default_generators[dev.index].initial_seed()
    return int(seed) & ((1 << 63) - 1)


def quantize_mx4(x: torch.Tensor, group_size: int = 32, rounding_mode: int = 4, seed=None):
    """MXFP4 quantize (``mslk/quantize/triton/quantize_kernels/mx4.py:216-355``): ``(xq uint8 [..., K/2], scales int8,
    flattened swizzled [roundup(M,128) * roundup(K/group,4)])``.  ``rounding_mode``: 0 nearest, 1 floor, 2 even,
    3 stochastic (``seed``, default the CUDA generator's initial seed), 4 ceil."""
    name = "quantize_mx4"
    dev = _require_cuda(name, x)
    if x.dtype not in (torch.bfloat16, torch.float16):
        raise RuntimeError(f"Expected fp16/bf16, got {x.dtype}")
    lead, K = x.shape[:-2], x.shape[-1]
    assert K % group_size == 0, f"N must be divisible by {group_size}, got {K}"
    x2 = x.reshape(-1, K)
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    M = x2.shape[0]
    pr, pc = (M + 127) // 128 * 128, (K // group_size + 3) // 4 * 4
    q = torch.empty((M, K // 2), dtype=torch.uint8, device=dev)
    s = torch.empty((pr * pc,), dtype=torch.int8, device=dev)
    with torch.cuda.device(dev):
        check(lib.mslk_b200_quantize_mx4_seeded(_ptr(x2), _DTYPE_CODE[x.dtype], M, K, x2.stride(0), int(group_size),
                                                int(rounding_mode), _mx4_seed(seed, rounding_mode, dev), _ptr(q), _ptr(s),
                                                _stream(dev)), name)
    return q.view(*lead, -1, K // 2), s


def quantize_mx4_stacked(m_sizes: torch.Tensor, x: torch.Tensor, group_size: int = 32, rounding_mode: int = 4, seed=None):
    """MXFP4 quantize of stacked MoE segments (``mslk/quantize/triton/quantize_kernels/mx4_stacked.py:221-360``):
    ``(xq uint8 [M, K/2], scales int8 flattened [(M + 127 G) * roundup(K/group, 4)])`` with every segment's scale rows
    starting on a 128-row boundary; padding is zero."""
    name = "quantize_mx4_stacked"
    dev = _require_cuda(name, x, m_sizes)
    if x.dtype not in (torch.bfloat16, torch.float16):
        raise RuntimeError(f"Expected fp16/bf16, got {x.dtype}")
    x2 = x.reshape(-1, x.shape[-1])
    M, K = x2.shape
    assert K % group_size == 0, f"N must be divisible by {group_size}, got {K}"
    assert m_sizes.dtype == torch.int64, f"Expected m_sizes int64, got {m_sizes.dtype}"
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    G = m_sizes.shape[0]
    pc = (K // group_size + 3) // 4 * 4
    q = torch.empty((M, K // 2), dtype=torch.uint8, device=dev)
    s = torch.empty(((M + 127 * G) * pc,), dtype=torch.int8, device=dev)
    with torch.cuda.device(dev):
        check(lib.mslk_b200_quantize_mx4_stacked_seeded(_ptr(x2), _DTYPE_CODE[x.dtype], M, K, x2.stride(0),
                                                        _ptr(m_sizes.contiguous()), G, int(group_size), int(rounding_mode),
                                                        _mx4_seed(seed, rounding_mode, dev), _ptr(q), _ptr(s),
                                                        _stream(dev)), name)
    return q, s


def f4f4bf16(XQ, WQ, x_scale, w_scale, output=None, global_scale=None, mxfp4_block_size: int = 32) -> torch.Tensor:
    """FP4 GEMM: NVFP4 when ``global_scale`` is given (e4m3 scales per 16 elements), else MXFP4 (e8m0 scales per
    ``mxfp4_block_size`` = 32 or 16 elements), as the reference operator (``csrc/gemm/cutlass/f4f4bf16.cu:6413-6473``)."""
    name = "f4f4bf16"
    dev = _require_cuda(name, XQ, WQ, x_scale, w_scale, global_scale, output)
    if mxfp4_block_size not in (16, 32):
        raise RuntimeError(f"mxfp4_block_size must be 32 or 16, got {mxfp4_block_size}")
    if not (XQ.is_contiguous() and WQ.is_contiguous() and x_scale.is_contiguous() and w_scale.is_contiguous()):
        raise RuntimeError(f"{name}: XQ, WQ, x_scale and w_scale must be contiguous")
    M, K = XQ.shape[0], XQ.shape[1] * 2
    N = WQ.shape[0]
    if WQ.shape[1] * 2 != K:
        raise RuntimeError(f"{name}: K mismatch")
    if N % 16 != 0 or K % 16 != 0:
        raise RuntimeError(f"{name}: N and K must be multiples of 16")
    block = 16 if global_scale is not None else mxfp4_block_size
    if K % 32 != 0:
        raise RuntimeError(f"{name}: K must be a multiple of 32")
    _check_nvfp4_scale_extent(name, "x_scale", x_scale, M, K, block=block)
    _check_nvfp4_scale_extent(name, "w_scale", w_scale, N, K, block=block)
    if output is None:
        output = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    elif output.dtype != torch.bfloat16 or tuple(output.shape) != (M, N) or not output.is_contiguous():
        raise RuntimeError(f"{name}: output must be a contiguous bfloat16 [M,N] tensor")
    if M == 0 or N == 0 or K == 0:
        return output.zero_()
    if global_scale is None:
        with torch.cuda.device(dev):
            check(lib.mslk_b200_f4f4bf16_mx(_ptr(_as_bytes(XQ)), _ptr(_as_bytes(WQ)), _ptr(x_scale), _ptr(w_scale), _ptr(output),
                                            M, N, K, mxfp4_block_size, _stream(dev)), name)
        return output
    gs = global_scale.reshape(-1).to(torch.float32)
    with torch.cuda.device(dev):
        wsz = lib.mslk_b200_f4f4bf16_workspace_bytes(M, N, K)   # few tokens: scratch for K splitting
        ws = torch.empty(wsz, dtype=torch.uint8, device=dev) if wsz else None
        check(lib.mslk_b200_f4f4bf16_ws(_ptr(XQ), _ptr(WQ), _ptr(x_scale), _ptr(w_scale), _ptr(gs), _ptr(output),
                                        M, N, K, _ptr(ws) if wsz else None, wsz, _stream(dev)), name)
    return output


# --------------------------------------------------------------------------- fused GEMM + all-gather

def f8f8bf16_rowwise_allgather(XQ, WQ_shard, x_scale, w_scale_shard, out_ptrs, rank: int, out_local: torch.Tensor,
                               bias_shard=None) -> torch.Tensor:
    """N-sharded GEMM whose epilogue writes this rank's ``[M, N/P]`` column block into the
    ``[M, N]`` output buffer of every rank (``out_ptrs``: device pointers of all ranks' buffers,
    e.g. ``torch.distributed._symmetric_memory`` ``buffer_ptrs``; ``out_local`` is this rank's).
    Ranks must synchronise afterwards before reading columns written by peers."""
    import ctypes
    dev = _check_rowwise_args("f8f8bf16_rowwise_allgather", XQ, WQ_shard, x_scale, w_scale_shard)
    _require_cuda("f8f8bf16_rowwise_allgather", XQ, out_local, bias_shard)
    M, K = XQ.shape
    n_local = WQ_shard.shape[0]
    world = len(out_ptrs)
    if out_local.dtype != torch.bfloat16 or tuple(out_local.shape) != (M, n_local * world) or not out_local.is_contiguous():
        raise RuntimeError("f8f8bf16_rowwise_allgather: out_local must be a contiguous bfloat16 [M, N] tensor")
    if int(out_ptrs[rank]) != out_local.data_ptr():
        raise RuntimeError("f8f8bf16_rowwise_allgather: out_ptrs[rank] must be the address of out_local")
    kind = 0
    if bias_shard is not None:
        kind = 1 if bias_shard.dtype == torch.float32 else 2
    arr = (ctypes.c_void_p * world)(*[int(p) for p in out_ptrs])
    xs, ws = x_scale.contiguous(), w_scale_shard.contiguous()
    with torch.cuda.device(dev):
        check(lib.mslk_b200_f8f8bf16_rowwise_allgather(
            _ptr(XQ), _ptr(WQ_shard), _ptr(xs), _ptr(ws), _ptr(bias_shard), kind, arr, world, rank,
            M, n_local, K, _stream(dev)), "f8f8bf16_rowwise_allgather")
    return out_local


# --------------------------------------------------------------------------- fused GEMM + reduce-scatter

def f8f8bf16_rowwise_scatter(XQ_kshard, WQ_kshard, x_scale, w_scale, stage_ptrs, rank: int) -> None:
    """K-sharded GEMM whose epilogue deposits each owner's rows of the partial product in slot
    ``rank`` of that owner's ``[world, M/world, N]`` bf16 staging buffer (``stage_ptrs``: device
    pointers of all ranks' staging buffers).  Follow with a cross-rank barrier and
    :func:`reduce_slots` on the local staging buffer."""
    import ctypes
    dev = _check_rowwise_args("f8f8bf16_rowwise_scatter", XQ_kshard, WQ_kshard, x_scale, w_scale)
    M, K = XQ_kshard.shape
    N = WQ_kshard.shape[0]
    world = len(stage_ptrs)
    arr = (ctypes.c_void_p * world)(*[int(p) for p in stage_ptrs])
    xs, ws = x_scale.contiguous(), w_scale.contiguous()
    with torch.cuda.device(dev):
        check(lib.mslk_b200_f8f8bf16_rowwise_scatter(_ptr(XQ_kshard), _ptr(WQ_kshard), _ptr(xs), _ptr(ws), arr, world,
                                                     rank, M, N, K, _stream(dev)), "f8f8bf16_rowwise_scatter")


def reduce_slots(stage: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[rows, N] = sum_s stage[s]`` for a contiguous bf16 ``[slots, rows, N]`` tensor (fp32 accumulation)."""
    dev = _require_cuda("reduce_slots", stage, out)
    slots, rows, cols = stage.shape
    if stage.dtype != torch.bfloat16 or not stage.is_contiguous():
        raise RuntimeError("reduce_slots: stage must be a contiguous bfloat16 [slots, rows, N] tensor")
    if out is None:
        out = torch.empty((rows, cols), dtype=torch.bfloat16, device=dev)
    with torch.cuda.device(dev):
        check(lib.mslk_b200_reduce_slots_bf16(_ptr(stage), slots, rows, cols, _ptr(out), _stream(dev)), "reduce_slots")
    return out


# --------------------------------------------------------------------------- NVFP4, stacked groups (MoE)

def calculate_group_max(input: torch.Tensor, m_sizes: torch.Tensor):
    """Per-group NVFP4 global scale ``2688 / max|x|`` and the group index of every row:
    ``(global_scale fp32 [G], tensor_idx int64 [M])``."""
    name = "calculate_group_max"
    dev = _require_cuda(name, input, m_sizes)
    assert input.ndim >= 1, f"input.ndim needs to be >= 1, but got {input.ndim}."
    x2 = input.reshape(1 if input.ndim == 1 else -1, input.shape[-1])
    if x2.dtype not in (torch.bfloat16, torch.float16):
        raise RuntimeError(f"{name}: input must be bfloat16 or float16, got {x2.dtype}")
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    if m_sizes.dtype != torch.int64:
        m_sizes = m_sizes.to(torch.int64)
    M, K = x2.shape
    G = m_sizes.numel()
    out = torch.empty((G,), dtype=torch.float32, device=dev)
    tensor_idx = torch.empty((M,), dtype=torch.int64, device=dev)
    with torch.cuda.device(dev):
        check(lib.mslk_b200_calculate_group_max_dt(_ptr(x2), _DTYPE_CODE[x2.dtype], M, K, x2.stride(0), _ptr(m_sizes.contiguous()), G, _ptr(out),
                                                _ptr(tensor_idx), _stream(dev)), name)
    return out, tensor_idx


def nvfp4_quantize_stacked(m_sizes: torch.Tensor, input: torch.Tensor, global_scale: torch.Tensor):
    """NVFP4 quantization of stacked groups: ``(xq [M, K/2] packed, scale [(M + 127 G), roundup(K/16, 4)] swizzled)``;
    every group's scale rows start on a 128-row boundary."""
    name = "nvfp4_quantize_stacked"
    dev = _require_cuda(name, input, m_sizes, global_scale)
    assert input.ndim >= 1, f"input.ndim needs to be >= 1, but got {input.ndim}."
    x2 = input.reshape(-1, input.shape[-1])
    M, K = x2.shape
    assert K % 16 == 0, f"K must be divisible by 16, but got {K}."
    if x2.dtype not in (torch.bfloat16, torch.float16):
        raise RuntimeError(f"{name}: input must be bfloat16 or float16, got {x2.dtype}")
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    if m_sizes.dtype != torch.int64:
        m_sizes = m_sizes.to(torch.int64)
    G = m_sizes.shape[0]
    padded_cols = (K // 16 + 3) // 4 * 4
    xq = torch.empty((M, K // 2), device=dev, dtype=torch.uint8)
    scale = torch.empty((M + G * 127, padded_cols), device=dev, dtype=torch.uint8)
    gs = global_scale.reshape(-1).to(torch.float32)
    if gs.numel() != G:
        raise RuntimeError(f"{name}: global_scale must hold one value per group")
    with torch.cuda.device(dev):
        check(lib.mslk_b200_quantize_nvfp4_stacked_dt(_ptr(x2), _DTYPE_CODE[x2.dtype], M, K, x2.stride(0), _ptr(m_sizes.contiguous()), G, _ptr(gs),
                                                   _ptr(xq), _ptr(scale), _stream(dev)), name)
    fp4 = getattr(torch, "float4_e2m1fn_x2", None)
    return (xq.view(fp4) if fp4 is not None else xq), scale.view(FP8_DTYPE)


def _as_bytes(t: torch.Tensor) -> torch.Tensor:
    return t if t.dtype == torch.uint8 else t.view(torch.uint8)


def f4f4bf16_grouped_stacked(XQ, WQ, x_scale, w_scale, M_sizes, global_scale=None, starting_row_after_padding=None,
                             use_mx: bool = True) -> torch.Tensor:
    """Grouped NVFP4 GEMM over stacked rows: ``XQ [total_M, K/2]``, ``WQ [G, N, K/2]``, fp32 ``global_scale [G]``."""
    name = "f4f4bf16_grouped_stacked"
    dev = _require_cuda(name, XQ, WQ, x_scale, w_scale, M_sizes, global_scale, starting_row_after_padding)
    # the reference's rule (csrc/gemm/cutlass/f4f4bf16_grouped.cu:321-374): MXFP4 unless use_mx is off, then NVFP4
    # with its per-group global scales
    if not use_mx and global_scale is None:
        raise RuntimeError(f"{name}: the NVFP4 mode (use_mx=False) needs global_scale")
    if use_mx and global_scale is not None:
        raise RuntimeError(f"{name}: global_scale is for the NVFP4 mode; pass use_mx=False with it")
    if M_sizes.dtype != torch.int64:
        raise RuntimeError("M_sizes must be int64.")
    if WQ.dim() != 3 or WQ.shape[0] != M_sizes.shape[0]:
        raise RuntimeError("Weights should be shape [G, N, K].")
    if not (XQ.is_contiguous() and WQ.is_contiguous() and x_scale.is_contiguous() and w_scale.is_contiguous()):
        raise RuntimeError(f"{name}: XQ, WQ, x_scale and w_scale must be contiguous")
    total_M = XQ.shape[0]
    G, N, K = WQ.shape[0], WQ.shape[1], WQ.shape[2] * 2
    srp = None
    if starting_row_after_padding is not None:
        if starting_row_after_padding.numel() % (G + 1) != 0 or starting_row_after_padding.dtype != torch.int64:
            raise RuntimeError(f"{name}: starting_row_after_padding must be int64 with a multiple of G+1 entries")
        srp = starting_row_after_padding.contiguous()
    block = 32 if use_mx else 16
    if total_M:
        _check_nvfp4_scale_extent(name, "w_scale", w_scale, N, K, groups=G, block=block)
        # the group sizes live on the device: the host can only check the smallest layout any split of total_M needs
        _check_nvfp4_scale_extent(name, "x_scale", x_scale, total_M, K, block=block)
    if use_mx:
        Y = torch.empty((total_M, N), dtype=torch.bfloat16, device=dev)
        if total_M == 0:
            return Y
        with torch.cuda.device(dev):
            check(lib.mslk_b200_f4f4bf16_grouped_stacked_mx(
                _ptr(_as_bytes(XQ)), _ptr(_as_bytes(WQ)), _ptr(x_scale), _ptr(w_scale), _ptr(M_sizes.contiguous()),
                _ptr(srp), G, total_M, N, K, 32, _ptr(Y), _stream(dev)), name)
        return Y
    gs = global_scale.reshape(-1).to(torch.float32)
    if gs.numel() != G:
        raise RuntimeError(f"{name}: global_scale must hold one value per group")
    Y = torch.empty((total_M, N), dtype=torch.bfloat16, device=dev)
    if total_M == 0:
        return Y
    with torch.cuda.device(dev):
        check(lib.mslk_b200_f4f4bf16_grouped_stacked(
            _ptr(_as_bytes(XQ)), _ptr(_as_bytes(WQ)), _ptr(x_scale), _ptr(w_scale), _ptr(M_sizes.contiguous()), _ptr(gs),
            _ptr(srp), G, total_M, N, K, _ptr(Y), _stream(dev)), name)
    return Y


def _f4f4bf16_grouped_mm_2d2d(name, dev, XQ, WQ, x_scale, w_scale, offsets, output, global_scale, nvfp4):
    G = offsets.shape[0]
    M, N, K = XQ.shape[0], WQ.shape[-1], WQ.shape[-2] * 2
    if XQ.shape[1] * 2 != K:
        raise RuntimeError("for 2d-2d grouped GEMM, XQ shape must be (M, total_K) and WQ shape must be (total_K, N).")
    if output is not None and (output.dim() != 3 or tuple(output.shape) != (G, M, N) or output.dtype != torch.bfloat16
                               or not output.is_contiguous()):
        raise RuntimeError("for 2d-2d grouped GEMM, output shape must be (G, M, N).")
    block = 16 if nvfp4 else 32
    if G and M and N:
        # every group's scale block is padded on its own, so these are lower bounds; the kernel checks the real need
        _check_nvfp4_scale_extent(name, "x_scale", x_scale, M, K, block=block)
        _check_nvfp4_scale_extent(name, "w_scale", w_scale, N, K, block=block)
    out = output if output is not None else torch.empty((G, M, N), dtype=torch.bfloat16, device=dev)
    if out.numel() == 0:
        return out
    gs = None
    if nvfp4:
        gs = global_scale.reshape(-1).to(torch.float32)
        if gs.numel() != G:
            raise RuntimeError(f"{name}: global_scale must hold one value per group")
    with torch.cuda.device(dev):
        check(lib.mslk_b200_f4f4bf16_grouped_mm_2d2d(
            _ptr(_as_bytes(XQ)), _ptr(_as_bytes(WQ.transpose(-2, -1))), _ptr(x_scale), _ptr(w_scale),
            _ptr(offsets.contiguous()), _ptr(gs), G, M, N, K, block, x_scale.numel(), w_scale.numel(), _ptr(out),
            _stream(dev)), name)
    return out


def f4f4bf16_grouped_mm(XQ, WQ, x_scale, w_scale, offsets, output=None, global_scale=None) -> torch.Tensor:
    """``torch._scaled_grouped_mm``-style grouped FP4 GEMM (NVFP4 or MXFP4 by the scale dtype), int32 END ``offsets [G]``.
    2D-3D: ``XQ [total_M, K/2]``, ``WQ [G, K/2, N]`` (the transposed view of a contiguous ``[G, N, K/2]`` tensor),
    offsets along M, output ``[total_M, N]``.  2D-2D: ``XQ [M, total_K/2]``, ``WQ [total_K/2, N]`` (transposed view of
    ``[N, total_K/2]``), offsets along K (multiples of 32), output ``[G, M, N]``
    (csrc/gemm/cutlass/f4f4bf16_grouped.cu:376-475)."""
    name = "f4f4bf16_grouped_mm"
    dev = _require_cuda(name, XQ, WQ, x_scale, w_scale, offsets, global_scale, output)
    if offsets.dtype != torch.int32:
        raise RuntimeError("offsets must be int32.")
    if offsets.dim() != 1:
        raise RuntimeError("offsets must be 1D tensor.")
    if not XQ.is_contiguous():
        raise RuntimeError("XQ must be row major.")
    if not WQ.transpose(-2, -1).is_contiguous():
        raise RuntimeError("WQ must be column major.")
    if not (x_scale.is_contiguous() and w_scale.is_contiguous()):
        raise RuntimeError("x_scale and w_scale must be contiguous.")
    # the reference tells the formats apart by the scale dtype (csrc/gemm/cutlass/f4f4bf16_grouped.cu:396-440):
    # float8_e4m3fn = NVFP4 (needs global_scale), float8_e8m0fnu = MXFP4
    nvfp4 = x_scale.dtype == FP8_DTYPE
    if nvfp4 and global_scale is None:
        raise RuntimeError(f"{name}: NVFP4 (float8_e4m3fn scales) needs global_scale")
    if not nvfp4 and global_scale is not None:
        raise RuntimeError(f"{name}: global_scale is for NVFP4 (float8_e4m3fn scales)")
    if XQ.dim() == 2 and WQ.dim() == 2:
        return _f4f4bf16_grouped_mm_2d2d(name, dev, XQ, WQ, x_scale, w_scale, offsets, output, global_scale, nvfp4)
    if XQ.dim() != 2 or WQ.dim() != 3:
        raise RuntimeError("Invalid input shapes. Must be one of 2D-2D, 2D-3D.")
    G = offsets.shape[0]
    total_M = XQ.shape[0]
    N, K = WQ.shape[-1], WQ.shape[-2] * 2
    if XQ.shape[1] * 2 != K or WQ.shape[0] != G:
        raise RuntimeError("for 2d-3d grouped GEMM, XQ shape must be (total_M, K) and WQ shape must be (G, K, N).")
    if total_M and N:
        _check_nvfp4_scale_extent(name, "w_scale", w_scale, N, K, groups=G, block=16 if nvfp4 else 32)
        _check_nvfp4_scale_extent(name, "x_scale", x_scale, total_M, K, block=16 if nvfp4 else 32)
    out = output if output is not None else torch.empty((total_M, N), dtype=torch.bfloat16, device=dev)
    if out.dim() != 2 or out.shape[0] != total_M or out.shape[1] != N or out.dtype != torch.bfloat16 or not out.is_contiguous():
        raise RuntimeError("for 2d-3d grouped GEMM, output shape must be (total_M, N).")
    if out.numel() == 0:
        return out
    wq = WQ.transpose(-2, -1)
    if not nvfp4:
        with torch.cuda.device(dev):
            check(lib.mslk_b200_f4f4bf16_grouped_mm_mx(
                _ptr(_as_bytes(XQ)), _ptr(_as_bytes(wq)), _ptr(x_scale), _ptr(w_scale), _ptr(offsets.contiguous()),
                G, total_M, N, K, 32, _ptr(out), _stream(dev)), name)
        return out
    gs = global_scale.reshape(-1).to(torch.float32)
    if gs.numel() != G:
        raise RuntimeError(f"{name}: global_scale must hold one value per group")
    with torch.cuda.device(dev):
        check(lib.mslk_b200_f4f4bf16_grouped_mm(
            _ptr(_as_bytes(XQ)), _ptr(_as_bytes(wq)), _ptr(x_scale), _ptr(w_scale), _ptr(offsets.contiguous()), _ptr(gs),
            G, total_M, N, K, _ptr(out), _stream(dev)), name)
    return out


# --------------------------------------------------------------------------- SwiGLU (+ FP8 row quantize)

def _check_silu_args(name, x0, x1, valid_token_count):
    assert x0.ndim == 2 and x0.stride(1) == 1
    assert x1.ndim == 2 and x1.stride(1) == 1
    assert x0.shape == x1.shape
    assert x0.dtype == x1.dtype
    dev = _require_cuda(name, x0, x1, valid_token_count)
    if x0.dtype not in (torch.bfloat16, torch.float16):
        raise RuntimeError(f"{name}: inputs must be bfloat16 or float16, got {x0.dtype}")
    if valid_token_count is not None and valid_token_count.dtype != torch.int32:
        valid_token_count = valid_token_count.to(torch.int32)
    return dev, valid_token_count


def silu_mul(x0: torch.Tensor, x1: torch.Tensor, valid_token_count: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x0 * sigmoid(x0) * x1`` for ``[T, D]`` inputs; rows at or past ``valid_token_count`` are not written."""
    dev, vtc = _check_silu_args("silu_mul", x0, x1, valid_token_count)
    T, D = x0.shape
    out = torch.empty((T, D), dtype=x0.dtype, device=dev)
    with torch.cuda.device(dev):
        check(lib.mslk_b200_silu_mul(_ptr(x0), _ptr(x1), _DTYPE_CODE[x0.dtype], T, D, x0.stride(0), x1.stride(0),
                                     _ptr(vtc), _ptr(out), _stream(dev)), "silu_mul")
    return out


def silu_mul_quant(x0: torch.Tensor, x1: torch.Tensor, scale_ub: Optional[torch.Tensor] = None,
                   valid_token_count: Optional[torch.Tensor] = None):
    """Fused ``quantize_fp8_row(x0 * sigmoid(x0) * x1)``: returns ``(y_fp8 [T, D], inverse scale fp32 [T])``."""
    dev, vtc = _check_silu_args("silu_mul_quant", x0, x1, valid_token_count)
    _require_cuda("silu_mul_quant", x0, scale_ub)
    ub = None
    if scale_ub is not None:
        ub = scale_ub if scale_ub.dtype == torch.float32 else scale_ub.to(torch.float32)
    T, D = x0.shape
    out = torch.empty((T, D), dtype=FP8_DTYPE, device=dev)
    inv_scale = torch.empty((T,), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        check(lib.mslk_b200_silu_mul_quant(_ptr(x0), _ptr(x1), _DTYPE_CODE[x0.dtype], T, D, x0.stride(0),
                                           x1.stride(0), _ptr(ub), _ptr(vtc), _ptr(out), _ptr(inv_scale),
                                           _stream(dev)), "silu_mul_quant")
    return out, inv_scale


# --------------------------------------------------------------------------- MoE token gather / scatter

_SCATTER_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2, torch.int32: 3}


def _index_bits(name: str, t: torch.Tensor) -> int:
    if t.dtype == torch.int32:
        return 32
    if t.dtype == torch.int64:
        return 64
    raise RuntimeError(f"{name}: index tensors must be int32 or int64, got {t.dtype}")


def _valid_count(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    if t is not None and t.dtype != torch.int32:
        t = t.to(torch.int32)
    return t


def _gather_args(name, x, token_indices, expert_indices, scores, valid_token_count):
    dev = _require_cuda(name, x, token_indices, expert_indices, scores, valid_token_count)
    assert x.dim() == 2 and scores.dim() == 2
    T, D = x.shape
    E = scores.shape[1]
    a = token_indices.shape[0]
    assert x.is_contiguous()
    assert token_indices.is_contiguous()
    assert expert_indices.is_contiguous()
    assert tuple(token_indices.shape) == (a,)
    assert tuple(expert_indices.shape) == (a,)
    assert tuple(scores.shape) == (T, E)
    if x.dtype not in (torch.bfloat16, torch.float16):
        raise RuntimeError(f"{name}: x must be bfloat16 or float16, got {x.dtype}")
    if scores.dtype not in _DTYPE_CODE:
        raise RuntimeError(f"{name}: unsupported scores dtype {scores.dtype}")
    return dev, T, D, E, a


def gather_scale_dense_tokens(x, token_indices, expert_indices, scores, valid_token_count=None) -> torch.Tensor:
    """``out[i] = x[token_indices[i]] * scores[token_indices[i], expert_indices[i]]`` -> ``[a, D]`` in ``x.dtype``."""
    name = "gather_scale_dense_tokens"
    dev, T, D, E, a = _gather_args(name, x, token_indices, expert_indices, scores, valid_token_count)
    out = torch.empty((a, D), device=dev, dtype=x.dtype)
    if a == 0 or D == 0:
        return out
    vtc = _valid_count(valid_token_count)
    with torch.cuda.device(dev):
        check(lib.mslk_b200_gather_scale_dense_tokens(
            _ptr(x), _DTYPE_CODE[x.dtype], T, D, _ptr(token_indices), _index_bits(name, token_indices),
            _ptr(expert_indices), _index_bits(name, expert_indices), _ptr(scores), _DTYPE_CODE[scores.dtype], E,
            scores.stride(0), scores.stride(1), a, _ptr(vtc), _ptr(out), _stream(dev)), name)
    return out


def gather_scale_quant_dense_tokens(x, token_indices, expert_indices, scores, scale_ub=None, valid_token_count=None):
    """The same gather followed by per-row FP8 quantization: ``(fp8 [a, D], inverse scale fp32 [a])``."""
    name = "gather_scale_quant_dense_tokens"
    dev, T, D, E, a = _gather_args(name, x, token_indices, expert_indices, scores, valid_token_count)
    _require_cuda(name, x, scale_ub)
    out = torch.empty((a, D), device=dev, dtype=FP8_DTYPE)
    out_scale = torch.empty((a,), device=dev, dtype=torch.float32)
    if a == 0 or D == 0:
        return out, out_scale
    ub = None
    if scale_ub is not None:
        ub = scale_ub if scale_ub.dtype == torch.float32 else scale_ub.to(torch.float32)
    vtc = _valid_count(valid_token_count)
    with torch.cuda.device(dev):
        check(lib.mslk_b200_gather_scale_quant_dense_tokens(
            _ptr(x), _DTYPE_CODE[x.dtype], T, D, _ptr(token_indices), _index_bits(name, token_indices),
            _ptr(expert_indices), _index_bits(name, expert_indices), _ptr(scores), _DTYPE_CODE[scores.dtype], E,
            scores.stride(0), scores.stride(1), a, _ptr(ub), _ptr(vtc), _ptr(out), _ptr(out_scale), _stream(dev)), name)
    return out, out_scale


def scatter_add_dense_tokens(out_tokens, in_tokens, token_indices, valid_token_count=None) -> None:
    """``out_tokens[token_indices[i]] += in_tokens[i]`` (atomic adds in the tensors' dtype)."""
    name = "scatter_add_dense_tokens"
    dev = _require_cuda(name, out_tokens, in_tokens, token_indices, valid_token_count)
    assert in_tokens.is_contiguous()
    assert token_indices.is_contiguous()
    assert out_tokens.is_contiguous()
    a, D = in_tokens.shape
    if a == 0:
        return
    assert token_indices.shape == (a,)
    assert out_tokens.ndim == 2 and out_tokens.shape[1] == D
    if in_tokens.dtype != out_tokens.dtype or in_tokens.dtype not in _SCATTER_DTYPE_CODE:
        raise RuntimeError(f"{name}: in/out tokens must share a dtype of float32, bfloat16, float16 or int32")
    vtc = _valid_count(valid_token_count)
    with torch.cuda.device(dev):
        check(lib.mslk_b200_scatter_add_dense_tokens(
            _ptr(out_tokens), out_tokens.shape[0], _ptr(in_tokens), _SCATTER_DTYPE_CODE[in_tokens.dtype], a, D,
            _ptr(token_indices), _index_bits(name, token_indices), _ptr(vtc), _stream(dev)), name)


def scatter_add_padded_tokens(in_tokens, token_counts, token_indices, out_tokens) -> None:
    """``out_tokens[token_indices[i]] += in_tokens[rank(i), i]`` over the rows counted by ``token_counts``."""
    name = "scatter_add_padded_tokens"
    dev = _require_cuda(name, in_tokens, token_counts, token_indices, out_tokens)
    assert in_tokens.is_contiguous()
    assert token_counts.is_contiguous()
    assert token_indices.is_contiguous()
    assert out_tokens.is_contiguous()
    EP, T_K, D = in_tokens.shape
    E = token_counts.shape[0]
    assert tuple(token_indices.shape) == (T_K,)
    assert T_K % out_tokens.shape[0] == 0 and out_tokens.shape[1] == D
    if in_tokens.dtype != out_tokens.dtype or in_tokens.dtype not in _SCATTER_DTYPE_CODE:
        raise RuntimeError(f"{name}: in/out tokens must share a dtype of float32, bfloat16, float16 or int32")
    with torch.cuda.device(dev):
        check(lib.mslk_b200_scatter_add_padded_tokens(
            _ptr(in_tokens), _SCATTER_DTYPE_CODE[in_tokens.dtype], EP, T_K, D, _ptr(token_counts),
            _index_bits(name, token_counts), E, _ptr(token_indices), _index_bits(name, token_indices),
            _ptr(out_tokens), out_tokens.shape[0], _stream(dev)), name)
