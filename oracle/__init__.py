"""CPU oracle for the FP8-rowwise / NVFP4 GEMM hot path.  TEST INFRASTRUCTURE ONLY.

This package is the checker, never the product: it may be imported by the test
suite, by the smoke check and by the CPU-baseline / reference legs of the
benchmark, and by nothing under ``mslk_b200``.  It restates the reference's
arithmetic on the CPU:

* ``lowp_oracle.c`` (scalar C, loaded through ctypes) is the bit-exact
  statement of the quantizers and a slow fp32 GEMM for small cases;
* the ``*_torch`` functions below are the reference's own CPU formulas written
  with the same torch calls (fast enough for full-size parity checks and for
  timing the CPU baseline).

Parity pin: the C quantizer is checked against (i) outputs of the reference's
Triton kernels captured on a B200 and (ii) outputs of the reference's CPU torch
path captured by importing the reference; both sets live in ``tests/golden``
with the script that produced them.
"""

from __future__ import annotations

import ctypes
import math
import os
import subprocess
from typing import Optional, Sequence

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liblowp_oracle.so")
_lib = None

FP8_MAX = 448.0
DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def build(force: bool = False) -> str:
    """Compile ``lowp_oracle.c`` with the Makefile beside it; returns the .so path."""
    src = os.path.join(_HERE, "lowp_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_LIB_PATH)
        i64, vp, f32, i32 = ctypes.c_int64, ctypes.c_void_p, ctypes.c_float, ctypes.c_int
        L.oracle_f32_to_e4m3.argtypes = [f32]
        L.oracle_f32_to_e4m3.restype = ctypes.c_uint8
        L.oracle_e4m3_to_f32.argtypes = [ctypes.c_uint8]
        L.oracle_e4m3_to_f32.restype = f32
        L.oracle_f32_to_e2m1.argtypes = [f32]
        L.oracle_f32_to_e2m1.restype = ctypes.c_uint8
        L.oracle_f32_to_bf16.argtypes = [f32]
        L.oracle_f32_to_bf16.restype = ctypes.c_uint16
        L.oracle_quantize_fp8_row.argtypes = [vp, i32] + [i64] * 9 + [vp, vp, f32, vp, vp]
        L.oracle_quantize_fp8_row.restype = None
        L.oracle_quantize_fp8_row_cpu_path.argtypes = [vp, i64, i64, vp, vp, vp]
        L.oracle_quantize_fp8_row_cpu_path.restype = None
        L.oracle_gemm_f8_rowwise.argtypes = [vp, vp, vp, vp, vp, i32, i64, i64, i64, vp]
        L.oracle_gemm_f8_rowwise.restype = None
        L.oracle_gemm_f8_rowwise_grouped_stacked.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, vp]
        L.oracle_gemm_f8_rowwise_grouped_stacked.restype = None
        L.oracle_nvfp4_scale_offset.argtypes = [i64, i64, i64]
        L.oracle_nvfp4_scale_offset.restype = i64
        L.oracle_quantize_nvfp4.argtypes = [vp, i64, i64, vp, vp, vp]
        L.oracle_quantize_nvfp4.restype = None
        L.oracle_quantize_nvfp4_dt.argtypes = [vp, ctypes.c_int, i64, i64, vp, vp, vp]
        L.oracle_quantize_nvfp4_dt.restype = None
        L.oracle_quantize_mx4.argtypes = [vp, i32, i64, i64, i32, i32, vp, vp]
        L.oracle_quantize_mx4.restype = None
        L.oracle_quantize_mx4_stochastic.argtypes = [vp, i32, i64, i64, i32, ctypes.c_uint64, vp, vp, vp]
        L.oracle_quantize_mx4_stochastic.restype = None
        L.oracle_philox7_first_word.argtypes = [ctypes.c_uint64, ctypes.c_uint32]
        L.oracle_philox7_first_word.restype = ctypes.c_uint32
        L.oracle_gemm_nvfp4.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, vp]
        L.oracle_gemm_nvfp4.restype = None
        L.oracle_check_fma_division.argtypes = [vp, vp, i64]
        L.oracle_gather_scale_bf16.argtypes = [vp, i64, vp, i32, vp, i32, vp, i32, i64, i64, i64, i64, vp]
        L.oracle_gather_scale_bf16.restype = None
        L.oracle_gather_scale_quant_bf16.argtypes = [vp, i64, vp, i32, vp, i32, vp, i32, i64, i64, i64, i64, vp, vp, vp]
        L.oracle_gather_scale_quant_bf16.restype = None
        L.oracle_scatter_add.argtypes = [vp, vp, i32, i64, i64, vp, i32, i64, vp, i32, i64, i64]
        L.oracle_scatter_add.restype = None
        L.oracle_silu_mul.argtypes = [vp, vp, i32, i64, i64, i64, i64, i64, vp]
        L.oracle_silu_mul.restype = None
        L.oracle_silu_mul_quant.argtypes = [vp, vp, i32, i64, i64, i64, i64, vp, i64, vp, vp]
        L.oracle_silu_mul_quant.restype = None
        L.oracle_check_fma_division.restype = i64
        _lib = L
    return _lib


def _p(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _cpu(t: torch.Tensor) -> torch.Tensor:
    assert t.device.type == "cpu", "the oracle runs on CPU tensors"
    return t


# --------------------------------------------------------------------------
# per-row FP8 quantize
# --------------------------------------------------------------------------

def quantize_fp8_row(
    a: torch.Tensor,
    scale_ub: Optional[torch.Tensor] = None,
    zero_start_index_M: Optional[torch.Tensor] = None,
    align_rows_to: Optional[int] = None,
    eps: float = 1.0 / 512.0,
):
    """Bit-exact statement of the reference's GPU (Triton) row quantizer.

    Follows ``mslk/quantize/triton/fp8_quantize.py:210-316`` (host wrapper:
    4-D view, strides, ``align_rows_to`` padding) and ``:104-207`` (kernel).
    Returns ``(q float8_e4m3fn [..., K_out], scale fp32 [...])``.
    """
    a = _cpu(a)
    assert a.dim() <= 4 and a.dtype in DTYPE_CODE
    out_shape = list(a.shape)
    a4 = a
    while a4.dim() < 4:
        a4 = a4.unsqueeze(0)
    B, M, N, K = a4.shape
    K_out = K
    if align_rows_to is not None:
        K_out = (K + align_rows_to - 1) // align_rows_to * align_rows_to
        out_shape[-1] = K_out
    rows = B * M * N
    q = torch.empty((rows, K_out), dtype=torch.uint8)
    s = torch.empty((rows,), dtype=torch.float32)
    ub = None if scale_ub is None else _cpu(scale_ub).to(torch.float32).contiguous()
    zs = None
    if zero_start_index_M is not None:
        zs = _cpu(zero_start_index_M).reshape(B, M).to(torch.int64).contiguous()
    if rows > 0:
        lib().oracle_quantize_fp8_row(
            _p(a4), DTYPE_CODE[a.dtype], B, M, N, K, K_out,
            a4.stride(0), a4.stride(1), a4.stride(2), a4.stride(3),
            _p(ub), _p(zs), ctypes.c_float(eps), _p(q), _p(s),
        )
    return q.view(torch.float8_e4m3fn).view(out_shape), s.view(out_shape[:-1])


def quantize_fp8_row_cpu_path(a: torch.Tensor, scale_ub: Optional[torch.Tensor] = None):
    """C statement of the reference's *CPU torch* quantizer (``fp8_quantize.py:356-378``).

    Not bit-identical to the GPU arithmetic above (reciprocal-multiply, eps 1e-12);
    it exists so that fixtures produced by running the reference on CPU pin the
    shared pieces (bf16 decode, amax, e4m3 rounding) of the C oracle.
    """
    a = _cpu(a).contiguous()
    assert a.dtype == torch.bfloat16
    K = a.shape[-1]
    rows = a.numel() // K if K else 0
    q = torch.empty((rows, K), dtype=torch.uint8)
    s = torch.empty((rows,), dtype=torch.float32)
    ub = None if scale_ub is None else _cpu(scale_ub).to(torch.float32).contiguous()
    if rows:
        lib().oracle_quantize_fp8_row_cpu_path(_p(a), rows, K, _p(ub), _p(q), _p(s))
    return q.view(torch.float8_e4m3fn).view(a.shape), s.view(a.shape[:-1])


def quantize_fp8_row_cpu_path_torch(a: torch.Tensor, scale_ub: Optional[torch.Tensor] = None):
    """The same CPU formula written with the torch calls the reference uses
    (``fp8_quantize.py:360-378``); this is what the CPU baseline times."""
    row_max = torch.max(torch.abs(a), dim=-1)[0]
    if scale_ub is not None:
        row_max = torch.clamp(row_max, min=1e-12, max=scale_ub.item())
    else:
        row_max = torch.clamp(row_max, min=1e-12)
    a_scale = FP8_MAX / row_max.to(torch.float32)
    a_scale[a_scale == float("inf")] = 1.0
    a_fp8 = (a * a_scale[..., None]).to(torch.float8_e4m3fn)
    return a_fp8, (1 / a_scale).view(a.shape[:-1])


# --------------------------------------------------------------------------
# rowwise FP8 GEMM
# --------------------------------------------------------------------------

def gemm_f8_rowwise(xq, wq, x_scale, w_scale, bias: Optional[torch.Tensor] = None):
    """Slow scalar-C oracle (sequential fp32 accumulation); small shapes only."""
    xq, wq = _cpu(xq).contiguous(), _cpu(wq).contiguous()
    K = xq.shape[-1]
    M = xq.numel() // K if K else math.prod(xq.shape[:-1])
    N = wq.shape[0]
    y = torch.empty((M, N), dtype=torch.bfloat16)
    kind = 0
    if bias is not None:
        bias = bias.contiguous()
        kind = 1 if bias.dtype == torch.float32 else 2
    xs = x_scale.reshape(-1).to(torch.float32).contiguous()
    ws = w_scale.reshape(-1).to(torch.float32).contiguous()
    if M and N:
        lib().oracle_gemm_f8_rowwise(
            _p(xq.view(torch.uint8)), _p(wq.view(torch.uint8)), _p(xs), _p(ws),
            _p(bias), kind, M, N, K, _p(y))
    return y.view(*xq.shape[:-1], N)


def gemm_f8_rowwise_torch(xq, wq, x_scale, w_scale, bias: Optional[torch.Tensor] = None,
                          out_dtype=torch.bfloat16):
    """The reference tests' fp32 formula (``test/gemm/triton/grouped_gemm_test.py:124-129``,
    ``test/gemm/triton/fp8_gemm_test.py:123-127``): dequantize, fp32 matmul, scale.
    Runs on whatever device the tensors are on."""
    K = xq.shape[-1]
    x2 = xq.reshape(-1, K).to(torch.float32)
    y = (x2 @ wq.to(torch.float32).T) * x_scale.reshape(-1)[:, None].float() * w_scale.reshape(-1)[None, :].float()
    if bias is not None:
        if bias.dtype == torch.bfloat16:
            y = y.to(torch.bfloat16) + bias
        else:
            y = y + bias
    return y.to(out_dtype).view(*xq.shape[:-1], wq.shape[0])


def gemm_f8_rowwise_grouped_stacked_torch(xq, wq, x_scale, w_scale, m_sizes: Sequence[int],
                                          out_dtype=torch.bfloat16):
    """Per-group application of the formula above over the stacked layout
    (``test/gemm/triton/grouped_gemm_test.py:112-150``)."""
    N = wq.shape[1]
    y = torch.zeros((xq.shape[0], N), dtype=out_dtype, device=xq.device)
    off = 0
    for g, mg in enumerate(int(v) for v in m_sizes):
        if mg:
            y[off:off + mg] = gemm_f8_rowwise_torch(
                xq[off:off + mg], wq[g], x_scale[off:off + mg], w_scale[g], out_dtype=out_dtype)
        off += mg
    return y


def gemm_f8_rowwise_grouped_stacked(xq, wq, x_scale, w_scale, m_sizes):
    """Scalar-C stacked grouped oracle; small shapes only."""
    xq, wq = _cpu(xq).contiguous(), _cpu(wq).contiguous()
    G, N, K = wq.shape
    ms = torch.as_tensor(m_sizes, dtype=torch.int64).contiguous()
    y = torch.zeros((xq.shape[0], N), dtype=torch.bfloat16)
    xs = x_scale.reshape(-1).float().contiguous()
    ws = w_scale.reshape(-1).float().contiguous()
    lib().oracle_gemm_f8_rowwise_grouped_stacked(
        _p(xq.view(torch.uint8)), _p(wq.view(torch.uint8)), _p(xs), _p(ws), _p(ms), G, N, K, _p(y))
    return y


# --------------------------------------------------------------------------
# NVFP4
# --------------------------------------------------------------------------

def global_scale_nvfp4(x: torch.Tensor) -> torch.Tensor:
    """``(448*6)/amax(|x|)`` in fp32 (``mslk/quantize/triton/legacy/fp4_utils.py:78-92``)."""
    return (448.0 * 6.0) / torch.amax(torch.abs(x)).to(torch.float32)


def nvfp4_scale_shape(rows: int, K: int):
    nblk = K // 16
    return ((rows + 127) // 128 * 128, (nblk + 3) // 4 * 4)


def quantize_nvfp4(x: torch.Tensor, global_scale: Optional[torch.Tensor]):
    """Bit-exact statement of the reference's Triton NVFP4 quantizer
    (``mslk/quantize/triton/quantize_kernels/nvfp4.py:62-296``).
    Returns ``(packed uint8 [M, K/2], swizzled e4m3 scales [rows_pad, cols_pad])``."""
    x = _cpu(x).contiguous()
    assert x.dtype in (torch.bfloat16, torch.float16) and x.dim() == 2 and x.shape[1] % 16 == 0
    M, K = x.shape
    pr, pc = nvfp4_scale_shape(M, K)
    q = torch.empty((M, K // 2), dtype=torch.uint8)
    s = torch.zeros((pr * pc,), dtype=torch.uint8)
    gs = None if global_scale is None else _cpu(global_scale).reshape(1).float().contiguous()
    lib().oracle_quantize_nvfp4_dt(_p(x), DTYPE_CODE[x.dtype], M, K, _p(gs), _p(q), _p(s))
    return q, s.view(torch.float8_e4m3fn).view(pr, pc)


def to_blocked(x: torch.Tensor) -> torch.Tensor:
    """[rows, cols] -> flattened 128x4-tile swizzle (``legacy/primitives.py:51-86``)."""
    rows, cols = x.shape
    rb, cb = (rows + 127) // 128, (cols + 3) // 4
    padded = torch.zeros((rb * 128, cb * 4), dtype=x.dtype)
    padded[:rows, :cols] = x
    return padded.view(rb, 4, 32, cb, 4).permute(0, 3, 2, 1, 4).reshape(-1)


def from_blocked(x: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    """Inverse of :func:`to_blocked` (``legacy/primitives.py:89-119``)."""
    rb, cb = (rows + 127) // 128, (cols + 3) // 4
    p = x.reshape(rb, cb, 32, 4, 4).permute(0, 3, 2, 1, 4).reshape(rb * 128, cb * 4)
    return p[:rows, :cols].contiguous()


_E2M1 = [0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6]


def fp4_to_float(packed: torch.Tensor) -> torch.Tensor:
    """Packed e2m1 bytes -> fp32, element 2j in the low nibble
    (``legacy/fp4_utils.py:19-45``)."""
    lut = torch.tensor(_E2M1, dtype=torch.float32, device=packed.device)
    p = packed.view(torch.uint8).to(torch.int64)
    lo, hi = p & 0xF, (p >> 4) & 0xF
    return lut[torch.stack([lo, hi], dim=-1).reshape(*p.shape[:-1], p.shape[-1] * 2)]


def gemm_nvfp4_torch(xq, wq, x_scale, w_scale, global_scale, out_dtype=torch.bfloat16):
    """fp32 dequantize-matmul oracle for ``f4f4bf16`` (NVFP4):
    ``(fp4(xq)*sx) @ (fp4(wq)*sw).T * global_scale`` with ``sx/sw`` un-swizzled
    (``legacy/fp4_utils.py:95-120``; epilogue ``f4f4bf16_common.cuh:274-281``)."""
    M, K = xq.shape[0], xq.shape[1] * 2
    N = wq.shape[0]
    dev = xq.device
    sx = from_blocked(x_scale.view(torch.uint8).cpu().reshape(-1), M, K // 16).view(torch.float8_e4m3fn).float().to(dev)
    sw = from_blocked(w_scale.view(torch.uint8).cpu().reshape(-1), N, K // 16).view(torch.float8_e4m3fn).float().to(dev)
    xf = fp4_to_float(xq) * sx.repeat_interleave(16, dim=1)
    wf = fp4_to_float(wq) * sw.repeat_interleave(16, dim=1)
    y = (xf @ wf.T) * global_scale.reshape(()).float().to(dev)
    return y.to(out_dtype)


def gemm_nvfp4(xq, wq, x_scale, w_scale, global_scale):
    """Scalar-C NVFP4 GEMM oracle; small shapes only."""
    xq, wq = _cpu(xq).contiguous().view(torch.uint8), _cpu(wq).contiguous().view(torch.uint8)
    M, K = xq.shape[0], xq.shape[1] * 2
    N = wq.shape[0]
    y = torch.empty((M, N), dtype=torch.bfloat16)
    gs = global_scale.reshape(1).float().contiguous()
    sx = x_scale.contiguous().view(torch.uint8)
    sw = w_scale.contiguous().view(torch.uint8)
    lib().oracle_gemm_nvfp4(_p(xq), _p(wq), _p(sx), _p(sw), _p(gs), M, N, K, _p(y))
    return y


# --------------------------------------------------------------------------
# MXFP4 (e8m0 scales per 32 or 16 elements)
# --------------------------------------------------------------------------

MX_ROUND_ADD = {0: -1, 1: 0, 2: (1 << 21) - 1, 4: (1 << 23) - 1}     # nearest / floor / even / ceil of the shared exponent


def quantize_mx4(x: torch.Tensor, group_size: int = 32, rounding_mode: int = 4, seed: Optional[int] = None,
                 stream_rows: Optional[torch.Tensor] = None):
    """MXFP4 quantize (``mslk/quantize/triton/quantize_kernels/mx4.py:28-355``): returns
    ``(xq uint8 [M, K/2], scales uint8, flattened swizzled [ceil(M/128)*128 * ceil(K/group/4)*4])``.  Rounding mode 3
    (stochastic) needs ``seed``; ``stream_rows`` (int32 per row) replaces the row index its random streams use."""
    x2 = _cpu(x).reshape(-1, x.shape[-1]).contiguous()
    M, K = x2.shape
    assert K % group_size == 0 and x2.dtype in (torch.bfloat16, torch.float16)
    pr, pc = (M + 127) // 128 * 128, (K // group_size + 3) // 4 * 4
    q = torch.empty((M, K // 2), dtype=torch.uint8)
    s = torch.empty((pr * pc,), dtype=torch.uint8)
    if int(rounding_mode) == 3:
        assert seed is not None, "stochastic rounding needs a seed"
        rows = None if stream_rows is None else stream_rows.to(torch.int32).contiguous()
        lib().oracle_quantize_mx4_stochastic(_p(x2.view(torch.int16)), 1 if x2.dtype == torch.bfloat16 else 2, M, K,
                                             group_size, int(seed) & 0x7FFFFFFFFFFFFFFF,
                                             None if rows is None else _p(rows), _p(q), _p(s))
        return q, s
    lib().oracle_quantize_mx4(_p(x2.view(torch.int16)), 1 if x2.dtype == torch.bfloat16 else 2, M, K, group_size,
                              MX_ROUND_ADD[int(rounding_mode)], _p(q), _p(s))
    return q, s


def gemm_mx4_torch(xq, wq, x_scale, w_scale, group_size: int = 32, out_dtype=torch.bfloat16):
    """fp32 dequantize-matmul formula of the MXFP4 GEMM: ``(fp4(xq) * 2^(sx-127)) @ (fp4(wq) * 2^(sw-127)).T`` with the
    e8m0 scales un-swizzled (the check the reference's tests make against the unquantized product, in exact form)."""
    M, K = xq.shape[0], xq.shape[1] * 2
    N = wq.shape[0]
    dev = xq.device
    sx = from_blocked(x_scale.view(torch.uint8).cpu().reshape(-1), M, K // group_size).to(torch.int32)
    sw = from_blocked(w_scale.view(torch.uint8).cpu().reshape(-1), N, K // group_size).to(torch.int32)
    fx = torch.ldexp(torch.ones(sx.shape, dtype=torch.float32), sx - 127).to(dev)
    fw = torch.ldexp(torch.ones(sw.shape, dtype=torch.float32), sw - 127).to(dev)
    xf = fp4_to_float(xq) * fx.repeat_interleave(group_size, dim=1)
    wf = fp4_to_float(wq) * fw.repeat_interleave(group_size, dim=1)
    return (xf @ wf.T).to(out_dtype)


# --------------------------------------------------------------------------
# fused SwiGLU (+ per-row FP8 quantize)
# --------------------------------------------------------------------------

def silu_mul(x0: torch.Tensor, x1: torch.Tensor, valid_token_count: Optional[int] = None) -> torch.Tensor:
    """fp32 ``x0 * sigmoid(x0) * x1`` (``mslk/moe/activation.py:181-217``); rows past the count stay 0."""
    x0, x1 = _cpu(x0), _cpu(x1)
    assert x0.dim() == 2 and x0.shape == x1.shape and x0.dtype == x1.dtype and x0.stride(1) == 1 and x1.stride(1) == 1
    T, D = x0.shape
    y = torch.zeros((T, D), dtype=torch.float32)
    valid = T if valid_token_count is None else int(valid_token_count)
    if T and D:
        lib().oracle_silu_mul(_p(x0), _p(x1), DTYPE_CODE[x0.dtype], T, D, x0.stride(0), x1.stride(0), valid, _p(y))
    return y


def silu_mul_quant(x0: torch.Tensor, x1: torch.Tensor, scale_ub: Optional[torch.Tensor] = None,
                   valid_token_count: Optional[int] = None):
    """Statement of ``mslk/moe/activation.py:220-294`` with exact ``expf`` / IEEE division in the sigmoid.

    Returns ``(q float8_e4m3fn [T, D], inverse scale fp32 [T])``; rows past the count are 0.  The GPU
    kernels use approximate exp2 / division, so agreement with them is to within one e4m3 code on a
    small fraction of elements (rounding boundaries) and a few ulps on the scale, not bit for bit.
    """
    x0, x1 = _cpu(x0), _cpu(x1)
    assert x0.dim() == 2 and x0.shape == x1.shape and x0.dtype == x1.dtype and x0.stride(1) == 1 and x1.stride(1) == 1
    T, D = x0.shape
    q = torch.zeros((T, D), dtype=torch.uint8)
    s = torch.zeros((T,), dtype=torch.float32)
    ub = None if scale_ub is None else _cpu(scale_ub).to(torch.float32).contiguous()
    valid = T if valid_token_count is None else int(valid_token_count)
    if T and D:
        lib().oracle_silu_mul_quant(_p(x0), _p(x1), DTYPE_CODE[x0.dtype], T, D, x0.stride(0), x1.stride(0),
                                    _p(ub), valid, _p(q), _p(s))
    return q.view(torch.float8_e4m3fn), s


# --------------------------------------------------------------------------
# MoE token gather / scatter
# --------------------------------------------------------------------------

def _bits(t: torch.Tensor) -> int:
    assert t.dtype in (torch.int32, torch.int64)
    return 32 if t.dtype == torch.int32 else 64


def gather_scale_dense_tokens(x, token_indices, expert_indices, scores, valid_token_count: Optional[int] = None):
    """Exact statement of ``mslk/moe/gather_scatter.py:431-486`` for bf16 ``x``; rows past the count stay 0."""
    x, token_indices, expert_indices, scores = _cpu(x), _cpu(token_indices), _cpu(expert_indices), _cpu(scores)
    assert x.dtype == torch.bfloat16 and x.is_contiguous() and scores.dtype in DTYPE_CODE
    a, D = token_indices.shape[0], x.shape[1]
    out = torch.zeros((a, D), dtype=torch.bfloat16)
    valid = a if valid_token_count is None else int(valid_token_count)
    if a and D:
        lib().oracle_gather_scale_bf16(_p(x), D, _p(token_indices), _bits(token_indices), _p(expert_indices),
                                       _bits(expert_indices), _p(scores), DTYPE_CODE[scores.dtype], scores.stride(0),
                                       scores.stride(1), a, valid, _p(out))
    return out


def gather_scale_quant_dense_tokens(x, token_indices, expert_indices, scores, scale_ub=None,
                                    valid_token_count: Optional[int] = None):
    """``mslk/moe/gather_scatter.py:537-655`` with IEEE divisions; returns ``(fp8 [a, D], inverse scale [a])``."""
    x, token_indices, expert_indices, scores = _cpu(x), _cpu(token_indices), _cpu(expert_indices), _cpu(scores)
    assert x.dtype == torch.bfloat16 and x.is_contiguous() and scores.dtype in DTYPE_CODE
    a, D = token_indices.shape[0], x.shape[1]
    q = torch.zeros((a, D), dtype=torch.uint8)
    s = torch.zeros((a,), dtype=torch.float32)
    ub = None if scale_ub is None else _cpu(scale_ub).to(torch.float32).contiguous()
    valid = a if valid_token_count is None else int(valid_token_count)
    if a and D:
        lib().oracle_gather_scale_quant_bf16(_p(x), D, _p(token_indices), _bits(token_indices), _p(expert_indices),
                                             _bits(expert_indices), _p(scores), DTYPE_CODE[scores.dtype],
                                             scores.stride(0), scores.stride(1), a, valid, _p(ub), _p(q), _p(s))
    return q.view(torch.float8_e4m3fn), s


_SCATTER_CODE = {torch.float32: 0, torch.bfloat16: 1, torch.int32: 3}


def scatter_add_dense_tokens(out_tokens, in_tokens, token_indices, valid_token_count: Optional[int] = None):
    """In place ``out_tokens[token_indices[i]] += in_tokens[i]`` in row order (``gather_scatter.py:489-526``)."""
    out_tokens, in_tokens, token_indices = _cpu(out_tokens), _cpu(in_tokens), _cpu(token_indices)
    assert out_tokens.is_contiguous() and in_tokens.is_contiguous() and in_tokens.dtype == out_tokens.dtype
    a, D = in_tokens.shape
    valid = a if valid_token_count is None else int(valid_token_count)
    if a and D:
        lib().oracle_scatter_add(_p(out_tokens), _p(in_tokens), _SCATTER_CODE[in_tokens.dtype], a, D, _p(token_indices),
                                 _bits(token_indices), valid, None, 32, 1, 1)


def scatter_add_padded_tokens(in_tokens, token_counts, token_indices, out_tokens):
    """In place statement of ``gather_scatter.py:677-740`` for ``in_tokens [EP, T_K, D]``."""
    in_tokens, token_counts, token_indices, out_tokens = (_cpu(in_tokens), _cpu(token_counts), _cpu(token_indices),
                                                          _cpu(out_tokens))
    assert out_tokens.is_contiguous() and in_tokens.is_contiguous() and in_tokens.dtype == out_tokens.dtype
    EP, T_K, D = in_tokens.shape
    E = token_counts.shape[0]
    if T_K and D:
        lib().oracle_scatter_add(_p(out_tokens), _p(in_tokens), _SCATTER_CODE[in_tokens.dtype], T_K, D,
                                 _p(token_indices), _bits(token_indices), T_K, _p(token_counts), _bits(token_counts),
                                 E, EP)


# --------------------------------------------------------------------------
# NVFP4 for stacked groups (MoE)
# --------------------------------------------------------------------------

def calculate_group_max(x: torch.Tensor, m_sizes: Sequence[int]):
    """``mslk/quantize/triton/legacy/global_scale.py:40-230``: per group ``2688 / max|x|`` (IEEE division here;
    the GPU kernels use an approximate one, so agreement is to a couple of ulps), ``1e-8`` replacing a zero
    maximum, ``FLT_MAX`` for groups without rows; plus the group index of every row."""
    x = _cpu(x)
    out = torch.full((len(m_sizes),), torch.finfo(torch.float32).max, dtype=torch.float32)
    idx = torch.zeros((x.shape[0],), dtype=torch.int64)
    r = 0
    for g, m in enumerate(m_sizes):
        if m > 0:
            amax = x[r:r + m].abs().max().float()
            out[g] = torch.tensor(2688.0) / torch.where(amax == 0, torch.tensor(1e-8), amax)
            idx[r:r + m] = g
        r += m
    return out, idx


def nvfp4_quantize_stacked(m_sizes: Sequence[int], x: torch.Tensor, global_scale: torch.Tensor):
    """``mslk/quantize/triton/legacy/quantize_stacked.py:22-178``: every group quantized with its own global scale
    (bit-exact block arithmetic of :func:`quantize_nvfp4`), its scale rows padded to a multiple of 128.  Returns
    ``(packed uint8 [M, K/2], scale bytes [sum of padded rows, cols_pad] swizzled per group, padded row starts)``."""
    x = _cpu(x)
    M, K = x.shape
    q = torch.zeros((M, K // 2), dtype=torch.uint8)
    scales, starts = [], [0]
    r = 0
    for g, m in enumerate(m_sizes):
        if m > 0:
            qg, sg = quantize_nvfp4(x[r:r + m].contiguous(), global_scale[g:g + 1])
            q[r:r + m] = qg
            scales.append(sg.view(torch.uint8).reshape(-1, sg.shape[-1]))
        starts.append(starts[-1] + (m + 127) // 128 * 128)
        r += m
    pc = (K // 16 + 3) // 4 * 4
    s = torch.cat(scales, dim=0) if scales else torch.zeros((0, pc), dtype=torch.uint8)
    return q, s.view(torch.float8_e4m3fn), starts


def gemm_nvfp4_grouped_stacked(xq, wq, x_scale, w_scale, m_sizes: Sequence[int], global_scale, starts=None):
    """Per group :func:`gemm_nvfp4_torch` on its rows, weights, scale blocks and global scale
    (``csrc/gemm/cutlass/f4f4bf16_grouped/f4f4bf16_grouped_common.cuh:57-148`` pointer arithmetic)."""
    xq, wq = _cpu(xq), _cpu(wq)
    G, N = wq.shape[0], wq.shape[1]
    K = wq.shape[2] * 2
    pc = (K // 16 + 3) // 4 * 4
    xs = _cpu(x_scale).view(torch.uint8).reshape(-1, pc)
    ws = _cpu(w_scale).view(torch.uint8).reshape(G, -1, pc)
    y = torch.zeros((xq.shape[0], N), dtype=torch.bfloat16)
    r, pr = 0, 0
    for g, m in enumerate(m_sizes):
        if starts is not None:
            pr = int(starts[g])
        mp = (m + 127) // 128 * 128
        if m > 0:
            y[r:r + m] = gemm_nvfp4_torch(xq[r:r + m], wq[g], xs[pr:pr + mp].view(torch.float8_e4m3fn),
                                          ws[g].view(torch.float8_e4m3fn), global_scale[g:g + 1])
        r += m
        pr += mp
    return y
