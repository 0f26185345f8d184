"""ctypes binding of the C-ABI library ``libmslk_b200.so`` (declared in ``include/mslk_b200.h``).

There is no fallback: if the library is missing or cannot be loaded, importing
this module raises, and every wrapper raises ``RuntimeError`` with the library's
own message when a call is rejected.
"""

from __future__ import annotations

import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libmslk_b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python -m mslk_b200.build` (needs nvcc with sm_100a support). "
        "mslk_b200 has no CPU or eager fallback.")

lib = ctypes.CDLL(LIB_PATH)

_i64, _vp, _f32, _int = ctypes.c_int64, ctypes.c_void_p, ctypes.c_float, ctypes.c_int

lib.mslk_b200_abi_version.restype = _int
lib.mslk_b200_last_error.restype = ctypes.c_char_p
lib.mslk_b200_device_status.argtypes = [ctypes.POINTER(_int)]
lib.mslk_b200_device_status.restype = _int
lib.mslk_b200_selftest_wait_timeout.argtypes = [ctypes.c_uint64, _vp, _vp]
lib.mslk_b200_selftest_wait_timeout.restype = _int
lib.mslk_b200_quantize_fp8_row.argtypes = [_vp, _int] + [_i64] * 9 + [_vp, _vp, _f32, _vp, _vp, _vp]
lib.mslk_b200_quantize_fp8_row.restype = _int
lib.mslk_b200_f8f8bf16_rowwise.argtypes = [_vp, _vp, _vp, _vp, _vp, _int, _vp, _i64, _i64, _i64, _vp]
lib.mslk_b200_f8f8bf16_rowwise.restype = _int
lib.mslk_b200_f8f8bf16_rowwise_workspace_bytes.argtypes = [_i64, _i64, _i64]
lib.mslk_b200_f8f8bf16_rowwise_workspace_bytes.restype = ctypes.c_size_t
lib.mslk_b200_f8f8bf16_rowwise_ws.argtypes = [_vp, _vp, _vp, _vp, _vp, _int, _vp, _i64, _i64, _i64, _vp, ctypes.c_size_t, _vp]
lib.mslk_b200_f8f8bf16_rowwise_ws.restype = _int
lib.mslk_b200_f8f8bf16_rowwise_allgather.argtypes = [_vp, _vp, _vp, _vp, _vp, _int, ctypes.POINTER(_vp), _int, _int,
                                                     _i64, _i64, _i64, _vp]
lib.mslk_b200_f8f8bf16_rowwise_allgather.restype = _int
lib.mslk_b200_f8f8bf16_rowwise_scatter.argtypes = [_vp, _vp, _vp, _vp, ctypes.POINTER(_vp), _int, _int, _i64, _i64, _i64, _vp]
lib.mslk_b200_f8f8bf16_rowwise_scatter.restype = _int
lib.mslk_b200_reduce_slots_bf16.argtypes = [_vp, _int, _i64, _i64, _vp, _vp]
lib.mslk_b200_reduce_slots_bf16.restype = _int
lib.mslk_b200_f8f8bf16_rowwise_noalloc.argtypes = [_vp, _vp, _vp, _vp, _vp, _int, _vp, _i64, _i64, _i64, _vp]
lib.mslk_b200_f8f8bf16_rowwise_noalloc.restype = _int
lib.mslk_b200_f8f8bf16_rowwise_grouped_stacked.argtypes = [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _vp]
lib.mslk_b200_f8f8bf16_rowwise_grouped_stacked.restype = _int
lib.mslk_b200_quantize_nvfp4.argtypes = [_vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp]
lib.mslk_b200_quantize_nvfp4.restype = _int
lib.mslk_b200_quantize_nvfp4_dt.argtypes = [_vp, _int, _i64, _i64, _i64, _vp, _vp, _vp, _vp]
lib.mslk_b200_quantize_nvfp4_dt.restype = _int
lib.mslk_b200_f4f4bf16.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]
lib.mslk_b200_f4f4bf16.restype = _int
lib.mslk_b200_quantize_mx4.argtypes = [_vp, _int, _i64, _i64, _i64, _int, _int, _vp, _vp, _vp]
lib.mslk_b200_quantize_mx4.restype = _int
lib.mslk_b200_quantize_mx4_stacked.argtypes = [_vp, _int, _i64, _i64, _i64, _vp, _i64, _int, _int, _vp, _vp, _vp]
lib.mslk_b200_quantize_mx4_stacked.restype = _int
lib.mslk_b200_quantize_mx4_seeded.argtypes = [_vp, _int, _i64, _i64, _i64, _int, _int, ctypes.c_uint64, _vp, _vp, _vp]
lib.mslk_b200_quantize_mx4_seeded.restype = _int
lib.mslk_b200_quantize_mx4_stacked_seeded.argtypes = [_vp, _int, _i64, _i64, _i64, _vp, _i64, _int, _int, ctypes.c_uint64,
                                                      _vp, _vp, _vp]
lib.mslk_b200_quantize_mx4_stacked_seeded.restype = _int
lib.mslk_b200_f4f4bf16_mx.argtypes = [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp]
lib.mslk_b200_f4f4bf16_mx.restype = _int
lib.mslk_b200_f4f4bf16_grouped_stacked_mx.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _int, _vp, _vp]
lib.mslk_b200_f4f4bf16_grouped_stacked_mx.restype = _int
lib.mslk_b200_f4f4bf16_grouped_mm_mx.argtypes = [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _int, _vp, _vp]
lib.mslk_b200_f4f4bf16_grouped_mm_mx.restype = _int
lib.mslk_b200_f4f4bf16_grouped_mm_2d2d.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _int,
                                                   ctypes.c_size_t, ctypes.c_size_t, _vp, _vp]
lib.mslk_b200_f4f4bf16_grouped_mm_2d2d.restype = _int
lib.mslk_b200_debug_nvfp4_pair_timers.argtypes = [_vp]
lib.mslk_b200_debug_nvfp4_pair_timers.restype = _int
lib.mslk_b200_f4f4bf16_workspace_bytes.argtypes = [_i64, _i64, _i64]
lib.mslk_b200_f4f4bf16_workspace_bytes.restype = ctypes.c_size_t
lib.mslk_b200_f4f4bf16_ws.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, ctypes.c_size_t, _vp]
lib.mslk_b200_f4f4bf16_ws.restype = _int
lib.mslk_b200_f8f8bf16_rowwise_batched.argtypes = [_vp, _vp, _vp, _vp, _vp, _int, _vp, _i64, _i64, _i64, _i64, _vp]
lib.mslk_b200_f8f8bf16_rowwise_batched.restype = _int
lib.mslk_b200_f8f8bf16_rowwise_grouped_stacked_scatter_add.argtypes = [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp,
                                                                       _int, _vp, _i64, _vp]
lib.mslk_b200_f8f8bf16_rowwise_grouped_stacked_scatter_add.restype = _int
lib.mslk_b200_f4f4bf16_grouped_stacked.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _vp]
lib.mslk_b200_f4f4bf16_grouped_stacked.restype = _int
lib.mslk_b200_f4f4bf16_grouped_mm.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _vp]
lib.mslk_b200_f4f4bf16_grouped_mm.restype = _int
lib.mslk_b200_quantize_nvfp4_stacked.argtypes = [_vp, _i64, _i64, _i64, _vp, _i64, _vp, _vp, _vp, _vp]
lib.mslk_b200_quantize_nvfp4_stacked.restype = _int
lib.mslk_b200_calculate_group_max.argtypes = [_vp, _i64, _i64, _i64, _vp, _i64, _vp, _vp, _vp]
lib.mslk_b200_calculate_group_max.restype = _int
lib.mslk_b200_quantize_nvfp4_stacked_dt.argtypes = [_vp, _int, _i64, _i64, _i64, _vp, _i64, _vp, _vp, _vp, _vp]
lib.mslk_b200_quantize_nvfp4_stacked_dt.restype = _int
lib.mslk_b200_calculate_group_max_dt.argtypes = [_vp, _int, _i64, _i64, _i64, _vp, _i64, _vp, _vp, _vp]
lib.mslk_b200_calculate_group_max_dt.restype = _int
lib.mslk_b200_gather_scale_dense_tokens.argtypes = [_vp, _int, _i64, _i64, _vp, _int, _vp, _int, _vp, _int, _i64, _i64, _i64,
                                                    _i64, _vp, _vp, _vp]
lib.mslk_b200_gather_scale_dense_tokens.restype = _int
lib.mslk_b200_gather_scale_quant_dense_tokens.argtypes = [_vp, _int, _i64, _i64, _vp, _int, _vp, _int, _vp, _int, _i64, _i64,
                                                          _i64, _i64, _vp, _vp, _vp, _vp, _vp]
lib.mslk_b200_gather_scale_quant_dense_tokens.restype = _int
lib.mslk_b200_scatter_add_dense_tokens.argtypes = [_vp, _i64, _vp, _int, _i64, _i64, _vp, _int, _vp, _vp]
lib.mslk_b200_scatter_add_dense_tokens.restype = _int
lib.mslk_b200_scatter_add_padded_tokens.argtypes = [_vp, _int, _i64, _i64, _i64, _vp, _int, _i64, _vp, _int, _vp, _i64, _vp]
lib.mslk_b200_scatter_add_padded_tokens.restype = _int
lib.mslk_b200_silu_mul_quant.argtypes = [_vp, _vp, _int, _i64, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp]
lib.mslk_b200_silu_mul_quant.restype = _int
lib.mslk_b200_silu_mul.argtypes = [_vp, _vp, _int, _i64, _i64, _i64, _i64, _vp, _vp, _vp]
lib.mslk_b200_silu_mul.restype = _int


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib.mslk_b200_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"{what} failed (code {rc}): {msg}")


def device_status() -> int:
    """Synchronises the current device and returns (and clears) its kernel status word."""
    out = _int(0)
    check(lib.mslk_b200_device_status(ctypes.byref(out)), "mslk_b200_device_status")
    return out.value
