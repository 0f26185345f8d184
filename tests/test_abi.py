"""CPU tests: the C-ABI library loads and exports every symbol the header declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "mslk_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mslk_b200_\w+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    syms = _declared_symbols()
    for s in ["mslk_b200_quantize_fp8_row", "mslk_b200_f8f8bf16_rowwise",
              "mslk_b200_f8f8bf16_rowwise_grouped_stacked", "mslk_b200_quantize_nvfp4",
              "mslk_b200_f4f4bf16", "mslk_b200_last_error", "mslk_b200_device_status"]:
        assert s in syms


def test_library_loads_and_exports_all_declared_symbols():
    from mslk_b200 import build
    path = build.build(torch_ops=False)
    lib = ctypes.CDLL(path)
    for s in _declared_symbols():
        assert hasattr(lib, s), s
    lib.mslk_b200_abi_version.restype = ctypes.c_int
    assert lib.mslk_b200_abi_version() == 1


def test_argument_errors_need_no_gpu():
    from mslk_b200._lib import lib, check
    import pytest
    # K_out < K is rejected before any CUDA call
    rc = lib.mslk_b200_quantize_fp8_row(None, 1, 1, 1, 2, 8, 4, 0, 0, 8, 1, None, None, 0.0, None, None, None)
    assert rc != 0
    with pytest.raises(RuntimeError, match="bad shape"):
        check(rc, "quantize_fp8_row")
    rc = lib.mslk_b200_quantize_nvfp4(None, 4, 24, 24, None, None, None, None)
    assert rc != 0 and b"multiple of 16" in lib.mslk_b200_last_error()
    rc = lib.mslk_b200_f8f8bf16_rowwise(None, None, None, None, None, 7, None, 4, 4, 16, None)
    assert rc != 0 and b"bias_kind" in lib.mslk_b200_last_error()
