"""GPU test of the failure path every pipeline kernel relies on: a wait on an mbarrier that nothing signals
must run out by itself, leave a code in the device status word and let the kernel return normally.
The wait is made to expire by using a flag that nothing sets and a 1 ms limit; nothing faults, traps or hangs."""
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_bounded_wait_expires_records_status_and_context_stays_usable():
    from mslk_b200 import ops
    from mslk_b200._lib import check, device_status, lib
    assert device_status() == 0
    returned = torch.zeros(1, dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    t0 = time.perf_counter()
    check(lib.mslk_b200_selftest_wait_timeout(1_000_000, returned.data_ptr(), st), "selftest_wait_timeout")
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    assert elapsed < 1.0, f"a 1 ms wait limit took {elapsed:.3f} s to expire"
    assert int(returned.item()) == 1, "the kernel did not see its wait give up"
    assert device_status() == 3, "the expired wait did not leave the epilogue-timeout code"
    assert device_status() == 0, "reading the status word clears it"
    # the same context still runs real kernels
    x = torch.randn((64, 256), device="cuda").bfloat16()
    q, s = ops.quantize_fp8_row(x)
    y = ops.f8f8bf16_rowwise(q, q, s, s)
    torch.cuda.synchronize()
    assert torch.isfinite(y.float()).all() and device_status() == 0


def test_status_word_is_visible_through_the_operator_layer():
    from mslk_b200 import compat
    from mslk_b200._lib import check, lib
    compat.install()
    import mslk.gemm  # noqa: F401
    check(lib.mslk_b200_selftest_wait_timeout(200_000, None, torch.cuda.current_stream().cuda_stream), "selftest")
    assert torch.ops.mslk.device_status() == 3
    assert torch.ops.mslk.device_status() == 0


def test_selftest_rejects_long_limits():
    from mslk_b200._lib import lib
    assert lib.mslk_b200_selftest_wait_timeout(10_000_000_000, None, None) != 0
    assert b"limit" in lib.mslk_b200_last_error()
