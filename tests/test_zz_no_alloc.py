"""GPU test of the allocation-free few-token GEMM entry point (collected last on purpose).

Who needs it: a host that cannot get device memory at call time -- an inference server that gave
all free HBM to its KV-cache pool, a runtime with a frozen memory plan, a thread that must not
call cudaMalloc because that stalls the whole device.  ``mslk_b200_f8f8bf16_rowwise_noalloc``
keeps the split-K scratch in an 8 MiB array inside the library instead.

The test calls it through the C ABI twice in a row (the second call meets the scratch as the
first left it) and compares with the regular entry point, and checks that torch's allocator was
not touched while it ran.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1.6e-2, 1e-2   # the tolerance of the other GEMM tests


def _inputs(M, N, K, seed):
    from mslk_b200 import ops
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((M, K), generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn((N, K), generator=g) * 0.02).to(torch.bfloat16).cuda()
    xq, xs = ops.quantize_fp8_row(x)
    wq, ws = ops.quantize_fp8_row(w)
    return xq, wq, xs, ws


# (16, 28672, 8192) and (32, 8192, 28672): few-token shapes whose split-K scratch WOULD exceed the built-in
# array; up to 32 tokens the kernel splits K inside thread-block clusters and needs no scratch, so they are served
@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (16, 6144, 4096), (32, 4096, 14336), (7, 1000, 512), (64, 1024, 4096),
                                   (16, 28672, 8192), (32, 8192, 28672)])
def test_noalloc_matches_regular_entry_point_twice(M, N, K):
    from mslk_b200._lib import check, device_status, lib
    xq, wq, xs, ws = _inputs(M, N, K, seed=M + N)
    bias = torch.randn(N, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    y_ref = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    check(lib.mslk_b200_f8f8bf16_rowwise(xq.data_ptr(), wq.data_ptr(), xs.data_ptr(), ws.data_ptr(), bias.data_ptr(), 1,
                                         y_ref.data_ptr(), M, N, K, st), "regular entry point")
    outs = [torch.zeros((M, N), dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    torch.cuda.synchronize()
    reserved_before = torch.cuda.memory_reserved()
    for y in outs:   # two calls in a row on the shared built-in scratch
        check(lib.mslk_b200_f8f8bf16_rowwise_noalloc(xq.data_ptr(), wq.data_ptr(), xs.data_ptr(), ws.data_ptr(),
                                                     bias.data_ptr(), 1, y.data_ptr(), M, N, K, st), "noalloc entry point")
    torch.cuda.synchronize()
    assert torch.cuda.memory_reserved() == reserved_before, "torch's allocator was used"
    scale = max(1.0, float(y_ref.float().std()))
    for y in outs:
        torch.testing.assert_close(y.float(), y_ref.float(), rtol=RTOL, atol=ATOL * scale)
    assert torch.equal(outs[0], outs[1]), "second call on the used scratch differs from the first"
    assert device_status() == 0


def test_noalloc_rejects_what_it_cannot_serve():
    from mslk_b200._lib import lib
    M, N, K = 128, 4096, 4096      # real buffers of the full size: nothing could be read out of bounds
    xq, wq, xs, ws = _inputs(M, N, K, seed=1)
    y = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    args = (xq.data_ptr(), wq.data_ptr(), xs.data_ptr(), ws.data_ptr(), None, 0, y.data_ptr())
    # the split-K scratch of this shape (16 MiB) is larger than the built-in buffer
    assert lib.mslk_b200_f8f8bf16_rowwise_noalloc(*args, M, N, K, st) != 0
    assert b"built-in buffer holds" in lib.mslk_b200_last_error()
    # more tokens than the kernel behind this entry point takes (rejected on the sizes alone)
    assert lib.mslk_b200_f8f8bf16_rowwise_noalloc(*args, 200, N, K, st) != 0
    assert b"1..128 tokens" in lib.mslk_b200_last_error()
