"""GPU tests through the operator layer (torch.ops.mslk.* and the reference's Python symbols),
mirroring the reference's own cases: test/gemm/gemm_test.py:361-505 (dense), :725-856 (stacked),
:2374-2396 (NVFP4), test/quantize/triton/fp8_quantize_test.py:37-220."""
import pytest
import torch

import oracle
from helpers import randn_bf16, u8

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mslk():
    from mslk_b200 import compat
    compat.install()
    import mslk.gemm  # noqa: F401
    torch.backends.cuda.matmul.allow_tf32 = False
    return torch.ops.mslk


@pytest.mark.parametrize("M,N,K", [(256, 128, 256), (2048, 2048, 4096), (4096, 4096, 8192), (0, 256, 4096)])
@pytest.mark.parametrize("use_bias", [False, True])
def test_reference_dense_cases(mslk, M, N, K, use_bias):
    from mslk.quantize.triton.fp8_quantize import quantize_fp8_row
    x = (torch.randn(M, K, device="cuda") * 0.1).bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.01).bfloat16()
    bias = torch.randn(N, device="cuda") if use_bias else None
    xq, xs = quantize_fp8_row(x)
    wq, ws = quantize_fp8_row(w)
    zq = mslk.f8f8bf16_rowwise(xq, wq, xs, ws, bias=bias)
    zq_ref = (x @ w.T).to(torch.bfloat16)
    if use_bias:
        zq_ref = zq_ref + bias
    torch.testing.assert_close(zq, zq_ref.to(torch.bfloat16), atol=9e-2, rtol=9e-2)
    if M:
        torch.testing.assert_close(zq.float(), oracle.gemm_f8_rowwise_torch(xq, wq, xs, ws, bias).float(), rtol=1.6e-2, atol=1e-2)


def test_cuda_graph_capture_dense_and_grouped(mslk):
    from mslk.quantize.triton.fp8_quantize import quantize_fp8_row
    M, N, K, G = 512, 512, 1024, 4
    x = (torch.randn(M, K, device="cuda") * 0.1).bfloat16()
    w = (torch.randn(G, N, K, device="cuda") * 0.01).bfloat16()
    wq, ws = quantize_fp8_row(w)
    ms = torch.tensor([128, 0, 256, 128], dtype=torch.int64, device="cuda")
    xq, xs = quantize_fp8_row(x)
    mslk.f8f8bf16_rowwise(xq, wq[0], xs, ws[0])
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        xq_g, xs_g = quantize_fp8_row(x)
        y1 = mslk.f8f8bf16_rowwise(xq_g, wq[0], xs_g, ws[0])
        y2 = mslk.f8f8bf16_rowwise_grouped_stacked(xq_g, wq, xs_g, ws.view(-1), ms)
    g.replay()
    torch.cuda.synchronize()
    torch.testing.assert_close(y1.float(), oracle.gemm_f8_rowwise_torch(xq, wq[0], xs, ws[0]).float(), rtol=1.6e-2, atol=1e-2)
    torch.testing.assert_close(y2.float(), oracle.gemm_f8_rowwise_grouped_stacked_torch(xq, wq, xs, ws, ms.tolist()).float(),
                               rtol=1.6e-2, atol=1e-2)


@pytest.mark.parametrize("G", [1, 16, 64])
def test_reference_stacked_cases(mslk, G):
    from mslk.quantize.triton.fp8_quantize import quantize_fp8_row
    M, N, K = 2048, 1024, 512
    ms = torch.randint(1, M // 64 // G + 2, (G,)) * 64
    total = int(ms.sum())
    x = (torch.randn(total, K, device="cuda") * 0.1).bfloat16()
    w = (torch.randn(G, N, K, device="cuda") * 0.01).bfloat16()
    xq, xs = quantize_fp8_row(x)
    wq, ws = quantize_fp8_row(w)
    y = mslk.f8f8bf16_rowwise_grouped_stacked(xq, wq, xs, ws.view(-1), ms.cuda())
    off = 0
    for g in range(G):
        mg = int(ms[g])
        ref = (x[off:off + mg] @ w[g].T).to(torch.bfloat16)
        torch.testing.assert_close(y[off:off + mg], ref, atol=8e-2, rtol=8e-2)
        off += mg


@pytest.mark.parametrize("M,N,K", [(1, 256, 2048), (250, 512, 2048), (250, 1024, 3584)])
def test_reference_nvfp4_cases(mslk, M, N, K):
    from mslk.quantize.triton.fp4_quantize import triton_quantize_nvfp4
    from mslk.quantize.triton.fp4_utils import global_scale_nvfp4
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16) * 0.1
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.01
    gx, gw = global_scale_nvfp4(x), global_scale_nvfp4(w)
    xq, sx = triton_quantize_nvfp4(x, gx)
    wq, sw = triton_quantize_nvfp4(w, gw)
    out = mslk.f4f4bf16(xq, wq, sx, sw, global_scale=1 / (gx * gw))
    torch.testing.assert_close(out, (x @ w.T).to(torch.bfloat16), atol=5e-2, rtol=5e-2)


def test_quantize_symbols_and_per_row_alias(mslk):
    from mslk.quantize.triton.fp8_quantize import quantize_fp8_row, triton_quantize_fp8_row
    a = randn_bf16((6, 4, 2, 33), 1).cuda()
    q1, s1 = quantize_fp8_row(a, align_rows_to=16)
    q2, s2 = triton_quantize_fp8_row(a, align_rows_to=16)
    q_ref, s_ref = oracle.quantize_fp8_row(a.cpu(), align_rows_to=16)
    assert torch.equal(u8(q1.cpu()), u8(q_ref)) and torch.equal(s1.cpu(), s_ref)
    assert torch.equal(u8(q2), u8(q1)) and torch.equal(s2, s1)
    q3, s3 = mslk.quantize_fp8_per_row(a)
    q_ref, s_ref = oracle.quantize_fp8_row(a.cpu())
    assert torch.equal(u8(q3.cpu()), u8(q_ref)) and torch.equal(s3.cpu(), s_ref)
    q4, s4 = quantize_fp8_row(a, output_device=torch.device("cpu"))
    assert q4.device.type == "cpu" and torch.equal(u8(q4), u8(q_ref))


def test_torch_compile_uses_fake_kernels(mslk):
    from mslk.quantize.triton.fp8_quantize import quantize_fp8_row
    w = (torch.randn(256, 512, device="cuda") * 0.02).bfloat16()
    wq, ws = quantize_fp8_row(w)

    def f(x):
        xq, xs = quantize_fp8_row(x)
        return mslk.f8f8bf16_rowwise(xq, wq, xs, ws)

    x = torch.randn(64, 512, device="cuda").bfloat16()
    y = torch.compile(f, backend="eager", fullgraph=True)(x)
    torch.testing.assert_close(y, f(x))


def test_export_strict_and_run(mslk):
    """The reference's export case (test/gemm/gemm_test.py:259-289): export with strict=True, then run the
    exported program on the GPU and compare with the eager call."""
    from mslk.quantize.triton.fp8_quantize import quantize_fp8_row

    class Mod(torch.nn.Module):
        def forward(self, xq, wq, xs, ws):
            return torch.ops.mslk.f8f8bf16_rowwise(xq, wq, xs, ws)

    x = (torch.randn(256, 256, device="cuda") * 0.1).bfloat16()
    w = (torch.randn(256, 256, device="cuda") * 0.01).bfloat16()
    xq, xs = quantize_fp8_row(x)
    wq, ws = quantize_fp8_row(w)
    ep = torch.export.export(Mod().cuda(), (xq, wq, xs, ws), strict=True)
    y = ep.module()(xq, wq, xs, ws)
    assert torch.equal(y, mslk.f8f8bf16_rowwise(xq, wq, xs, ws))


def test_operators_reject_a_cpu_tensor_in_every_pointer_argument(mslk):
    """A host tensor in a slot whose raw pointer reaches a kernel must raise through TORCH_CHECK, not launch."""
    from mslk.quantize.triton.fp8_quantize import quantize_fp8_row
    x = (torch.randn(64, 256, device="cuda") * 0.1).bfloat16()
    w = (torch.randn(128, 256, device="cuda") * 0.01).bfloat16()
    xq, xs = quantize_fp8_row(x)
    wq, ws = quantize_fp8_row(w)
    out = torch.empty((64, 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="output must be a CUDA tensor"):
        mslk.f8f8bf16_rowwise_out(xq, wq, xs, ws, out.cpu())
    with pytest.raises(RuntimeError, match="x_scale must be a CUDA tensor"):
        mslk.f8f8bf16_rowwise(xq, wq, xs.cpu(), ws)
    with pytest.raises(RuntimeError, match="bias must be a CUDA tensor"):
        mslk.f8f8bf16_rowwise(xq, wq, xs, ws, bias=torch.zeros(128))
    ms = torch.tensor([64], dtype=torch.int64, device="cuda")
    with pytest.raises(RuntimeError, match="w_scale must be a CUDA tensor"):
        mslk.f8f8bf16_rowwise_grouped_stacked(xq, wq[None], xs, ws.cpu(), ms)
    with pytest.raises(RuntimeError, match="x_scale must be a CUDA tensor"):
        mslk.f8f8bf16_rowwise_grouped_stacked(xq, wq[None], xs.cpu(), ws, ms)
    # NVFP4: output, global_scale, short scale tensors
    from mslk.quantize.triton.fp4_quantize import triton_quantize_nvfp4
    from mslk.quantize.triton.fp4_utils import global_scale_nvfp4
    gx, gw = global_scale_nvfp4(x), global_scale_nvfp4(w)
    q4, sx = triton_quantize_nvfp4(x, gx)
    w4, sw = triton_quantize_nvfp4(w, gw)
    gs = 1 / (gx * gw)
    with pytest.raises(RuntimeError, match="output must be a CUDA tensor"):
        mslk.f4f4bf16(q4, w4, sx, sw, output=out.cpu(), global_scale=gs)
    with pytest.raises(RuntimeError, match="global_scale must be a CUDA tensor"):
        mslk.f4f4bf16(q4, w4, sx, sw, global_scale=gs.cpu())
    with pytest.raises(RuntimeError, match="x_scale holds"):
        mslk.f4f4bf16(q4, w4, sx.reshape(-1)[: 64 * 16], sw, global_scale=gs)
    torch.testing.assert_close(mslk.f4f4bf16(q4, w4, sx, sw, global_scale=gs), (x @ w.T).to(torch.bfloat16), atol=5e-2, rtol=5e-2)


def test_device_status_operator(mslk):
    """torch.ops.mslk.device_status() reads (and clears) the device status word without ctypes."""
    assert mslk.device_status() == 0
