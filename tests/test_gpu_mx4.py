"""GPU parity tests of the MXFP4 path through the C ABI: the e8m0 quantizer (bit-exact against the oracle and against
outputs of the reference's Triton kernel captured on a B200) and the MXFP4 forms of f4f4bf16, f4f4bf16_grouped_stacked
and f4f4bf16_grouped_mm (the reference's cases, test/gemm/gemm_test.py:2591-2790,2791-2822; exact dequantize-matmul
formula with the 1-ulp bound, and the reference's own tolerance against the unquantized product)."""
import pytest
import torch

import oracle
from helpers import assert_sharp_bf16, load_golden
from golden.make_golden import MX4_CASES, mx4_inputs

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from mslk_b200 import ops as _ops
    torch.backends.cuda.matmul.allow_tf32 = False
    return _ops


def _status():
    from mslk_b200._lib import device_status
    return device_status()


@pytest.mark.parametrize("group", [32, 16])
@pytest.mark.parametrize("mode", [4, 1, 2])
def test_quantizer_bit_exact_vs_oracle(ops, group, mode):
    for i, (name, shape, dtype) in enumerate(MX4_CASES):
        x = mx4_inputs(name, shape, dtype, 700 + i)
        q_ref, s_ref = oracle.quantize_mx4(x, group, mode)
        q, s = ops.quantize_mx4(x.cuda(), group, mode)
        assert torch.equal(q.cpu(), q_ref), (name, group, mode)
        assert torch.equal(s.cpu().view(torch.uint8), s_ref), (name, group, mode)
    assert _status() == 0


def test_quantizer_matches_reference_triton_fixture(ops):
    gold = load_golden("mx4_triton_b200.npz")
    if gold is None:
        pytest.skip("fixture captured from the reference's Triton kernel not present")
    for i, (name, shape, dtype) in enumerate(MX4_CASES):
        x = mx4_inputs(name, shape, dtype, 700 + i).cuda()
        for group in (32, 16):
            for mode in (4, 1, 2):
                q, s = ops.quantize_mx4(x, group, mode)
                key = f"{name}.g{group}.m{mode}"
                assert torch.equal(q.cpu(), torch.from_numpy(gold[key + ".q"])), key
                assert torch.equal(s.cpu().view(torch.uint8), torch.from_numpy(gold[key + ".s"]).reshape(-1)), key
    assert _status() == 0


def test_quantizer_python_symbols_and_errors(ops):
    from mslk_b200 import compat
    compat.install()
    from mslk.quantize.triton.fp4_quantize import triton_quantize_mx4, triton_quantize_mx4_unpack
    x = torch.randn((3, 40, 128), device="cuda").bfloat16()
    q, s = triton_quantize_mx4_unpack(x)
    assert q.shape == (3, 40, 64) and s.dtype == torch.int8 and s.numel() == 128 * 4
    q2, s2 = triton_quantize_mx4(x)
    assert torch.equal(q, q2) and torch.equal(s, s2)
    with pytest.raises(RuntimeError, match="rounding mode"):
        ops.quantize_mx4(x, 32, 0)
    with pytest.raises(AssertionError):
        ops.quantize_mx4(x[..., :48], 32, 4)


def _mx_case(ops, M, N, K, group, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = (torch.randn((M, K), generator=g, device="cuda") * 0.1).bfloat16()
    w = (torch.randn((N, K), generator=g, device="cuda") * 0.01).bfloat16()
    xq, sx = ops.quantize_mx4(x, group)
    wq, sw = ops.quantize_mx4(w, group)
    return x, w, xq, wq, sx, sw


@pytest.mark.parametrize("M,N,K", [(1, 256, 2048), (250, 512, 2048), (250, 1024, 3584), (128, 128, 128), (130, 144, 96),
                                   (300, 272, 320), (2048, 4096, 4096), (512, 2048, 1056)])
@pytest.mark.parametrize("group", [32, 16])
def test_gemm_mxfp4(ops, M, N, K, group):
    x, w, xq, wq, sx, sw = _mx_case(ops, M, N, K, group, seed=M + K)
    y = ops.f4f4bf16(xq, wq, sx, sw, mxfp4_block_size=group)
    y_ref = oracle.gemm_mx4_torch(xq, wq, sx, sw, group)
    assert_sharp_bf16(y, y_ref, f"f4f4bf16 MXFP4 group {group} {M}x{N}x{K}")
    torch.testing.assert_close(y, (x @ w.T).to(torch.bfloat16), atol=8.0e-2, rtol=8.0e-2)   # the reference's own check
    assert _status() == 0


def test_gemm_mxfp4_through_the_operator(ops):
    from mslk_b200 import compat
    compat.install()
    import mslk.gemm  # noqa: F401
    from mslk.quantize.triton.fp4_quantize import triton_quantize_mx4_unpack
    A = torch.randn((250, 2048), dtype=torch.bfloat16, device="cuda") * 0.1
    B = torch.randn((512, 2048), dtype=torch.bfloat16, device="cuda") * 0.01
    aq, a_scale = triton_quantize_mx4_unpack(A)
    bq, b_scale = triton_quantize_mx4_unpack(B)
    out = torch.ops.mslk.f4f4bf16(aq, bq, a_scale, b_scale)
    torch.testing.assert_close(out, A @ B.t(), atol=8.0e-2, rtol=8.0e-2)
    aq, a_scale = triton_quantize_mx4_unpack(A, group_size=16)
    bq, b_scale = triton_quantize_mx4_unpack(B, group_size=16)
    out16 = torch.ops.mslk.f4f4bf16(aq, bq, a_scale, b_scale, None, None, 16)
    torch.testing.assert_close(out16, A @ B.t(), atol=8.0e-2, rtol=8.0e-2)
    assert _status() == 0


def _grouped_mx(ops, m_sizes, N, K, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    xs = [(torch.randn((m, K), generator=g, device="cuda") * 0.1).bfloat16() for m in m_sizes]
    ws = [(torch.randn((N, K), generator=g, device="cuda") * 0.01).bfloat16() for _ in m_sizes]
    xqs, wqs, xss, wss = [], [], [], []
    for x, w in zip(xs, ws):
        q, s = ops.quantize_mx4(x, 32)
        xqs.append(q)
        xss.append(s)
        q, s = ops.quantize_mx4(w, 32)
        wqs.append(q)
        wss.append(s)
    return xs, ws, xqs, wqs, xss, wss


@pytest.mark.parametrize("m_sizes,N,K", [([256], 256, 2048), ([500] * 4, 1024, 2048), ([64, 232, 600], 512, 2048),
                                         ([0, 129, 1, 128, 0, 300], 384, 512), ([300, 0, 1000, 129, 2047, 620], 2048, 1024)])
def test_grouped_mxfp4(ops, m_sizes, N, K):
    xs, ws, xqs, wqs, xss, wss = _grouped_mx(ops, m_sizes, N, K, seed=sum(m_sizes) + N)
    xq = torch.cat(xqs, dim=0)
    wq = torch.stack(wqs, dim=0)
    x_scale = torch.cat(xss, dim=0)     # every group's swizzled block, padded to 128 rows, one after the other
    w_scale = torch.stack(wss, dim=0)
    ms = torch.tensor(m_sizes, dtype=torch.int64, device="cuda")
    y = ops.f4f4bf16_grouped_stacked(xq, wq, x_scale, w_scale, ms)       # use_mx=True is the default
    assert y.shape == (sum(m_sizes), N)
    r = 0
    for g, m in enumerate(m_sizes):
        if m:
            y_ref = oracle.gemm_mx4_torch(xqs[g], wqs[g], xss[g], wss[g], 32)
            assert_sharp_bf16(y[r:r + m], y_ref, f"grouped MXFP4 group {g} of {m_sizes}")
            torch.testing.assert_close(y[r:r + m], (xs[g] @ ws[g].T).to(torch.bfloat16), atol=8.0e-2, rtol=8.0e-2)
        r += m
    # the end-offset form with e8m0-typed scales selects the same arithmetic
    e8 = getattr(torch, "float8_e8m0fnu", None)
    if e8 is not None:
        offsets = ms.cumsum(0).to(torch.int32)
        y2 = ops.f4f4bf16_grouped_mm(xq, wq.transpose(-2, -1), x_scale.view(e8), w_scale.view(e8), offsets)
        assert torch.equal(y, y2)
    assert _status() == 0
