"""GPU parity tests of the fused SwiGLU (+ per-row FP8 quantize) kernels, through the C ABI.

Three checkers: (1) outputs captured from the reference's Triton kernel on a B200 -- bit for bit;
(2) the CPU oracle, which evaluates the sigmoid with exact expf / IEEE division -- the kernel (like
the reference's) uses approximate exp2 / division, so agreement is to one e4m3 code on few elements
and ulps on the scale; (3) the reference's own test tolerance on the dequantized product
(test/moe/activation_test.py:97-168: rtol 1e-1, atol 1e-3)."""
import pytest
import torch

import oracle
from helpers import load_golden, u8
from golden.make_golden import SILU_CASES, silu_inputs

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from mslk_b200 import ops as _ops
    return _ops


def _case_inputs(i, name, T, D, ub, valid, contiguous, x=None):
    x = silu_inputs(name, T, D, 400 + i) if x is None else x
    x = x.cuda()
    x0, x1 = x[:, :D], x[:, D:]
    if contiguous:
        x0, x1 = x0.contiguous(), x1.contiguous()
    ubt = None if ub is None else torch.tensor([ub], dtype=torch.float32, device="cuda")
    vt = None if valid is None else torch.tensor([valid], dtype=torch.int32, device="cuda")
    return x0, x1, ubt, vt


def _code_distance(qa, qb):
    """|difference| of two e4m3 byte tensors measured in code steps along the ordered value line."""
    def order(b):
        b = b.to(torch.int16)
        mag = b & 0x7f
        return torch.where((b & 0x80) != 0, -mag, mag)
    return (order(qa) - order(qb)).abs()


def _check_against_oracle(q, s, x0, x1, ub, valid, tag):
    T = x0.shape[0]
    n = T if valid is None else valid
    q_ref, s_ref = oracle.silu_mul_quant(x0.cpu(), x1.cpu(), None if ub is None else ub.cpu(), valid)
    s, q = s.cpu(), u8(q.cpu())
    assert torch.allclose(s[:n], s_ref[:n], rtol=2e-6, atol=0), f"{tag}: inverse scales differ"
    dist = _code_distance(q[:n], u8(q_ref)[:n])
    assert int(dist.max()) <= 1, f"{tag}: a byte is more than one e4m3 code away from the oracle"
    assert float((dist != 0).float().mean()) < 2e-3, f"{tag}: too many bytes differ from the oracle"


def test_triton_fixture_bit_exact(ops):
    gold = load_golden("silu_mul_quant_triton_b200.npz")
    if gold is None:
        pytest.skip("fixture captured from the reference's Triton kernel not present")
    for i, (name, T, D, ub, valid, contiguous) in enumerate(SILU_CASES):
        x0, x1, ubt, vt = _case_inputs(i, name, T, D, ub, valid, contiguous)
        q, s = ops.silu_mul_quant(x0, x1, ubt, vt)
        n = T if valid is None else valid
        s_ref = torch.from_numpy(gold[f"{name}.s"]).reshape(T)
        q_ref = torch.from_numpy(gold[f"{name}.q"]).reshape(T, D)
        assert torch.equal(s.cpu()[:n].view(torch.int32), s_ref[:n].view(torch.int32)), f"{name}: inverse scales differ"
        qa = u8(q.cpu())[:n]
        if not torch.equal(qa, q_ref[:n]):
            bad = (qa != q_ref[:n]).nonzero()
            raise AssertionError(f"{name}: {bad.shape[0]} bytes differ from the Triton capture, first at {bad[0].tolist()}")


def test_case_list_against_oracle(ops):
    for i, case in enumerate(SILU_CASES):
        name, T, D, ub, valid, contiguous = case
        x0, x1, ubt, vt = _case_inputs(i, *case)
        q, s = ops.silu_mul_quant(x0, x1, ubt, vt)
        _check_against_oracle(q, s, x0, x1, ubt, valid, name)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("D", [8, 100, 2049, 4096, 6152, 16384, 16392, 16408, 28672, 32768, 40000])
def test_widths_and_dtypes(ops, dtype, D):
    # every dispatch bucket of the vector kernel, the general kernel (odd D) and very wide rows
    g = torch.Generator().manual_seed(D)
    x = (torch.randn((5, 2 * D), generator=g) * 1.5).to(dtype).cuda()
    x0, x1 = x[:, :D], x[:, D:]
    q, s = ops.silu_mul_quant(x0, x1)
    _check_against_oracle(q, s, x0, x1, None, None, f"D={D} {dtype}")
    y = ops.silu_mul(x0, x1)
    y_ref = oracle.silu_mul(x0.cpu(), x1.cpu()).to(dtype)
    assert torch.allclose(y.cpu().float(), y_ref.float(), rtol=2 ** -7, atol=1e-6)


def test_like_reference_test(ops):
    # test/moe/activation_test.py:97-168: T in a set of small and partial sizes, D = 5120, optional ub,
    # partial token counts; dequantized product against the torch expression within rtol 1e-1 / atol 1e-3
    D = 5120
    for T, partial, use_ub in [(1, False, False), (128, True, True), (2048, False, True), (16384, True, False)]:
        g = torch.Generator().manual_seed(T)
        x0 = torch.randn((T, D), generator=g).to(torch.bfloat16).cuda()
        x1 = torch.randn((T, D), generator=g).to(torch.bfloat16).cuda()
        n = max(T // 2, 1) if partial else T
        vt = torch.tensor([n], dtype=torch.int32, device="cuda") if partial else None
        ub = torch.tensor([1200.0], dtype=torch.float32, device="cuda") if use_ub else None
        q, s = ops.silu_mul_quant(x0, x1, ub, vt)
        ref = (x0[:n].float() * torch.sigmoid(x0[:n].float()) * x1[:n].float())
        deq = q[:n].float() * s[:n, None]
        torch.testing.assert_close(deq, ref, rtol=1e-1, atol=1e-3)
        y = ops.silu_mul(x0, x1, vt)
        torch.testing.assert_close(y[:n].float(), ref, rtol=1e-2, atol=1e-3)


def test_rows_past_valid_count_untouched(ops):
    T, D = 64, 1024
    g = torch.Generator().manual_seed(3)
    x0 = torch.randn((T, D), generator=g).to(torch.bfloat16).cuda()
    x1 = torch.randn((T, D), generator=g).to(torch.bfloat16).cuda()
    from mslk_b200._lib import check, lib
    q = torch.full((T, D), 0x55, dtype=torch.uint8, device="cuda")
    s = torch.full((T,), -7.0, dtype=torch.float32, device="cuda")
    vt = torch.tensor([10], dtype=torch.int32, device="cuda")
    check(lib.mslk_b200_silu_mul_quant(x0.data_ptr(), x1.data_ptr(), 1, T, D, D, D, None, vt.data_ptr(), q.data_ptr(),
                                       s.data_ptr(), torch.cuda.current_stream().cuda_stream), "silu_mul_quant")
    torch.cuda.synchronize()
    assert bool((q[10:] == 0x55).all()) and bool((s[10:] == -7.0).all())
    assert bool((s[:10] > 0).all())
    # a count larger than T processes every row; zero processes none
    for count, expect in ((1000, T), (0, 0)):
        q.fill_(0x55)
        vt.fill_(count)
        check(lib.mslk_b200_silu_mul_quant(x0.data_ptr(), x1.data_ptr(), 1, T, D, D, D, None, vt.data_ptr(),
                                           q.data_ptr(), s.data_ptr(), torch.cuda.current_stream().cuda_stream), "silu")
        torch.cuda.synchronize()
        touched = int((q != 0x55).any(dim=1).sum())
        assert touched == expect


def test_empty_and_rejected(ops):
    e = torch.empty((0, 128), dtype=torch.bfloat16, device="cuda")
    q, s = ops.silu_mul_quant(e, e)
    assert q.shape == (0, 128) and s.shape == (0,)
    assert ops.silu_mul(e, e).shape == (0, 128)
    x = torch.zeros((4, 128), dtype=torch.float32, device="cuda")
    with pytest.raises(RuntimeError):
        ops.silu_mul_quant(x, x)
    with pytest.raises(RuntimeError):
        ops.silu_mul_quant(x.cpu().bfloat16(), x.cpu().bfloat16())
    with pytest.raises(AssertionError):
        ops.silu_mul_quant(x.bfloat16(), x.bfloat16()[:, :64])


def test_operator_and_module_paths(ops):
    import mslk_b200.moe.activation as act
    g = torch.Generator().manual_seed(9)
    x0 = torch.randn((33, 2048), generator=g).to(torch.bfloat16).cuda()
    x1 = torch.randn((33, 2048), generator=g).to(torch.bfloat16).cuda()
    q0, s0 = ops.silu_mul_quant(x0, x1)
    q1, s1 = torch.ops.mslk.silu_mul_quant(x0, x1)
    q2, s2 = act.silu_mul_quant(x0, x1, None, None)
    assert torch.equal(u8(q0), u8(q1)) and torch.equal(u8(q0), u8(q2)) and torch.equal(s0, s1) and torch.equal(s0, s2)
    assert torch.equal(torch.ops.mslk.silu_mul(x0, x1), ops.silu_mul(x0, x1))


def test_feeds_the_down_projection(ops):
    # the fused op replaces silu_mul -> quantize_fp8_row in front of f8f8bf16_rowwise: its inverse
    # scale is the x_scale of the GEMM
    T, D, N = 256, 2048, 512
    g = torch.Generator().manual_seed(11)
    x0 = torch.randn((T, D), generator=g).to(torch.bfloat16).cuda()
    x1 = torch.randn((T, D), generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn((N, D), generator=g) * 0.05).to(torch.bfloat16).cuda()
    wq, ws = ops.quantize_fp8_row(w)
    xq, xs = ops.silu_mul_quant(x0, x1)
    y = ops.f8f8bf16_rowwise(xq, wq, xs, ws)
    ref = (x0.float() * torch.sigmoid(x0.float()) * x1.float()) @ w.float().T
    err = (y.float() - ref).norm() / ref.norm()
    assert float(err) < 0.06
