"""GPU parity tests of the MoE token gather / scatter kernels, through the C ABI.

gather_scale_dense_tokens is exact (one fp32 product, one rounding): bit for bit against the oracle.
gather_scale_quant_dense_tokens: bit for bit against outputs captured from the reference's Triton kernel
on a B200; against the oracle (IEEE instead of approximate division) to a few ulps / one e4m3 code.
scatter-add: exact for int32 and for one contribution per row; the reference's tolerance
(test/moe/gather_scatter_test.py:297-303: atol 1e-3, rtol 1.6e-2) where the order of atomics matters."""
import pytest
import torch

import oracle
from helpers import load_golden, u8
from golden.make_golden import GATHER_CASES, gather_inputs

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from mslk_b200 import ops as _ops
    return _ops


def _status():
    from mslk_b200._lib import device_status
    return device_status()


def _order(b):
    b = b.to(torch.int16)
    return torch.where((b & 0x80) != 0, -(b & 0x7f), b & 0x7f)


@pytest.mark.parametrize("E,T,D,partial,rowmajor", [
    (2, 1, 5120, False, True), (8, 128, 5120, True, False), (2, 4096, 5120, False, False),
    (8, 4096, 5120, True, True), (4, 37, 264, False, False), (3, 50, 100, True, True), (2, 9, 8, False, True),
])
def test_gather_scale_exact(ops, E, T, D, partial, rowmajor):
    # test/moe/gather_scatter_test.py:52-127
    x, tok, ex, scores = gather_inputs(T, D, E, 7 * T + E, rowmajor)
    n = T // 2 if partial else T
    vt = torch.tensor([n], dtype=torch.int32, device="cuda") if partial else None
    tok_d, ex_d = tok.clone(), ex.clone()
    if partial:                      # as the reference's test: invalid rows carry -1
        tok_d[n:] = -1
        ex_d[n:] = -1
    out = ops.gather_scale_dense_tokens(x.cuda(), tok_d.cuda(), ex_d.cuda(), scores.cuda(), vt)
    ref = oracle.gather_scale_dense_tokens(x, tok, ex, scores, n)
    assert torch.equal(out.cpu()[:n].view(torch.int16), ref[:n].view(torch.int16))
    # and the torch expression of the reference's test
    tref = x[tok.long()] * scores[tok.long(), ex].view(-1, 1)
    assert torch.equal(out.cpu()[:n], tref[:n])
    assert _status() == 0


def test_gather_scale_quant_triton_fixture_bit_exact(ops):
    gold = load_golden("gather_scale_quant_triton_b200.npz")
    if gold is None:
        pytest.skip("fixture captured from the reference's Triton kernel not present")
    for i, (name, T, D, E, ub, valid, rowmajor) in enumerate(GATHER_CASES):
        x, tok, ex, scores = gather_inputs(T, D, E, 500 + i, rowmajor)
        ubt = None if ub is None else torch.tensor([ub], dtype=torch.float32, device="cuda")
        vt = None if valid is None else torch.tensor([valid], dtype=torch.int32, device="cuda")
        q, s = ops.gather_scale_quant_dense_tokens(x.cuda(), tok.cuda(), ex.cuda(), scores.cuda(), ubt, vt)
        n = T if valid is None else valid
        s_ref = torch.from_numpy(gold[f"{name}.s"]).reshape(T)
        q_ref = torch.from_numpy(gold[f"{name}.q"]).reshape(T, D)
        assert torch.equal(s.cpu()[:n].view(torch.int32), s_ref[:n].view(torch.int32)), f"{name}: inverse scales differ"
        assert torch.equal(u8(q.cpu())[:n], q_ref[:n]), f"{name}: bytes differ from the Triton capture"
    assert _status() == 0


@pytest.mark.parametrize("E,T,D,partial,rowmajor,use_ub", [
    (2, 1, 5120, False, True, True), (8, 128, 5120, True, False, True), (2, 4096, 5120, False, True, False),
    (4, 33, 2056, False, False, False), (3, 20, 100, True, True, True), (2, 6, 33000, False, True, False),
])
def test_gather_scale_quant_vs_oracle_and_reference_tolerance(ops, E, T, D, partial, rowmajor, use_ub):
    # test/moe/gather_scatter_test.py:128-219: scale within rtol 1e-5, bytes within one fp8 step
    x, tok, ex, scores = gather_inputs(T, D, E, 11 * T + E, rowmajor)
    n = T // 2 if partial else T
    vt = torch.tensor([n], dtype=torch.int32, device="cuda") if partial else None
    ub = torch.tensor([1200.0]) if use_ub else None
    q, s = ops.gather_scale_quant_dense_tokens(x.cuda(), tok.cuda(), ex.cuda(), scores.cuda(),
                                               None if ub is None else ub.cuda(), vt)
    q_ref, s_ref = oracle.gather_scale_quant_dense_tokens(x, tok, ex, scores, ub, n)
    torch.testing.assert_close(s.cpu()[:n], s_ref[:n], atol=1e-7, rtol=1e-5)
    d = (_order(u8(q.cpu())[:n]) - _order(u8(q_ref)[:n])).abs()
    if n:   # products of two bf16 values land on exact e4m3 ties often enough for a one-ulp scale to tip a few
        assert int(d.max()) <= 1 and int((d != 0).sum()) <= max(8, 2e-3 * d.numel())
    torch.testing.assert_close(q.cpu()[:n].float(), q_ref[:n].float(), atol=0.0625, rtol=0.125)
    assert _status() == 0


@pytest.mark.parametrize("num_tokens,dim,partial,k,dtype", [
    (1, 5120, False, 1, torch.bfloat16), (128, 5120, True, 1, torch.bfloat16), (2048, 5120, False, 1, torch.bfloat16),
    (128, 5120, False, 4, torch.int32), (2048, 5120, True, 4, torch.int32), (64, 100, False, 1, torch.bfloat16),
    (64, 36, True, 4, torch.int32), (256, 1024, False, 1, torch.float32), (256, 1024, False, 1, torch.float16),
])
def test_scatter_add_dense_exact_cases(ops, num_tokens, dim, partial, k, dtype):
    # test/moe/gather_scatter_test.py:228-306 (int32 when several rows land on one token, as there)
    g = torch.Generator().manual_seed(num_tokens + k)
    a = num_tokens * k
    in_tokens = (torch.randn((a, dim), generator=g) * (8 if dtype == torch.int32 else 1)).to(dtype)
    out_tokens = (torch.randn((num_tokens, dim), generator=g) * (8 if dtype == torch.int32 else 1)).to(dtype)
    n = num_tokens // 2 if partial else num_tokens
    vt = torch.tensor([n * k], dtype=torch.int32, device="cuda") if partial else None
    tok = -torch.ones(a, dtype=torch.int32)
    if n:
        tok[: n * k] = (torch.randperm(n * k, generator=g) % n).to(torch.int32)
    test = out_tokens.clone().cuda()
    ops.scatter_add_dense_tokens(test, in_tokens.cuda(), tok.cuda(), vt)
    ref = out_tokens.clone()
    if n:
        ref.scatter_add_(0, tok[: n * k].long().view(-1, 1).expand(-1, dim), in_tokens[: n * k])
    assert torch.equal(test.cpu(), ref)
    if dtype in (torch.bfloat16, torch.int32, torch.float32):
        ref2 = out_tokens.clone()
        oracle.scatter_add_dense_tokens(ref2, in_tokens, tok, n * k)
        assert torch.equal(test.cpu(), ref2)
    assert _status() == 0


def test_scatter_add_dense_bf16_several_rows_per_token(ops):
    g = torch.Generator().manual_seed(5)
    num_tokens, k, dim = 512, 4, 2048
    in_tokens = torch.randn((num_tokens * k, dim), generator=g).to(torch.bfloat16)
    out_tokens = torch.randn((num_tokens, dim), generator=g).to(torch.bfloat16)
    tok = (torch.randperm(num_tokens * k, generator=g) % num_tokens).to(torch.int64)
    test = out_tokens.clone().cuda()
    ops.scatter_add_dense_tokens(test, in_tokens.cuda(), tok.cuda())
    ref = out_tokens.float().index_add_(0, tok, in_tokens.float())
    # k roundings of 2^-9 relative to the running sum
    torch.testing.assert_close(test.cpu().float(), ref, atol=6e-2, rtol=1.6e-2)
    assert _status() == 0


@pytest.mark.parametrize("num_tokens,num_experts,ep_size,dim,balanced,k", [
    (64, 16, 2, 5120, True, 1), (256, 128, 16, 5120, False, 1), (64, 16, 16, 5120, False, 4),
    (256, 128, 2, 5120, True, 4), (64, 16, 2, 72, False, 4),
])
def test_scatter_add_padded(ops, num_tokens, num_experts, ep_size, dim, balanced, k):
    # test/moe/gather_scatter_test.py:308-406
    g = torch.Generator().manual_seed(num_experts + k)
    dtype = torch.bfloat16 if k == 1 else torch.int32
    a = num_tokens * k
    in_tokens = (torch.randn((ep_size, a, dim), generator=g) * (8 if k > 1 else 1)).to(dtype)
    out_tokens = (torch.randn((num_tokens, dim), generator=g) * (8 if k > 1 else 1)).to(dtype)
    if balanced:
        counts = torch.full((num_experts,), a // num_experts, dtype=torch.int32)
    else:
        counts = torch.bincount(torch.randint(0, num_experts, (a,), generator=g), minlength=num_experts)
    tok = (torch.randperm(a, generator=g) % num_tokens).to(torch.int32)
    test = out_tokens.clone().cuda()
    ops.scatter_add_padded_tokens(in_tokens.cuda(), counts.cuda(), tok.cuda(), test)
    ref = out_tokens.clone()
    oracle.scatter_add_padded_tokens(in_tokens, counts, tok, ref)
    # the reference test's own formulation: per rank, the slice of rows of that rank's experts
    ref2 = out_tokens.clone()
    cs = [0] + torch.cumsum(counts, 0).tolist()
    per = num_experts // ep_size
    for rank in range(ep_size):
        s0, e0 = cs[per * rank], cs[per * (rank + 1)]
        if s0 != e0:
            ref2.scatter_add_(0, tok[s0:e0].long().view(-1, 1).expand(-1, dim), in_tokens[rank, s0:e0])
    assert torch.equal(ref, ref2)
    if dtype == torch.int32 or k == 1:
        assert torch.equal(test.cpu(), ref)
    assert _status() == 0


def test_bad_index_is_reported_not_followed(ops):
    x, tok, ex, scores = gather_inputs(16, 64, 2, 1, True)
    tok[3] = 99                         # outside [0, T): the row is skipped and the status word says so
    out = torch.zeros((16, 64), dtype=torch.bfloat16, device="cuda")
    from mslk_b200._lib import check, lib
    xd, td, ed, sd = x.cuda(), tok.cuda(), ex.cuda(), scores.cuda()
    check(lib.mslk_b200_gather_scale_dense_tokens(
        xd.data_ptr(), 1, 16, 64, td.data_ptr(), 32, ed.data_ptr(), 64, sd.data_ptr(), 1,
        2, sd.stride(0), sd.stride(1), 16, None, out.data_ptr(), torch.cuda.current_stream().cuda_stream), "gather")
    assert _status() == 0x100
    assert float(out[3].float().abs().max()) == 0.0 and float(out[4].float().abs().max()) > 0.0
    assert _status() == 0


def test_operator_paths_and_empty(ops):
    import mslk_b200.moe.gather_scatter as gs
    x, tok, ex, scores = gather_inputs(32, 1024, 4, 2, False)
    xd, td, ed, sd = x.cuda(), tok.cuda(), ex.cuda(), scores.cuda()
    a = torch.ops.mslk.gather_scale_dense_tokens(xd, td, ed, sd)
    assert torch.equal(a, gs.gather_scale_dense_tokens(xd, td, ed, sd))
    q = torch.ops.mslk.gather_scale_quant_dense_tokens(xd, td, ed, sd)
    q2, s2 = gs.gather_scale_quant_dense_tokens(xd, td, ed, sd)
    assert torch.equal(u8(q), u8(q2)) and s2.shape == (32,)
    out = torch.zeros((32, 1024), dtype=torch.bfloat16, device="cuda")
    torch.ops.mslk.scatter_add_dense_tokens(out, a, td)
    assert torch.equal(out[td.long()], a)
    e = gs.gather_scale_dense_tokens(xd, td[:0], ed[:0], sd)
    assert e.shape == (0, 1024)
    gs.scatter_add_dense_tokens(out, a[:0], td[:0])
    with pytest.raises(RuntimeError):
        gs.gather_scale_dense_tokens(x, tok, ex, scores)
    assert _status() == 0
