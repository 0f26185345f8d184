"""GPU parity tests of the per-row FP8 quantizer: the CUDA kernel (through the C ABI)
must equal the oracle bit for bit -- quantized bytes and fp32 scales."""
import pytest
import torch

import oracle
from helpers import bf16, load_golden, randn_bf16, u8
from golden.make_golden import FP8_ROW_CASES, _fp8_inputs

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from mslk_b200 import ops as _ops
    return _ops


def _status():
    from mslk_b200._lib import device_status
    return device_status()


def _assert_same(q, s, q_ref, s_ref, tag):
    assert q.shape == q_ref.shape and s.shape == s_ref.shape, tag
    assert torch.equal(s.cpu().view(torch.int32), s_ref.view(torch.int32)), f"{tag}: scales differ"
    qa, qb = u8(q.cpu()), u8(q_ref)
    if not torch.equal(qa, qb):
        bad = (qa != qb).nonzero()
        raise AssertionError(f"{tag}: {bad.shape[0]} bytes differ, first at {bad[0].tolist()}")


def test_reference_case_list(ops):
    for i, (name, shape, kw) in enumerate(FP8_ROW_CASES):
        a, ub, zs = _fp8_inputs(name, shape, kw, seed=i)
        q_ref, s_ref = oracle.quantize_fp8_row(a, ub, zs, kw.get("align_rows_to"))
        q, s = ops.quantize_fp8_row(a.cuda(), None if ub is None else ub.cuda(),
                                    None if zs is None else zs.cuda(), kw.get("align_rows_to"))
        _assert_same(q, s, q_ref, s_ref, name)
    assert _status() == 0


def test_triton_fixture_if_present(ops):
    gold = load_golden("fp8_row_triton_b200.npz")
    if gold is None:
        pytest.skip("fixture captured from the reference's Triton kernel not present")
    for i, (name, shape, kw) in enumerate(FP8_ROW_CASES):
        a, ub, zs = _fp8_inputs(name, shape, kw, seed=i)
        q, s = ops.quantize_fp8_row(a.cuda(), None if ub is None else ub.cuda(),
                                    None if zs is None else zs.cuda(), kw.get("align_rows_to"))
        assert torch.equal(s.cpu().reshape(-1).view(torch.int32),
                           torch.from_numpy(gold[f"{name}.s"]).reshape(-1).view(torch.int32)), name
        assert torch.equal(u8(q.cpu()).reshape(-1), torch.from_numpy(gold[f"{name}.q"]).reshape(-1)), name


def test_column_sweep_like_reference(ops):
    # test/quantize/triton/fp8_quantize_test.py:145-166: K = 1..9000 step 100, with and without padding
    for n_col in range(1, 9000, 100):
        a = randn_bf16((2, n_col), n_col)
        for align in (None, 8):
            q_ref, s_ref = oracle.quantize_fp8_row(a, None, None, align)
            q, s = ops.quantize_fp8_row(a.cuda(), align_rows_to=align)
            _assert_same(q, s, q_ref, s_ref, f"K={n_col} align={align}")
    assert _status() == 0


@pytest.mark.parametrize("shape", [(4096, 4096), (1, 4096), (16, 4096), (128, 14336), (2048, 14336),
                                   (512, 28672), (333, 777), (1, 128), (128, 1), (8192, 4096), (64, 5120),
                                   (32, 8192), (7, 32768), (3, 40000)])
def test_baseline_shapes_bit_exact(ops, shape):
    a = randn_bf16(shape, 7)
    q_ref, s_ref = oracle.quantize_fp8_row(a)
    q, s = ops.quantize_fp8_row(a.cuda())
    _assert_same(q, s, q_ref, s_ref, str(shape))
    assert _status() == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [(64, 4096), (5, 100), (16, 14336)])
def test_other_input_dtypes(ops, dtype, shape):
    g = torch.Generator().manual_seed(3)
    a = (torch.randn(shape, generator=g) * 3).to(dtype)
    q_ref, s_ref = oracle.quantize_fp8_row(a)
    q, s = ops.quantize_fp8_row(a.cuda())
    _assert_same(q, s, q_ref, s_ref, f"{dtype} {shape}")


def test_value_ranges_and_scale_ub(ops):
    # large and tiny magnitudes (true-division fallback rows), and an upper bound that clamps
    g = torch.Generator().manual_seed(5)
    base = torch.randn((12, 512), generator=g)
    mags = torch.tensor([1e-30, 1e-20, 1e-6, 1e-3, 1.0, 30.0, 1e4, 1e10, 1e20, 1e30, 3e38, 0.0])[:, None]
    a = (base.clamp(-3, 3) / 3 * mags).to(torch.bfloat16)
    for ub in (None, torch.tensor([0.5]), torch.tensor([1200.0])):
        q_ref, s_ref = oracle.quantize_fp8_row(a, ub)
        q, s = ops.quantize_fp8_row(a.cuda(), None if ub is None else ub.cuda())
        _assert_same(q, s, q_ref, s_ref, f"ub={ub}")


def test_strided_rows_and_views(ops):
    a = randn_bf16((64, 4096), 11).cuda()
    view = a[:, 1024:3072]            # row stride 4096, 16-byte aligned rows -> vector path
    q, s = ops.quantize_fp8_row(view)
    q_ref, s_ref = oracle.quantize_fp8_row(view.cpu())
    _assert_same(q, s, q_ref, s_ref, "column slice")
    odd = a[:, 3:1003]                # misaligned rows -> general path
    q, s = ops.quantize_fp8_row(odd)
    q_ref, s_ref = oracle.quantize_fp8_row(odd.cpu())
    _assert_same(q, s, q_ref, s_ref, "odd slice")
    t = a.t()                         # inner stride != 1
    q, s = ops.quantize_fp8_row(t)
    q_ref, s_ref = oracle.quantize_fp8_row(t.cpu())
    _assert_same(q, s, q_ref, s_ref, "transposed")


def test_empty_and_errors(ops):
    q, s = ops.quantize_fp8_row(torch.empty((0, 128), dtype=torch.bfloat16, device="cuda"))
    assert q.shape == (0, 128) and s.shape == (0,)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.quantize_fp8_row(torch.zeros((2, 16), dtype=torch.bfloat16))
    with pytest.raises(Exception, match="same device"):
        ops.quantize_fp8_row(torch.zeros((2, 16), dtype=torch.bfloat16, device="cuda"), scale_ub=torch.ones(1))


def test_full_size_properties(ops):
    # size-independent properties at a full benchmark size: round trip within the reference's own
    # tolerance (test/quantize/fp8_quantize_correctness_test.py:119-124), every row hits +-448
    a = randn_bf16((8192, 8192), 13).cuda()
    q, s = ops.quantize_fp8_row(a)
    deq = q.float() * s[:, None]
    torch.testing.assert_close(deq, a.float(), atol=2.5e-1, rtol=1e-3 + 2 ** -4)
    assert (q.float().abs().amax(dim=1) == 448).all()
    assert torch.equal(s.cpu(), a.float().abs().amax(dim=1).clamp(min=1 / 512).cpu() / 448)  # true division on CPU
    # quantizing with fp32 input of the same values gives the same result as bf16 input
    q2, s2 = ops.quantize_fp8_row(a.float())
    assert torch.equal(u8(q2), u8(q)) and torch.equal(s2, s)
    assert _status() == 0
