"""GPU parity tests of the NVFP4 quantizer (bit-exact) and the NVFP4 GEMM (tolerance) through the C ABI."""
import pytest
import torch

import oracle
from helpers import bf16, load_golden, randn_bf16, u8
from golden.make_golden import NVFP4_CASES

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from mslk_b200 import ops as _ops
    torch.backends.cuda.matmul.allow_tf32 = False
    return _ops


def _status():
    from mslk_b200._lib import device_status
    return device_status()


def test_quantize_matches_reference_fixtures(ops):
    # torch reference of the reference's own test and its Triton kernel run on a B200
    for fname in ("nvfp4_torch_ref.npz", "nvfp4_triton_b200.npz"):
        gold = load_golden(fname)
        assert gold is not None, fname
        for name, shape in NVFP4_CASES:
            x = bf16(gold[f"{name}.x"]).cuda()
            gs = torch.from_numpy(gold[f"{name}.gs"]).cuda()
            q, s = ops.quantize_nvfp4(x, gs)
            assert torch.equal(q.cpu(), torch.from_numpy(gold[f"{name}.q"])), (fname, name)
            assert torch.equal(u8(s.cpu()).reshape(-1), torch.from_numpy(gold[f"{name}.s_blocked"]).reshape(-1)), (fname, name)
    assert _status() == 0


@pytest.mark.parametrize("shape", [(4096, 4096), (4000, 4096), (4096, 4080), (4000, 4080), (1, 8192), (32, 8192),
                                   (250, 3584), (128, 16)])
@pytest.mark.parametrize("use_gs", [True, False])
def test_quantize_bit_exact_vs_oracle(ops, shape, use_gs):
    x = randn_bf16(shape, 5)
    gs = oracle.global_scale_nvfp4(x) if use_gs else None
    q_ref, s_ref = oracle.quantize_nvfp4(x, gs)
    q, s = ops.quantize_nvfp4(x.cuda(), None if gs is None else gs.cuda())
    assert torch.equal(q.cpu(), q_ref)
    assert torch.equal(u8(s.cpu()), u8(s_ref))


def _gemm_case(ops, M, N, K, seed=0):
    x = randn_bf16((M, K), seed).cuda()
    w = randn_bf16((N, K), seed + 1).cuda()
    gx = (448.0 * 6.0) / x.abs().amax().float()
    gw = (448.0 * 6.0) / w.abs().amax().float()
    xq, sx = ops.quantize_nvfp4(x, gx)
    wq, sw = ops.quantize_nvfp4(w, gw)
    alpha = (1.0 / (gx * gw)).reshape(1)
    y = ops.f4f4bf16(xq, wq, sx, sw, global_scale=alpha)
    return x, w, xq, wq, sx, sw, alpha, y


@pytest.mark.parametrize("M,N,K", [(128, 128, 256), (128, 128, 64), (1, 256, 2048), (250, 512, 2048),
                                   (250, 1024, 3584), (130, 144, 320), (512, 2048, 1024), (32, 4096, 8192),
                                   (300, 272, 96)])
def test_gemm_vs_fp32_dequant_formula(ops, M, N, K):
    x, w, xq, wq, sx, sw, alpha, y = _gemm_case(ops, M, N, K)
    y_ref = oracle.gemm_nvfp4_torch(xq, wq, sx, sw, alpha)
    scale = max(1.0, float(y_ref.float().std()))
    torch.testing.assert_close(y.float(), y_ref.float(), rtol=1.6e-2, atol=1e-2 * scale)
    # sanity against the unquantized product (4-bit error: norm bound only; the reference's own
    # end-to-end tolerance test with its data scales is in test_gpu_torch_ops.py)
    y_full = x.float() @ w.float().T
    assert (y.float() - y_full).norm() / y_full.norm() < 0.2
    assert _status() == 0


def test_gemm_small_vs_c_oracle(ops):
    x, w, xq, wq, sx, sw, alpha, y = _gemm_case(ops, 40, 48, 128, seed=3)
    y_c = oracle.gemm_nvfp4(xq.cpu(), wq.cpu(), sx.cpu(), sw.cpu(), alpha.cpu())
    torch.testing.assert_close(y.cpu().float(), y_c.float(), rtol=1.6e-2, atol=1e-2 * max(1.0, float(y_c.float().std())))


def test_gemm_large_tiles_and_output_arg(ops):
    # enough 256-wide tiles to take the single-accumulator configuration
    M, N, K = 8192, 8192, 1024
    x, w, xq, wq, sx, sw, alpha, y = _gemm_case(ops, M, N, K, seed=7)
    rows = torch.arange(0, M, 97, device="cuda")
    y_ref = oracle.gemm_nvfp4_torch(xq[rows], wq, _rows_of_scales(sx, rows, K), sw, alpha)
    torch.testing.assert_close(y[rows].float(), y_ref.float(), rtol=1.6e-2, atol=1e-2 * float(y_ref.float().std()))
    out = torch.empty_like(y)
    y2 = ops.f4f4bf16(xq, wq, sx, sw, output=out, global_scale=alpha)
    assert y2.data_ptr() == out.data_ptr() and torch.equal(out, y)
    with pytest.raises(RuntimeError, match="mxfp4_block_size"):
        ops.f4f4bf16(xq, wq, sx, sw, global_scale=alpha, mxfp4_block_size=8)
    assert _status() == 0


def _rows_of_scales(s_blocked, rows, K):
    """Blocked scales of a row subset (un-swizzle, pick rows, swizzle again)."""
    M = s_blocked.shape[0]
    plain = oracle.from_blocked(u8(s_blocked.cpu()).reshape(-1), M, K // 16)
    sub = plain[rows.cpu()]
    return oracle.to_blocked(sub).view(torch.float8_e4m3fn).cuda()


# ---------------------------------------------------------------------------
# Few tokens (1 <= M <= 128): the weight-streaming kernel (weights on the accumulator rows, tokens on
# the columns, K optionally split over CTAs).  Shapes: every token tile (16/32/64/128) with a ragged
# token count, N not a multiple of 128, K with a partial last scale atom (K % 64 != 0) and a partial
# last K block (K % 256 != 0), K long enough to be split; 65..128 tokens take this kernel only with more
# than one wave of 128-row weight blocks (N > 128 x SMs) or with long K split in clusters, otherwise the
# general kernel.
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (7, 144, 96), (16, 4096, 2048), (17, 384, 320), (33, 1024, 4096),
                                   (64, 272, 1056), (65, 256, 16384), (100, 4096, 2048), (128, 400, 16384),
                                   (3, 256, 32768), (1, 28672, 8192), (100, 19072, 320), (128, 28672, 512), (128, 512, 8192),
                                   (97, 2048, 16384)])
def test_few_token_gemm_vs_fp32_dequant_formula(ops, M, N, K):
    x, w, xq, wq, sx, sw, alpha, y = _gemm_case(ops, M, N, K, seed=11)
    y_ref = oracle.gemm_nvfp4_torch(xq, wq, sx, sw, alpha)
    scale = max(1.0, float(y_ref.float().std()))
    torch.testing.assert_close(y.float(), y_ref.float(), rtol=1.6e-2, atol=1e-2 * scale)
    assert _status() == 0


@pytest.mark.parametrize("M,N,K", [(5, 256, 16384), (40, 384, 32768), (5, 9600, 16384), (40, 9728, 16384)])
def test_few_token_gemm_split_and_unsplit_agree(ops, M, N, K):
    """With few 128-row weight blocks K is split inside thread-block clusters with or without workspace
    (first two shapes); with more than half as many blocks as SMs the entry point without workspace runs
    unsplit and the one with workspace splits K over independent CTAs.  All follow the same arithmetic up
    to the fp32 summation order."""
    from mslk_b200._lib import lib
    x, w, xq, wq, sx, sw, alpha, y_split = _gemm_case(ops, M, N, K, seed=13)
    assert lib.mslk_b200_f4f4bf16_workspace_bytes(M, N, K) > 0
    y_plain = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.mslk_b200_f4f4bf16(xq.data_ptr(), wq.data_ptr(), sx.data_ptr(), sw.data_ptr(), alpha.data_ptr(),
                                y_plain.data_ptr(), M, N, K, stream)
    assert rc == 0
    torch.cuda.synchronize()
    scale = max(1.0, float(y_plain.float().std()))
    torch.testing.assert_close(y_split.float(), y_plain.float(), rtol=8e-3, atol=4e-3 * scale)
    # repeated calls give identical bits (the partial tiles are summed in split order)
    y_again = ops.f4f4bf16(xq, wq, sx, sw, global_scale=alpha)
    assert torch.equal(y_again, y_split)
    assert _status() == 0


def test_few_token_gemm_workspace_size_contract():
    from mslk_b200._lib import lib
    assert lib.mslk_b200_f4f4bf16_workspace_bytes(1, 28672, 8192) == 0      # short K: unsplit
    assert lib.mslk_b200_f4f4bf16_workspace_bytes(256, 256, 32768) == 0     # more than 128 tokens: other kernels
    assert lib.mslk_b200_f4f4bf16_workspace_bytes(0, 256, 32768) == 0
    need = lib.mslk_b200_f4f4bf16_workspace_bytes(5, 256, 32768)
    assert need > 0 and need % 16 == 0


def test_quantizers_take_fp16_inputs_like_the_reference(ops):
    """fp16 inputs of quantize_nvfp4, calculate_group_max and nvfp4_quantize_stacked: bit-exact against the oracle and
    against outputs of the reference's Triton kernels captured on a B200."""
    import oracle
    from helpers import load_golden
    from golden.make_golden import NVFP4_F16_CASES, STACKED_F16_CASE, nvfp4_f16_inputs, unswizzle_stacked_scales
    gold = load_golden("nvfp4_f16_triton_b200.npz")
    for i, (name, shape) in enumerate(NVFP4_F16_CASES):
        x = nvfp4_f16_inputs(shape, 800 + i)
        gs = (448.0 * 6.0) / x.cuda().abs().amax().float()
        q, s = ops.quantize_nvfp4(x.cuda(), gs)
        q_ref, s_ref = oracle.quantize_nvfp4(x, gs.cpu())
        assert torch.equal(q.cpu().view(torch.uint8), q_ref), name
        assert torch.equal(s.cpu().view(torch.uint8), s_ref.view(torch.uint8)), name
        if gold is not None:
            assert torch.equal(gs.cpu().reshape(1), torch.from_numpy(gold[f"{name}.gs"])), name
            assert torch.equal(q.cpu().view(torch.uint8), torch.from_numpy(gold[f"{name}.q"])), name
            assert torch.equal(s.cpu().view(torch.uint8).reshape(-1), torch.from_numpy(gold[f"{name}.s_blocked"]).view(torch.uint8).reshape(-1)), name
    name, m_sizes, K = STACKED_F16_CASE
    x = nvfp4_f16_inputs((sum(m_sizes), K), 850).cuda()
    ms = torch.tensor(m_sizes, dtype=torch.int64, device="cuda")
    gs, idx = ops.calculate_group_max(x, ms)
    q, s = ops.nvfp4_quantize_stacked(ms, x, gs)
    q_ref, s_ref, _ = oracle.nvfp4_quantize_stacked(m_sizes, x.cpu(), gs.cpu())
    assert torch.equal(q.cpu().view(torch.uint8), q_ref)
    rows = unswizzle_stacked_scales(s, m_sizes, K)
    assert torch.equal(rows, unswizzle_stacked_scales(s_ref, m_sizes, K))
    if gold is not None:
        assert torch.equal(gs.cpu(), torch.from_numpy(gold[f"{name}.gs"]))
        assert torch.equal(idx.cpu(), torch.from_numpy(gold[f"{name}.idx"]))
        assert torch.equal(q.cpu().view(torch.uint8), torch.from_numpy(gold[f"{name}.q"]))
        assert torch.equal(rows, torch.from_numpy(gold[f"{name}.s_rows"]))
    from mslk_b200._lib import device_status
    assert device_status() == 0
