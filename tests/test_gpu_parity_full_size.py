"""GPU parity at the FULL sizes of the benchmark configurations, every output element checked.

Each case is compared with the reference tests' fp32 formula (dequantize, fp32 matmul on the GPU with TF32
off, scales; test/gemm/triton/grouped_gemm_test.py:112-150, test/gemm/gemm_test.py:725-856, :2374-2396) twice:
with the reference's tolerance (rtol 1.6e-2, atol 1e-2 on unit-variance data, scaled with the output spread)
and with the sharp bound of helpers.assert_sharp_bf16 (>= 99.9 % of the elements within one bf16 step, none
beyond two).  Shapes:
  * the four Llama-3-8B projections at M = 8192 and 8192^3 (what bench.py times),
  * the MoE configuration at full size: 16 experts, 16384 tokens, Zipf(1.2) counts with empty experts,
    (N, K) = (16384, 5120) and (5120, 8192),
  * the Llama-3-70B FFN shards at M = 8192 for 1/2/4/8 ranks: (57344/P, 8192) and (8192, 28672/P), plus the fused
    all-gather / reduce-scatter placements emulated on one GPU at those sizes,
  * NVFP4 8192^3 and M = 32 x (28672, 8192); grouped NVFP4 with Zipf counts against the per-group oracle.
"""
import pytest
import torch

import oracle
from helpers import assert_sharp_bf16, fp8_rowwise_formula_chunked, randn_bf16

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1.6e-2, 1e-2


@pytest.fixture(scope="module")
def ops():
    from mslk_b200 import ops as _ops
    torch.backends.cuda.matmul.allow_tf32 = False
    return _ops


def _status():
    from mslk_b200._lib import device_status
    return device_status()


def _randn(shape, seed, std=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda", dtype=torch.float32) * std).to(torch.bfloat16)


def _both_bounds(y, y_ref, tag):
    scale = max(1.0, float(y_ref.float().std()))
    torch.testing.assert_close(y.float(), y_ref.float(), rtol=RTOL, atol=ATOL * scale, msg=lambda m: f"{tag}: {m}")
    return assert_sharp_bf16(y, y_ref, tag)


@pytest.mark.parametrize("M,N,K", [(8192, 6144, 4096), (8192, 4096, 4096), (8192, 28672, 4096), (8192, 4096, 14336),
                                   (8192, 8192, 8192), (4096, 4096, 4096),
                                   (16384, 8192, 8192)])   # two column bands of 18 + 14 blocks (W resident, X streamed)
def test_dense_bench_shapes_every_element(ops, M, N, K):
    xq, xs = ops.quantize_fp8_row(_randn((M, K), 1))
    wq, ws = ops.quantize_fp8_row(_randn((N, K), 2, 0.02))
    y = ops.f8f8bf16_rowwise(xq, wq, xs, ws)
    _both_bounds(y, fp8_rowwise_formula_chunked(xq, wq, xs, ws), f"f8f8bf16_rowwise {M}x{N}x{K}")
    assert _status() == 0


@pytest.mark.parametrize("M,N,K", [(2048, 4096, 4096), (128, 28672, 4096), (16, 4096, 14336), (1, 6144, 4096)])
def test_dense_smaller_token_counts_sharp(ops, M, N, K):
    xq, xs = ops.quantize_fp8_row(_randn((M, K), 3))
    wq, ws = ops.quantize_fp8_row(_randn((N, K), 4, 0.02))
    y = ops.f8f8bf16_rowwise(xq, wq, xs, ws)
    _both_bounds(y, fp8_rowwise_formula_chunked(xq, wq, xs, ws), f"f8f8bf16_rowwise {M}x{N}x{K}")
    assert _status() == 0


@pytest.mark.parametrize("N,K", [(16384, 5120), (5120, 8192)])
def test_moe_full_size_zipf(ops, N, K):
    from microbench import zipf_counts
    E, tokens = 16, 16384
    counts = zipf_counts(E, tokens).tolist()
    assert sum(counts) == tokens and counts.count(0) >= 2
    xq, xs = ops.quantize_fp8_row(_randn((tokens, K), 5))
    wq, ws = ops.quantize_fp8_row(_randn((E, N, K), 6, 0.02))
    ms = torch.tensor(counts, dtype=torch.int64, device="cuda")
    y = ops.f8f8bf16_rowwise_grouped_stacked(xq, wq, xs, ws.view(-1), ms)
    y_ref = torch.empty_like(y)
    r = 0
    for g, m in enumerate(counts):
        if m:
            y_ref[r:r + m] = fp8_rowwise_formula_chunked(xq[r:r + m], wq[g], xs[r:r + m], ws[g])
        r += m
    _both_bounds(y, y_ref, f"grouped_stacked E=16 tokens=16384 N={N} K={K}")
    assert _status() == 0


@pytest.mark.parametrize("P", [1, 2, 4, 8])
def test_ffn70b_shard_shapes(ops, P):
    M = 8192
    # gate+up: rank 0's N shard of (57344, 8192)
    n_local = 57344 // P
    xq, xs = ops.quantize_fp8_row(_randn((M, 8192), 7))
    wq, ws = ops.quantize_fp8_row(_randn((n_local, 8192), 8, 0.01))
    y = ops.f8f8bf16_rowwise(xq, wq, xs, ws)
    _both_bounds(y, fp8_rowwise_formula_chunked(xq, wq, xs, ws), f"70B gate+up shard P={P}: {M}x{n_local}x8192")
    del xq, wq, y
    # down: rank 0's K shard of (8192, 28672); scales are those of the FULL rows
    K = 28672
    xq, xs = ops.quantize_fp8_row(_randn((M, K), 9))
    wq, ws = ops.quantize_fp8_row(_randn((8192, K), 10, 0.01))
    kl = K // P
    xq_k, wq_k = xq[:, :kl].contiguous(), wq[:, :kl].contiguous()
    y = ops.f8f8bf16_rowwise(xq_k, wq_k, xs, ws)
    _both_bounds(y, fp8_rowwise_formula_chunked(xq_k, wq_k, xs, ws), f"70B down shard P={P}: {M}x8192x{kl}")
    assert _status() == 0


@pytest.mark.parametrize("P", [2, 8])
def test_ffn70b_fused_collective_placements_emulated(ops, P):
    """The fused all-gather / reduce-scatter epilogues at the full shard sizes, the P ranks emulated by P buffers
    on this GPU (each 'rank' is one launch; nothing waits on another launch)."""
    M, N, K = 8192, 57344, 8192
    n_local = N // P
    xq, xs = ops.quantize_fp8_row(_randn((M, K), 11))
    wq, ws = ops.quantize_fp8_row(_randn((N, K), 12, 0.01))
    y_ref = fp8_rowwise_formula_chunked(xq, wq, xs, ws)
    bufs = [torch.zeros((M, N), dtype=torch.bfloat16, device="cuda") for _ in range(P)]
    ptrs = [b.data_ptr() for b in bufs]
    for r in range(P):
        sl = slice(r * n_local, (r + 1) * n_local)
        ops.f8f8bf16_rowwise_allgather(xq, wq[sl].contiguous(), xs, ws[sl].contiguous(), ptrs, r, bufs[r])
    _both_bounds(bufs[0], y_ref, f"fused all-gather placement P={P}")
    assert all(torch.equal(b, bufs[0]) for b in bufs[1:])
    del bufs, y_ref, wq
    N, K = 8192, 28672
    xq, xs = ops.quantize_fp8_row(_randn((M, K), 13))
    wq, ws = ops.quantize_fp8_row(_randn((N, K), 14, 0.01))
    y_ref = fp8_rowwise_formula_chunked(xq, wq, xs, ws)
    rows, kl = M // P, K // P
    stages = [torch.full((P, rows, N), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(P)]
    sptrs = [s.data_ptr() for s in stages]
    for r in range(P):
        ops.f8f8bf16_rowwise_scatter(xq[:, r * kl:(r + 1) * kl].contiguous(), wq[:, r * kl:(r + 1) * kl].contiguous(),
                                     xs, ws, sptrs, r)
    y = torch.cat([ops.reduce_slots(s) for s in stages], dim=0)
    # The P partial products are rounded to bf16 before the owner sums them in fp32 in rank order (NCCL's bf16
    # reduce-scatter rounds as often): against the unsharded fp32 formula an element may be off by one bf16 step
    # of its LARGEST partial product, which near a cancellation is more than the 1e-2 absolute bound, so that
    # bound is doubled here ...
    scale = max(1.0, float(y_ref.float().std()))
    torch.testing.assert_close(y.float(), y_ref.float(), rtol=RTOL, atol=2 * ATOL * scale)
    # ... and the sharp statement is made against exactly that arithmetic, emulated from the formula's own partial
    # products: |y - sum_r bf16(partial_r)| <= one bf16 step of the largest partial + one of the sum.
    parts = torch.stack([fp8_rowwise_formula_chunked(xq[:, r * kl:(r + 1) * kl].contiguous(),
                                                     wq[:, r * kl:(r + 1) * kl].contiguous(), xs, ws) for r in range(P)])
    emul = parts.float().sum(0)
    tol = (parts.float().abs().amax(0) + emul.abs()) * 2.0 ** -7
    err = (y.float() - emul).abs()
    worst = float((err - tol).max())
    frac_equal = float((y == emul.to(torch.bfloat16)).float().mean())
    print({"case": f"fused reduce-scatter P={P} vs fp32 sum of bf16 partials", "frac_equal": frac_equal,
           "max_err_over_bound": float((err / tol.clamp_min(1e-30)).max())})
    assert worst <= 0, f"an element is {worst} beyond one bf16 step of its largest partial product"
    assert frac_equal > 0.995
    assert _status() == 0


def _nvfp4_case(ops, M, N, K, seed):
    x, w = _randn((M, K), seed), _randn((N, K), seed + 1)
    gx = (448.0 * 6.0) / x.abs().amax().float()
    gw = (448.0 * 6.0) / w.abs().amax().float()
    xq, sx = ops.quantize_nvfp4(x, gx)
    wq, sw = ops.quantize_nvfp4(w, gw)
    alpha = (1.0 / (gx * gw)).reshape(1)
    return xq, wq, sx, sw, alpha


def _nvfp4_formula_chunked(xq, wq, sx, sw, alpha, rows_per_chunk=1024):
    """fp32 dequantize-matmul formula (mslk/quantize/triton/legacy/fp4_utils.py:95-120) in row chunks on the GPU."""
    M, K = xq.shape[0], xq.shape[1] * 2
    N = wq.shape[0]
    s_x = oracle.from_blocked(sx.view(torch.uint8).cpu().reshape(-1), M, K // 16).view(torch.float8_e4m3fn).cuda()
    s_w = oracle.from_blocked(sw.view(torch.uint8).cpu().reshape(-1), N, K // 16).view(torch.float8_e4m3fn).cuda()
    wf = oracle.fp4_to_float(wq) * s_w.float().repeat_interleave(16, dim=1)
    out = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    for r in range(0, M, rows_per_chunk):
        xf = oracle.fp4_to_float(xq[r:r + rows_per_chunk]) * s_x[r:r + rows_per_chunk].float().repeat_interleave(16, dim=1)
        out[r:r + rows_per_chunk] = ((xf @ wf.T) * alpha.reshape(()).float()).to(torch.bfloat16)
    return out


@pytest.mark.parametrize("M,N,K", [(8192, 8192, 8192), (32, 28672, 8192), (1, 28672, 8192), (2048, 8192, 8192)])
def test_nvfp4_bench_shapes_every_element(ops, M, N, K):
    xq, wq, sx, sw, alpha = _nvfp4_case(ops, M, N, K, seed=15)
    y = ops.f4f4bf16(xq, wq, sx, sw, global_scale=alpha)
    _both_bounds(y, _nvfp4_formula_chunked(xq, wq, sx, sw, alpha), f"f4f4bf16 {M}x{N}x{K}")
    assert _status() == 0


def test_grouped_nvfp4_zipf_against_per_group_oracle(ops):
    """Grouped NVFP4 with Zipf counts and empty experts against the per-group dequantize-matmul oracle
    (a whole wrong scale block would pass a norm bound against the unquantized product, not this)."""
    from microbench import zipf_counts
    from test_gpu_nvfp4_grouped import _grouped_problem
    m_sizes = zipf_counts(16, 4096).tolist()
    N, K = 1024, 2048
    X, W, ms, xq, wq, x_scale, w_scale, alpha = _grouped_problem(ops, m_sizes, N, K, seed=3)
    y = ops.f4f4bf16_grouped_stacked(xq, wq, x_scale, w_scale, ms, alpha, None, use_mx=False)
    y_or = oracle.gemm_nvfp4_grouped_stacked(xq.view(torch.uint8).cpu(), wq.view(torch.uint8).cpu(), x_scale.cpu(),
                                             w_scale.cpu(), m_sizes, alpha.cpu())
    total = sum(m_sizes)
    _both_bounds(y[:total].cpu(), y_or[:total], "f4f4bf16_grouped_stacked Zipf E=16 tokens=4096 N=1024 K=2048")
    assert _status() == 0


def _mx4_formula_chunked(xq, wq, sx, sw, group, rows_per_chunk=1024):
    """fp32 dequantize-matmul formula of the MXFP4 GEMM (e8m0 scales per `group` elements) in row chunks on the GPU."""
    M, K = xq.shape[0], xq.shape[1] * 2
    N = wq.shape[0]
    e_x = oracle.from_blocked(sx.view(torch.uint8).cpu().reshape(-1), M, K // group).to(torch.int32).cuda()
    e_w = oracle.from_blocked(sw.view(torch.uint8).cpu().reshape(-1), N, K // group).to(torch.int32).cuda()
    wf = oracle.fp4_to_float(wq) * torch.ldexp(torch.ones(e_w.shape, dtype=torch.float32, device="cuda"), e_w - 127).repeat_interleave(group, dim=1)
    out = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    for r in range(0, M, rows_per_chunk):
        xf = oracle.fp4_to_float(xq[r:r + rows_per_chunk]) * torch.ldexp(torch.ones(e_x[r:r + rows_per_chunk].shape, dtype=torch.float32, device="cuda"), e_x[r:r + rows_per_chunk] - 127).repeat_interleave(group, dim=1)
        out[r:r + rows_per_chunk] = (xf @ wf.T).to(torch.bfloat16)
    return out


@pytest.mark.parametrize("M,N,K,group", [(8192, 8192, 8192, 32), (8192, 8192, 8192, 16), (32, 28672, 8192, 32),
                                         (1, 28672, 8192, 16), (2048, 8192, 8192, 32)])
def test_mxfp4_bench_shapes_every_element(ops, M, N, K, group):
    """The MXFP4 modes at the sizes the bench times: CTA pairs with the two-instruction scale atoms, the few-token
    weight-streaming kernel, both block sizes; every element against the exact formula."""
    x, w = _randn((M, K), 21) * 0.1, _randn((N, K), 22) * 0.01
    xq, sx = ops.quantize_mx4(x, group)
    wq, sw = ops.quantize_mx4(w, group)
    y = ops.f4f4bf16(xq, wq, sx, sw, mxfp4_block_size=group)
    _both_bounds(y, _mx4_formula_chunked(xq, wq, sx, sw, group), f"f4f4bf16 MXFP4/{group} {M}x{N}x{K}")
    assert _status() == 0
