"""GPU parity tests of the rowwise-scaled FP8 GEMM (dense and grouped/stacked) through the C ABI.

Oracle: the reference tests' fp32 formula (dequantize, fp32 matmul, row x column scales),
test/gemm/triton/grouped_gemm_test.py:124-129.  Tolerance: rtol 1.6e-2 (same file, :138-150),
atol 1e-2 on unit-variance data.  Small cases are also checked against the scalar-C oracle.
"""
import pytest
import torch

import oracle
from helpers import randn_bf16

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


def _quant(ops, M, N, K, seed, w_std=0.02):
    x = randn_bf16((M, K), seed).cuda()
    w = randn_bf16((N, K), seed + 1, w_std).cuda()
    xq, xs = ops.quantize_fp8_row(x)
    wq, ws = ops.quantize_fp8_row(w)
    return xq, wq, xs, ws


def _close(y, y_ref, tag):
    assert y.shape == y_ref.shape and y.dtype == torch.bfloat16, tag
    # atol is stated for unit-variance data: scale it with the spread of the output
    scale = max(1.0, float(y_ref.float().std()))
    torch.testing.assert_close(y.float(), y_ref.float(), rtol=RTOL, atol=ATOL * scale, msg=lambda m: f"{tag}: {m}")


SMALL = [(1, 32, 128), (5, 33, 128), (7, 48, 144), (16, 64, 256), (128, 256, 256), (256, 128, 256),
         (129, 257, 512), (100, 8, 64), (3, 1, 32), (130, 520, 1040)]


@pytest.mark.parametrize("M,N,K", SMALL)
def test_small_shapes_vs_c_oracle(ops, M, N, K):
    xq, wq, xs, ws = _quant(ops, M, N, K, seed=M + N + K, w_std=1.0)
    y = ops.f8f8bf16_rowwise(xq, wq, xs, ws)
    y_c = oracle.gemm_f8_rowwise(xq.cpu(), wq.cpu(), xs.cpu(), ws.cpu())
    _close(y.cpu(), y_c, f"{M}x{N}x{K}")
    assert _status() == 0


LLAMA = [(M, N, K) for M in (1, 16, 128, 2048) for (N, K) in ((6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336))]


# (8192, 2048, 8192) and (6000, 1024, 16384): few column blocks, many row blocks -> the pair kernel orders its tiles in
# column bands (W resident in L2, X streamed); (5000, 5000, 2048): ragged edges under the tallest row band
@pytest.mark.parametrize("M,N,K", LLAMA + [(4096, 4096, 4096), (2048, 2048, 4096), (4096, 4096, 8192), (8192, 4096, 4096),
                                           (8192, 2048, 8192), (6000, 1024, 16384), (5000, 5008, 2048)])
def test_model_shapes_vs_fp32_formula(ops, M, N, K):
    xq, wq, xs, ws = _quant(ops, M, N, K, seed=1)
    y = ops.f8f8bf16_rowwise(xq, wq, xs, ws)
    y_ref = oracle.gemm_f8_rowwise_torch(xq, wq, xs, ws)
    _close(y, y_ref, f"{M}x{N}x{K}")
    assert _status() == 0


@pytest.mark.parametrize("bias_dtype", [torch.float32, torch.bfloat16])
def test_bias(ops, bias_dtype):
    M, N, K = 200, 384, 512
    xq, wq, xs, ws = _quant(ops, M, N, K, seed=9, w_std=1.0)
    bias = (torch.randn(N, device="cuda") * 10).to(bias_dtype)
    y = ops.f8f8bf16_rowwise(xq, wq, xs, ws, bias=bias)
    y_ref = oracle.gemm_f8_rowwise_torch(xq, wq, xs, ws, bias)
    _close(y, y_ref, f"bias {bias_dtype}")
    y_c = oracle.gemm_f8_rowwise(xq.cpu(), wq.cpu(), xs.cpu(), ws.cpu(), bias.cpu())
    _close(y.cpu(), y_c, f"bias {bias_dtype} vs C")


def test_3d_input_out_variant_and_fast_accum_flag(ops):
    B, T, N, K = 3, 50, 256, 256
    x = randn_bf16((B, T, K), 21).cuda()
    w = randn_bf16((N, K), 22).cuda()
    xq, xs = ops.quantize_fp8_row(x)
    wq, ws = ops.quantize_fp8_row(w)
    y = ops.f8f8bf16_rowwise(xq, wq, xs, ws, use_fast_accum=False)
    assert y.shape == (B, T, N)
    y_ref = oracle.gemm_f8_rowwise_torch(xq, wq, xs, ws)
    _close(y, y_ref, "3d")
    out = torch.full((B * T, N), 7.0, dtype=torch.bfloat16, device="cuda")
    ops.f8f8bf16_rowwise_out(xq, wq, xs, ws, out)
    assert torch.equal(out.view(B, T, N), y)


def test_empty_dims_and_errors(ops):
    xq, wq, xs, ws = _quant(ops, 4, 32, 64, seed=2)
    y = ops.f8f8bf16_rowwise(xq[:0], wq, xs[:0], ws)
    assert y.shape == (0, 32)
    # K == 0 gives zeros like the reference
    y = ops.f8f8bf16_rowwise(xq[:, :0].contiguous(), wq[:, :0].contiguous(), xs, ws)
    assert y.shape == (4, 32) and (y == 0).all()
    with pytest.raises(RuntimeError, match="float8_e4m3fn"):
        ops.f8f8bf16_rowwise(xq.view(torch.uint8), wq, xs, ws)
    with pytest.raises(RuntimeError, match="multiple of 16"):
        ops.f8f8bf16_rowwise(xq[:, :40].contiguous(), wq[:, :40].contiguous(), xs, ws)
    with pytest.raises(RuntimeError, match="float32"):
        ops.f8f8bf16_rowwise(xq, wq, xs.half(), ws)


def test_linearity_in_scales_full_size(ops):
    # size-independent property at a full benchmark size: doubling x_scale doubles y exactly (power of two),
    # and the result matches the fp32 formula on a sampled set of rows
    M, N, K = 8192, 8192, 8192
    xq, wq, xs, ws = _quant(ops, M, N, K, seed=4)
    y1 = ops.f8f8bf16_rowwise(xq, wq, xs, ws)
    y2 = ops.f8f8bf16_rowwise(xq, wq, xs * 2, ws)
    assert torch.equal(y2.float(), y1.float() * 2)
    rows = torch.arange(0, M, 61, device="cuda")
    y_ref = oracle.gemm_f8_rowwise_torch(xq[rows], wq, xs[rows], ws)
    _close(y1[rows], y_ref, "8192^3 sampled rows")
    assert _status() == 0


def _grouped_case(ops, G, m_sizes, N, K, seed):
    total = sum(m_sizes)
    x = randn_bf16((total, K), seed).cuda()
    w = randn_bf16((G, N, K), seed + 1, 0.02).cuda()
    xq, xs = ops.quantize_fp8_row(x)
    wq, ws = ops.quantize_fp8_row(w)
    ms = torch.tensor(m_sizes, dtype=torch.int64, device="cuda")
    y = ops.f8f8bf16_rowwise_grouped_stacked(xq, wq, xs, ws, ms)
    y_ref = oracle.gemm_f8_rowwise_grouped_stacked_torch(xq, wq, xs, ws, m_sizes)
    _close(y, y_ref, f"G={G} {m_sizes[:6]} N={N} K={K}")
    return xq, wq, xs, ws, ms, y


@pytest.mark.parametrize("G,m_sizes,N,K", [
    (1, [64], 512, 512),
    (4, [3, 0, 5, 1], 64, 128),
    (4, [128, 256, 0, 64], 512, 512),
    (16, [64 * ((i * 7) % 5) for i in range(16)], 1024, 512),
    (16, [0, 300, 0, 17, 129, 0, 1, 640, 128, 127, 0, 0, 255, 256, 257, 1000], 768, 640),
    (64, [((i * 37) % 9) * 16 for i in range(64)], 512, 1024),
])
def test_grouped_stacked(ops, G, m_sizes, N, K):
    xq, wq, xs, ws, ms, y = _grouped_case(ops, G, m_sizes, N, K, seed=G + N)
    # small cases also against the scalar-C oracle
    if sum(m_sizes) * N * K < 5e8:
        y_c = oracle.gemm_f8_rowwise_grouped_stacked(xq.cpu(), wq.cpu(), xs.cpu(), ws.cpu(), m_sizes)
        _close(y.cpu(), y_c, "grouped vs C")
    assert _status() == 0


def test_grouped_all_empty_and_rows_past_sum_untouched(ops):
    G, N, K = 4, 64, 128
    x = randn_bf16((10, K), 1).cuda()
    w = randn_bf16((G, N, K), 2).cuda()
    xq, xs = ops.quantize_fp8_row(x)
    wq, ws = ops.quantize_fp8_row(w)
    y = ops.f8f8bf16_rowwise_grouped_stacked(xq[:0], wq, xs[:0], ws, torch.zeros(G, dtype=torch.int64, device="cuda"))
    assert y.shape == (0, N)
    ms = torch.tensor([2, 0, 3, 0], dtype=torch.int64, device="cuda")
    y = ops.f8f8bf16_rowwise_grouped_stacked(xq, wq, xs, ws, ms)
    y_ref = oracle.gemm_f8_rowwise_grouped_stacked_torch(xq[:5], wq, xs[:5], ws, [2, 0, 3, 0])
    _close(y[:5], y_ref, "partial")
    with pytest.raises(RuntimeError, match="int64"):
        ops.f8f8bf16_rowwise_grouped_stacked(xq, wq, xs, ws, ms.int())
    assert _status() == 0


def test_grouped_moe_shape_zipf(ops):
    # the MoE configuration at reduced token count: 16 experts, Zipf(1.2) counts with empty experts
    E, N, K, tokens = 16, 2048, 5120, 4096
    g = torch.Generator().manual_seed(0)
    p = (torch.randperm(E, generator=g).float() + 1) ** -1.2
    counts = torch.bincount(torch.multinomial(p / p.sum(), tokens, replacement=True, generator=g), minlength=E)
    low = torch.argsort(p)[:2]
    counts[torch.argmax(counts)] += counts[low].sum()
    counts[low] = 0
    m_sizes = counts.tolist()
    assert sum(m_sizes) == tokens and m_sizes.count(0) >= 2
    _grouped_case(ops, E, m_sizes, N, K, seed=3)
    assert _status() == 0


@pytest.mark.parametrize("M", [1, 3, 16, 17, 32, 64, 100, 128])
@pytest.mark.parametrize("N,K", [(128, 128), (1000, 512), (4096, 4096), (6144, 1024)])
def test_few_token_shapes_split_and_unsplit(ops, M, N, K):
    # with scratch, M <= 32 takes the weight-streaming kernel with K split over independent CTAs (tickets);
    # without, the same kernel with the cluster split (N >= 2048) or the general kernel
    from mslk_b200._lib import lib, check
    xq, wq, xs, ws = _quant(ops, M, N, K, seed=M + N, w_std=1.0)
    bias = torch.randn(N, device="cuda") if (M + N) % 2 else None
    y_ref = oracle.gemm_f8_rowwise_torch(xq, wq, xs, ws, bias)
    st = torch.cuda.current_stream().cuda_stream
    bptr, bkind = (None, 0) if bias is None else (bias.data_ptr(), 1)

    def split_call():
        nbytes = lib.mslk_b200_f8f8bf16_rowwise_workspace_bytes(M, N, K)
        scratch = torch.empty((max(nbytes, 16),), dtype=torch.uint8, device="cuda")
        out = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
        check(lib.mslk_b200_f8f8bf16_rowwise_ws(xq.data_ptr(), wq.data_ptr(), xs.data_ptr(), ws.data_ptr(), bptr, bkind,
                                                out.data_ptr(), M, N, K, scratch.data_ptr(), nbytes, st), "ws")
        return out

    y = split_call()                                                # weight-streaming kernel, K split when useful
    _close(y, y_ref, f"decode split {M}x{N}x{K}")
    y2 = torch.empty_like(y)
    check(lib.mslk_b200_f8f8bf16_rowwise(xq.data_ptr(), wq.data_ptr(), xs.data_ptr(), ws.data_ptr(),
                                         None if bias is None else bias.data_ptr(), 0 if bias is None else 1,
                                         y2.data_ptr(), M, N, K, torch.cuda.current_stream().cuda_stream), "plain")
    _close(y2, y_ref, f"decode unsplit {M}x{N}x{K}")
    # the split result does not depend on CTA finishing order: repeated calls are bit-identical
    assert torch.equal(split_call(), y)
    assert _status() == 0


@pytest.mark.parametrize("M,N,K,bias_dtype", [
    (1, 2048, 16384, None), (20, 4096, 8576, torch.float32), (32, 2304, 4224, torch.bfloat16),
    (64, 4096, 8192, torch.bfloat16), (128, 2048, 16384, torch.float32), (5, 8192, 1024, None),
    (33, 6144, 8192, None), (16, 28672, 512, torch.float32)])
def test_few_token_shapes_cluster_split(ops, M, N, K, bias_dtype):
    """Without scratch the weight-streaming kernel splits K inside thread-block clusters (2, 4 or 8 CTAs whose
    partial tiles meet in distributed shared memory), also with a ragged last split, or runs unsplit (many
    weight blocks, short K); up to 128 tokens with long K.  Deterministic: repeated calls are bit-identical."""
    xq, wq, xs, ws = _quant(ops, M, N, K, seed=M + K, w_std=1.0)
    bias = None if bias_dtype is None else torch.randn(N, device="cuda").to(bias_dtype)
    y_ref = oracle.gemm_f8_rowwise_torch(xq, wq, xs, ws, bias)
    y = ops.f8f8bf16_rowwise(xq, wq, xs, ws, bias=bias)
    _close(y, y_ref, f"cluster split {M}x{N}x{K}")
    assert torch.equal(ops.f8f8bf16_rowwise(xq, wq, xs, ws, bias=bias), y)
    assert _status() == 0


def test_workspace_reuse_and_dirty_scratch(ops):
    from mslk_b200._lib import lib, check
    M, N, K = 8, 4096, 4096
    xq, wq, xs, ws = _quant(ops, M, N, K, seed=5)
    nbytes = lib.mslk_b200_f8f8bf16_rowwise_workspace_bytes(M, N, K)
    assert nbytes > 0
    scratch = torch.full((nbytes,), 0xAB, dtype=torch.uint8, device="cuda")   # deliberately dirty
    y_ref = oracle.gemm_f8_rowwise_torch(xq, wq, xs, ws)
    st = torch.cuda.current_stream().cuda_stream
    for _ in range(3):
        y = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
        check(lib.mslk_b200_f8f8bf16_rowwise_ws(xq.data_ptr(), wq.data_ptr(), xs.data_ptr(), ws.data_ptr(), None, 0,
                                                y.data_ptr(), M, N, K, scratch.data_ptr(), nbytes, st), "ws")
        _close(y, y_ref, "dirty scratch")
    assert _status() == 0


@pytest.mark.parametrize("M,N_local,K,world", [(300, 256, 512, 2), (4096, 2048, 1024, 4), (64, 520, 256, 3)])
def test_fused_allgather_placement_emulated_on_one_gpu(ops, M, N_local, K, world):
    # the ranks' output buffers are emulated by `world` buffers on this GPU; every "rank" writes its
    # column block into all of them, so each buffer must end up holding the unsharded result
    xq, wq, xs, ws = _quant(ops, M, N_local * world, K, seed=7)
    bias = torch.randn(N_local * world, device="cuda")
    y_ref = oracle.gemm_f8_rowwise_torch(xq, wq, xs, ws, bias)
    bufs = [torch.zeros((M, N_local * world), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    ptrs = [b.data_ptr() for b in bufs]
    for r in range(world):
        sl = slice(r * N_local, (r + 1) * N_local)
        ops.f8f8bf16_rowwise_allgather(xq, wq[sl].contiguous(), xs, ws[sl].contiguous(), ptrs, r, bufs[r],
                                       bias_shard=bias[sl].contiguous())
    for b in bufs:
        _close(b, y_ref, "fused all-gather placement")
    assert all(torch.equal(b, bufs[0]) for b in bufs)
    assert _status() == 0


@pytest.mark.parametrize("M,N,K,world", [(512, 256, 1024, 2), (1024, 1024, 2048, 4), (768, 320, 768, 3)])
def test_fused_reduce_scatter_emulated_on_one_gpu(ops, M, N, K, world):
    # K-sharded partial products are deposited by each "rank" into the owners' staging slots, then
    # every owner sums its slots: together the owners hold the unsharded result
    xq, wq, xs, ws = _quant(ops, M, N, K, seed=11)
    y_ref = oracle.gemm_f8_rowwise_torch(xq, wq, xs, ws)
    rows = M // world
    stages = [torch.full((world, rows, N), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    ptrs = [s.data_ptr() for s in stages]
    kl = K // world
    for r in range(world):
        ops.f8f8bf16_rowwise_scatter(xq[:, r * kl:(r + 1) * kl].contiguous(), wq[:, r * kl:(r + 1) * kl].contiguous(),
                                     xs, ws, ptrs, r)
    y = torch.cat([ops.reduce_slots(s) for s in stages], dim=0)
    _close(y, y_ref, "fused reduce-scatter")
    # slot contents are the individual partial products
    part0 = oracle.gemm_f8_rowwise_torch(xq[:, :kl].contiguous(), wq[:, :kl].contiguous(), xs, ws)
    _close(stages[1][0], part0[rows:2 * rows], "slot of rank 0 in owner 1")
    assert _status() == 0


# ------------------------------------------------------------------ batched (3D x 3D)

def _batched_case(ops, B, M, N, K, with_bias, seed):
    # test/gemm/gemm_test.py:507-597: x ~ U[0,1)*0.1, w ~ U[0,1)*0.01, fp32 bias [B, N]
    g = torch.Generator().manual_seed(seed)
    x = (torch.rand((B, M, K), generator=g) * 0.1).to(torch.bfloat16).cuda()
    w = (torch.rand((B, N, K), generator=g) * 0.01).to(torch.bfloat16).cuda()
    bias = torch.randn((B, N), generator=g).cuda() if with_bias else None
    xq, xs = ops.quantize_fp8_row(x)
    wq, ws = ops.quantize_fp8_row(w)
    assert xs.shape == (B, M) and ws.shape == (B, N)
    return x, w, bias, xq, wq, xs, ws


@pytest.mark.parametrize("B,M,N,K,with_bias", [
    (1, 256, 128, 256, False),     # the reference's cases
    (4, 4096, 256, 512, False),
    (4, 2048, 256, 512, True),
    (3, 100, 72, 144, True),       # ragged rows and columns: tiles straddle batch boundaries
    (5, 1, 40, 64, False),
    (2, 300, 1000, 640, True),
    (8, 512, 1024, 1024, False),   # tall enough for CTA pairs
    (16, 130, 8, 32, False),
])
def test_batched_equals_loop_over_dense(ops, B, M, N, K, with_bias):
    x, w, bias, xq, wq, xs, ws = _batched_case(ops, B, M, N, K, with_bias, seed=B * 1000 + M)
    y = ops.f8f8bf16_rowwise_batched(xq, wq, xs, ws, bias)
    assert y.shape == (B, M, N) and y.dtype == torch.bfloat16
    # the reference's tolerance against the unquantized bmm
    y_ref = torch.bmm(x.float(), w.float().transpose(1, 2))
    if bias is not None:
        y_ref += bias.unsqueeze(1)
    torch.testing.assert_close(y.float(), y_ref, atol=8.0e-2, rtol=8.0e-2)
    # the same quantized operands through the dense operator, batch by batch
    for b in range(B):
        y_b = ops.f8f8bf16_rowwise(xq[b], wq[b], xs[b], ws[b], None if bias is None else bias[b])
        _close(y[b], y_b, f"batch {b} vs dense operator")
        y_o = oracle.gemm_f8_rowwise_torch(xq[b].cpu(), wq[b].cpu(), xs[b].cpu(), ws[b].cpu(),
                                           None if bias is None else bias[b].cpu())
        _close(y[b].cpu(), y_o, f"batch {b} vs fp32 formula")
    assert _status() == 0


def test_batched_output_argument_empty_dims_and_errors(ops):
    x, w, bias, xq, wq, xs, ws = _batched_case(ops, 2, 64, 128, 128, False, seed=1)
    import mslk_b200.gemm  # noqa: F401  registers torch.ops.mslk.*
    out = torch.full((2, 64, 128), 7.0, dtype=torch.bfloat16, device="cuda")
    y = torch.ops.mslk.f8f8bf16_rowwise_batched(xq, wq, xs, ws, None, True, out)
    assert y.data_ptr() == out.data_ptr()
    assert torch.equal(out, ops.f8f8bf16_rowwise_batched(xq, wq, xs, ws))
    assert ops.f8f8bf16_rowwise_batched(xq[:, :0], wq, xs[:, :0], ws).shape == (2, 0, 128)
    z = ops.f8f8bf16_rowwise_batched(xq[:, :, :0].contiguous(), wq[:, :, :0].contiguous(), xs, ws)
    assert z.shape == (2, 64, 128) and float(z.float().abs().max()) == 0.0
    with pytest.raises(RuntimeError, match="3D"):
        ops.f8f8bf16_rowwise_batched(xq[0], wq, xs, ws)
    with pytest.raises(RuntimeError, match="fast_accum"):
        torch.ops.mslk.f8f8bf16_rowwise_batched(xq, wq, xs, ws, None, False)
    with pytest.raises(RuntimeError, match="float32"):
        ops.f8f8bf16_rowwise_batched(xq, wq, xs, ws, torch.zeros((2, 128), dtype=torch.bfloat16, device="cuda"))
    assert _status() == 0


# ------------------------------------------------------------------ grouped GEMM + fused scatter-add (MoE combine)

@pytest.mark.parametrize("G,m_sizes,N,K,topk", [
    (4, [128, 256, 0, 64], 512, 512, 1),
    (16, [0, 300, 0, 17, 129, 0, 1, 640, 128, 127, 0, 0, 255, 256, 257, 1000], 768, 640, 1),
    (8, [64] * 8, 256, 1024, 2),
    (4, [3, 0, 5, 1], 72, 128, 1),           # narrow, element-wise atomics for the ragged column tail
    (16, [256] * 16, 1024, 512, 4),
    (16, [512] * 16, 2048, 512, 1),          # enough 256 x 256 tiles for CTA pairs (swapped roles, vector reductions)
    (12, [300, 700, 0, 256, 1, 511, 512, 513, 40, 1000, 64, 900], 2304, 256, 2),
])
def test_grouped_scatter_add_epilogue(ops, G, m_sizes, N, K, topk):
    # mslk/gemm/triton/grouped_gemm.py:386-402: product row r is added to output[indices[r]]
    xq, wq, xs, ws, ms, y_plain = _grouped_case(ops, G, m_sizes, N, K, seed=G + N + topk)
    total = sum(m_sizes)
    T = max(total // topk, 1)
    g = torch.Generator().manual_seed(total)
    idx = (torch.randperm(total, generator=g) % T).to(torch.int32).cuda()
    out0 = (torch.randn((T, N), generator=g) * 0.5).to(torch.bfloat16).cuda()
    out = out0.clone()
    ret = ops.f8f8bf16_rowwise_grouped_stacked_scatter_add(xq, wq, xs, ws.view(-1), ms, out, idx)
    assert ret.data_ptr() == out.data_ptr()
    if topk == 1:
        # every output row receives at most one product row: one bf16 addition, exactly reproducible
        want = out0.clone()
        want[idx.long()] = (out0[idx.long()].float() + y_plain[:total].float()).to(torch.bfloat16)
        assert torch.equal(out, want)
    else:
        want = out0.float().index_add_(0, idx.long(), y_plain[:total].float())
        scale = max(1.0, float(want.std()))
        torch.testing.assert_close(out.float(), want, rtol=1.6e-2, atol=2e-2 * scale)
    # the reference's Python entry point, int64 indices
    import mslk_b200.gemm.triton.grouped_gemm as gg
    out2 = out0.clone()
    gg.grouped_gemm_fp8_rowwise(xq, wq.view(G * N, K), ms.int(), xs, ws.view(-1), _output_tensor=out2,
                                _scatter_add_indices=idx.long())
    if topk == 1:
        assert torch.equal(out2, out)
    assert torch.equal(gg.grouped_gemm_fp8_rowwise(xq, wq.view(G * N, K), ms.int(), xs, ws.view(-1))[:total], y_plain[:total])
    assert _status() == 0


def test_scatter_add_bad_index_reported(ops):
    xq, wq, xs, ws, ms, _ = _grouped_case(ops, 2, [16, 16], 128, 128, seed=1)
    idx = torch.arange(32, dtype=torch.int32, device="cuda")
    idx[5] = 1000
    out = torch.zeros((32, 128), dtype=torch.bfloat16, device="cuda")
    ops.f8f8bf16_rowwise_grouped_stacked_scatter_add(xq, wq, xs, ws.view(-1), ms, out, idx)
    assert _status() == 0x200
    assert float(out[5].float().abs().max()) == 0.0 and float(out[6].float().abs().max()) > 0.0
