"""GPU parity tests of the MXFP4 path through the C ABI: the e8m0 quantizer (bit-exact against the oracle and against
outputs of the reference's Triton kernel captured on a B200) and the MXFP4 forms of f4f4bf16, f4f4bf16_grouped_stacked
and f4f4bf16_grouped_mm (the reference's cases, test/gemm/gemm_test.py:2591-2790,2791-2822; exact dequantize-matmul
formula with the 1-ulp bound, and the reference's own tolerance against the unquantized product)."""
import pytest
import torch

import oracle
from helpers import assert_sharp_bf16, load_golden
from golden.make_golden import (MX4_CASES, MX4_NEAREST_CASES, MX4_SEEDS, MX4_STACKED_STOCHASTIC_CASES, MX4_STOCHASTIC_CASES,
                                mx4_inputs)

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
            if name in MX4_NEAREST_CASES and f"{name}.g{group}.m0.q" in gold:
                # nearest: floor(log2(max) + 0.5) through the GPU's log2f -- the same instruction sequence on both sides
                q, s = ops.quantize_mx4(x, group, 0)
                key = f"{name}.g{group}.m0"
                assert torch.equal(q.cpu(), torch.from_numpy(gold[key + ".q"])), key
                assert torch.equal(s.cpu().view(torch.uint8), torch.from_numpy(gold[key + ".s"]).reshape(-1)), key
                # the C restatement uses libm's log2f: equal except where a maximum sits on a rounding boundary
                q_or, s_or = oracle.quantize_mx4(x.cpu(), group, 0)
                assert float((s.cpu().view(torch.uint8) != s_or).float().mean()) < 1e-3, key
    assert _status() == 0


@pytest.mark.parametrize("group", [32, 16])
def test_stochastic_rounding_bit_exact_vs_oracle(ops, group):
    """Rounding mode 3 (the reference's tl.randint streams, mslk/quantize/triton/fp4_primitives/scale.py:213-261): same
    seed, same bytes as the C restatement -- integer work on both sides -- including zero groups, whose perturbed bit
    patterns turn into NaNs that the conversion saturates."""
    for i, (name, shape, dtype) in enumerate(MX4_CASES):
        x = mx4_inputs(name, shape, dtype, 700 + i)
        for seed in MX4_SEEDS + (0, 7):
            q_ref, s_ref = oracle.quantize_mx4(x, group, 3, seed=seed)
            q, s = ops.quantize_mx4(x.cuda(), group, 3, seed=seed)
            assert torch.equal(s.cpu().view(torch.uint8), s_ref), (name, group, seed)
            assert torch.equal(q.cpu(), q_ref), (name, group, seed)
    assert _status() == 0


def test_stochastic_rounding_matches_reference_triton_fixture(ops):
    gold = load_golden("mx4_triton_b200.npz")
    if gold is None or not any(".m3." in k for k in gold.keys()):
        pytest.skip("fixture of the stochastic mode captured from the reference's Triton kernel not present")
    for i, (name, shape, dtype) in enumerate(MX4_CASES):
        if name not in MX4_STOCHASTIC_CASES:
            continue
        x = mx4_inputs(name, shape, dtype, 700 + i).cuda()
        for group in (32, 16):
            for seed in MX4_SEEDS:
                key = f"{name}.g{group}.m3.seed{seed}"
                q, s = ops.quantize_mx4(x, group, 3, seed=seed)
                assert torch.equal(s.cpu().view(torch.uint8), torch.from_numpy(gold[key + ".s"]).reshape(-1)), key
                assert torch.equal(q.cpu(), torch.from_numpy(gold[key + ".q"])), key
    for name, m_sizes, K in MX4_STACKED_STOCHASTIC_CASES:
        x = mx4_inputs(name, (sum(m_sizes), K), "bf16", 900 + K).cuda()
        ms = torch.tensor(m_sizes, dtype=torch.int64, device="cuda")
        q, s = ops.quantize_mx4_stacked(ms, x, 32, 3, seed=MX4_SEEDS[0])
        assert torch.equal(s.cpu().view(torch.uint8), torch.from_numpy(gold[f"{name}.m3.s"]).reshape(-1)), name
        assert torch.equal(q.cpu(), torch.from_numpy(gold[f"{name}.m3.q"])), name
    assert _status() == 0


def test_stochastic_rounding_properties(ops):
    """What the reference's tests ask of the mode (test/quantize/triton/test_quantize_mx4.py:118-145,168-213): a seed
    replays, another seed differs, a zero group keeps scale byte 0, +inf saturates the scale at 252; and the point of it:
    averaged over seeds the dequantized values approach x more closely than one round-to-nearest pass does."""
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn((64, 128), generator=g, device="cuda").bfloat16()
    q0, s0 = ops.quantize_mx4(x, 32, 3, seed=0x12345678)
    q1, s1 = ops.quantize_mx4(x, 32, 3, seed=0x12345678)
    q2, _ = ops.quantize_mx4(x, 32, 3, seed=0x12345679)
    assert torch.equal(q0, q1) and torch.equal(s0, s1) and not torch.equal(q0, q2)
    torch.manual_seed(99)
    qa, sa = ops.quantize_mx4(x, 32, 3)                                        # the CUDA generator's initial seed
    qb, sb = ops.quantize_mx4(x, 32, 3, seed=torch.cuda.default_generators[0].initial_seed())
    assert torch.equal(qa, qb) and torch.equal(sa, sb)
    z = torch.zeros((1, 32), device="cuda", dtype=torch.bfloat16)
    _, sz = ops.quantize_mx4(z, 32, 3, seed=0x12345678)
    assert int(sz.view(torch.uint8)[0]) == 0
    xi = x.clone()
    xi[0, 0] = float("inf")
    _, si = ops.quantize_mx4(xi, 32, 3, seed=0x12345678)
    assert int(si.view(torch.uint8)[0]) == 252

    # unbiasedness of the element rounding: every group's maximum is 3.0 (mantissa 0.5, which the group stream's 22 random
    # bits cannot carry into the exponent), so every scale is 2^-1 and x / scale lies in (4.1, 6): between two e2m1 values
    from oracle import fp4_to_float
    xs = (torch.rand((32, 64), generator=g, device="cuda") * 0.9 + 2.05).bfloat16()
    xs[:, ::32] = 3.0
    acc = torch.zeros(xs.shape, device="cuda")
    n = 64
    for seed in range(n):
        q, s = ops.quantize_mx4(xs, 32, 3, seed=seed)
        sc = s.view(torch.uint8)[:512].reshape(32, 16)[:, :2]    # one 128 x 4 atom: row r < 32, column c at r * 16 + c
        assert bool((sc == 126).all())
        acc += fp4_to_float(q).to(acc.device) * 0.5
    err_sr = (acc / n - xs.float()).abs().mean()
    qn, sn = ops.quantize_mx4(xs, 32, 1)
    err_rn = (fp4_to_float(qn).to(acc.device) * 0.5 - xs.float()).abs().mean()
    assert float(err_sr) < 0.5 * float(err_rn), (float(err_sr), float(err_rn), n)
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
        ops.quantize_mx4(x, 32, 5)
    with pytest.raises(AssertionError):
        ops.quantize_mx4(x[..., :48], 32, 4)


def _mx_case(ops, M, N, K, group, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = (torch.randn((M, K), generator=g, device="cuda") * 0.1).bfloat16()
    w = (torch.randn((N, K), generator=g, device="cuda") * 0.01).bfloat16()
    xq, sx = ops.quantize_mx4(x, group)
    wq, sw = ops.quantize_mx4(w, group)
    return x, w, xq, wq, sx, sw


@pytest.mark.parametrize("M,N,K", [(2321, 2608, 1312), (2560, 2816, 544), (3100, 2304, 256)])
@pytest.mark.parametrize("fmt", ["mx32", "mx16", "nvfp4"])
def test_pair_kernel_ragged_shapes_both_accumulators(ops, M, N, K, fmt):
    """More than 74 tiles of 256 x 256, so CTA pairs take the problem and every pair runs several tiles, alternating
    between its two overlapping accumulators: ragged last row block, a last column block that ends inside a 64-column
    slab, a partial last K block, a single K block (the next tile's first instruction follows the hand-back at once)."""
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    x = (torch.randn((M, K), generator=g, device="cuda") * 0.1).bfloat16()
    w = (torch.randn((N, K), generator=g, device="cuda") * 0.01).bfloat16()
    if fmt == "nvfp4":
        gx, gw = 2688.0 / x.abs().amax().float(), 2688.0 / w.abs().amax().float()
        xq, sx = ops.quantize_nvfp4(x, gx)
        wq, sw = ops.quantize_nvfp4(w, gw)
        alpha = (1.0 / (gx * gw)).reshape(1)
        y = ops.f4f4bf16(xq, wq, sx, sw, global_scale=alpha)
        y_ref = oracle.gemm_nvfp4_torch(xq, wq, sx, sw, alpha)
    else:
        group = 32 if fmt == "mx32" else 16
        xq, sx = ops.quantize_mx4(x, group)
        wq, sw = ops.quantize_mx4(w, group)
        y = ops.f4f4bf16(xq, wq, sx, sw, mxfp4_block_size=group)
        y_ref = oracle.gemm_mx4_torch(xq, wq, sx, sw, group)
    assert_sharp_bf16(y, y_ref, f"pair kernel {fmt} {M}x{N}x{K}")
    assert _status() == 0


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


@pytest.mark.parametrize("M,N,K", [(1, 28672, 8192), (32, 28672, 8192), (16, 4096, 14336), (64, 8192, 8192), (7, 6144, 4096),
                                   (100, 8192, 28672), (3, 384, 1056)])
@pytest.mark.parametrize("group", [32, 16])
def test_gemm_mxfp4_few_tokens(ops, M, N, K, group):
    """Few-token shapes: the weight-streaming kernel (K split inside clusters on the long-K shapes) in both MX modes."""
    x, w, xq, wq, sx, sw = _mx_case(ops, M, N, K, group, seed=M + N)
    y = ops.f4f4bf16(xq, wq, sx, sw, mxfp4_block_size=group)
    y_ref = oracle.gemm_mx4_torch(xq, wq, sx, sw, group)
    assert_sharp_bf16(y, y_ref, f"f4f4bf16 MXFP4 few tokens, group {group} {M}x{N}x{K}")
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


# --------------------------------------------------------------------------- K-grouped ("2D-2D") form

def _kgrouped_case(ops, M, N, k_sizes, nvfp4, seed):
    """X [M, total_K], W [N, total_K] quantized group by group along K (every group its own swizzled scale block),
    packed bytes concatenated along K, scale blocks concatenated flat."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    xqs, wqs, xss, wss, gss, xs, ws = [], [], [], [], [], [], []
    for kg in k_sizes:
        x = (torch.randn((M, kg), generator=g, device="cuda") * 0.1).bfloat16()
        w = (torch.randn((N, kg), generator=g, device="cuda") * 0.01).bfloat16()
        xs.append(x)
        ws.append(w)
        if kg == 0:
            xqs.append(torch.empty((M, 0), dtype=torch.uint8, device="cuda"))
            wqs.append(torch.empty((N, 0), dtype=torch.uint8, device="cuda"))
            xss.append(torch.empty((0,), dtype=torch.uint8, device="cuda"))
            wss.append(torch.empty((0,), dtype=torch.uint8, device="cuda"))
            gss.append(torch.ones((), device="cuda"))
            continue
        if nvfp4:
            gx = (448.0 * 6.0) / x.abs().amax().float()
            gw = (448.0 * 6.0) / w.abs().amax().float()
            q, s = ops.quantize_nvfp4(x, gx)
            xqs.append(q.view(torch.uint8))
            xss.append(s.view(torch.uint8).reshape(-1))
            q, s = ops.quantize_nvfp4(w, gw)
            wqs.append(q.view(torch.uint8))
            wss.append(s.view(torch.uint8).reshape(-1))
            gss.append(1.0 / (gx * gw))
        else:
            q, s = ops.quantize_mx4(x, 32)
            xqs.append(q.view(torch.uint8))
            xss.append(s.view(torch.uint8).reshape(-1))
            q, s = ops.quantize_mx4(w, 32)
            wqs.append(q.view(torch.uint8))
            wss.append(s.view(torch.uint8).reshape(-1))
    return xs, ws, xqs, wqs, xss, wss, gss


@pytest.mark.parametrize("nvfp4", [False, True])
@pytest.mark.parametrize("M,N,k_sizes", [(256, 256, [2048]), (500, 1024, [2048] * 4), (200, 384, [256, 0, 800, 992, 32]),
                                         (1000, 2048, [3584] * 3), (64, 136, [96, 4096]),
                                         (600, 1536, [256, 0, 800, 992, 32, 4096]), (2048, 2048, [2048, 0, 6144, 992, 8192])])
def test_grouped_mm_2d2d(ops, M, N, k_sizes, nvfp4):
    """f4f4bf16_grouped_mm with 2D XQ and 2D WQ (test/gemm/gemm_test.py:2731-2790): groups along K, out [G, M, N];
    ragged and empty groups beside the reference's equal ones."""
    xs, ws, xqs, wqs, xss, wss, gss = _kgrouped_case(ops, M, N, k_sizes, nvfp4, seed=M + N + len(k_sizes))
    xq = torch.cat(xqs, dim=1).contiguous()
    wq = torch.cat(wqs, dim=1).contiguous()
    sdt = torch.float8_e4m3fn if nvfp4 else getattr(torch, "float8_e8m0fnu", None)
    if sdt is None:
        pytest.skip("this torch has no float8_e8m0fnu")
    x_scale = torch.cat(xss).view(sdt)
    w_scale = torch.cat(wss).view(sdt)
    offsets = torch.tensor(k_sizes, device="cuda").cumsum(0).to(torch.int32)
    gs = torch.stack([torch.as_tensor(v, device="cuda").float().reshape(()) for v in gss]) if nvfp4 else None
    out = ops.f4f4bf16_grouped_mm(xq, wq.transpose(-2, -1), x_scale, w_scale, offsets, None, gs)
    assert out.shape == (len(k_sizes), M, N)
    for g, kg in enumerate(k_sizes):
        if kg == 0:
            assert torch.count_nonzero(out[g]) == 0
            continue
        if nvfp4:
            y_ref = oracle.gemm_nvfp4_torch(xqs[g], wqs[g], xss[g].view(torch.float8_e4m3fn), wss[g].view(torch.float8_e4m3fn),
                                            gss[g].reshape(1))
        else:
            y_ref = oracle.gemm_mx4_torch(xqs[g], wqs[g], xss[g], wss[g], 32)
        assert_sharp_bf16(out[g], y_ref, f"2D-2D group {g} of {k_sizes} nvfp4={nvfp4}")
        # the reference's bound against the UNQUANTIZED product holds up to its largest K (3584); the quantization noise
        # of a sum grows with sqrt(K), so longer groups get that factor
        tol = 8.0e-2 * max(1.0, (kg / 3584.0) ** 0.5)
        torch.testing.assert_close(out[g], (xs[g] @ ws[g].T).to(torch.bfloat16), atol=tol, rtol=tol)
    assert _status() == 0


def test_grouped_mm_2d2d_through_the_operator_and_rejections(ops):
    from mslk_b200 import compat
    compat.install()
    import mslk.gemm  # noqa: F401
    e8 = getattr(torch, "float8_e8m0fnu", None)
    if e8 is None:
        pytest.skip("this torch has no float8_e8m0fnu")
    M, N, K, G = 256, 256, 2048, 2
    xs, ws, xqs, wqs, xss, wss, _ = _kgrouped_case(ops, M, N, [K] * G, False, seed=9)
    xq = torch.cat(xqs, dim=1).contiguous()
    wq = torch.cat(wqs, dim=1).contiguous()
    x_scale, w_scale = torch.cat(xss).view(e8), torch.cat(wss).view(e8)
    offsets = torch.arange(K, G * (K + 1), K, dtype=torch.int32, device="cuda")
    f4 = getattr(torch, "float4_e2m1fn_x2", None)
    a, b = (xq.view(f4), wq.view(f4)) if f4 is not None else (xq, wq)
    out = torch.ops.mslk.f4f4bf16_grouped_mm(a, b.transpose(-2, -1), x_scale, w_scale, offsets)
    X, W = torch.cat(xs, dim=1), torch.cat(ws, dim=1)
    for g in range(G):
        ref = X[:, g * K:(g + 1) * K] @ W[:, g * K:(g + 1) * K].T
        torch.testing.assert_close(out[g], ref, atol=8.0e-2, rtol=8.0e-2)
    assert _status() == 0
    # an offset that is no multiple of 32: that group's product is zero and the status word says why
    bad = torch.tensor([K + 16, 2 * K], dtype=torch.int32, device="cuda")
    out = ops.f4f4bf16_grouped_mm(xq, wq.transpose(-2, -1), x_scale, w_scale, bad)
    assert torch.count_nonzero(out) == 0          # group 0 ends and group 1 starts off the 32-element grid
    assert _status() & 0x400                      # reading the status word clears it
    assert _status() == 0


# --------------------------------------------------------------------------- stacked quantizer

@pytest.mark.parametrize("m_sizes,K,group", [([64, 64], 64, 32), ([50, 30, 48], 64, 32), ([16, 64, 128, 256], 128, 32),
                                             ([256, 512], 512, 32), ([50, 30, 48], 64, 16), ([64, 0, 64], 64, 32),
                                             ([16] * 64, 128, 32), ([128, 128], 80, 16), ([1, 1, 1, 1], 64, 16),
                                             ([5, 11, 19], 64, 16), ([300, 0, 1000, 129, 2047, 620], 1024, 32)])
def test_quantize_mx4_stacked_equals_per_segment(ops, m_sizes, K, group):
    """The reference's cases (test/quantize/triton/test_stacked_quantize_mx4.py:56-160): packed bytes equal the
    per-segment quantizer's, every segment's swizzled scale block sits at its 128-row-aligned offset, and every other
    byte of the scale buffer is zero."""
    M, G = sum(m_sizes), len(m_sizes)
    g = torch.Generator().manual_seed(M + K)
    x = (torch.randn((M, K), generator=g) * torch.exp2(torch.randint(-8, 8, (M, 1), generator=g).float())).bfloat16()
    ms = torch.tensor(m_sizes, dtype=torch.int64, device="cuda")
    q, s = ops.quantize_mx4_stacked(ms, x.cuda(), group)
    pc = (K // group + 3) // 4 * 4
    assert q.shape == (M, K // 2) and s.numel() == (M + 127 * G) * pc
    want = torch.zeros_like(s, device="cpu").view(torch.uint8)
    r = pad = 0
    for m in m_sizes:
        if m:
            q_ref, s_ref = oracle.quantize_mx4(x[r:r + m], group, 4)
            assert torch.equal(q[r:r + m].cpu(), q_ref), (m_sizes, r)
            want[pad * pc:pad * pc + s_ref.numel()] = s_ref.reshape(-1)
        r += m
        pad += (m + 127) // 128 * 128
    assert torch.equal(s.cpu().view(torch.uint8), want)
    assert _status() == 0


@pytest.mark.parametrize("m_sizes,K,group", [([50, 30, 48], 64, 32), ([130, 0, 7], 256, 32), ([5, 11, 19], 64, 16),
                                             ([300, 0, 1000, 129], 512, 32)])
def test_quantize_mx4_stacked_stochastic(ops, m_sizes, K, group):
    """Stochastic mode on stacked segments: the random streams are indexed by the row of the padded scale matrix
    (mslk/quantize/triton/fp4_primitives/scale.py:200-201), so segment g equals the oracle run on its rows with the
    stream rows shifted to the segment's 128-row-aligned start."""
    M, G = sum(m_sizes), len(m_sizes)
    g = torch.Generator().manual_seed(M + K)
    x = (torch.randn((M, K), generator=g) * torch.exp2(torch.randint(-8, 8, (M, 1), generator=g).float())).bfloat16()
    ms = torch.tensor(m_sizes, dtype=torch.int64, device="cuda")
    seed = 0x12345678
    q, s = ops.quantize_mx4_stacked(ms, x.cuda(), group, 3, seed=seed)
    pc = (K // group + 3) // 4 * 4
    want = torch.zeros_like(s, device="cpu").view(torch.uint8)
    r = pad = 0
    for m in m_sizes:
        if m:
            rows = torch.arange(pad, pad + m, dtype=torch.int32)
            q_ref, s_ref = oracle.quantize_mx4(x[r:r + m], group, 3, seed=seed, stream_rows=rows)
            assert torch.equal(q[r:r + m].cpu(), q_ref), (m_sizes, r)
            want[pad * pc:pad * pc + s_ref.numel()] = s_ref.reshape(-1)
        r += m
        pad += (m + 127) // 128 * 128
    assert torch.equal(s.cpu().view(torch.uint8), want)
    assert _status() == 0


def test_quantize_mx4_stacked_feeds_the_grouped_gemm(ops):
    from mslk_b200 import compat
    compat.install()
    from mslk.quantize.triton.quantize_kernels.mx4_stacked import quantize_mx4_stacked
    from mslk.quantize.triton.fp4_quantize import RoundingMode, triton_quantize_mx4_unpack
    m_sizes, N, K = [300, 0, 77, 1024], 512, 2048
    xs = [torch.randn((m, K), device="cuda").bfloat16() * 0.1 for m in m_sizes]
    ws = [torch.randn((N, K), device="cuda").bfloat16() * 0.01 for _ in m_sizes]
    ms = torch.tensor(m_sizes, dtype=torch.int64, device="cuda")
    xq, x_scale = quantize_mx4_stacked(ms, torch.cat(xs), rounding_mode=RoundingMode.ceil)
    wq, w_scale = zip(*[triton_quantize_mx4_unpack(w) for w in ws])
    y = ops.f4f4bf16_grouped_stacked(xq, torch.stack(wq), x_scale, torch.stack(w_scale), ms)
    r = 0
    for g, m in enumerate(m_sizes):
        if m:
            torch.testing.assert_close(y[r:r + m], (xs[g] @ ws[g].T).to(torch.bfloat16), atol=8.0e-2, rtol=8.0e-2)
        r += m
    assert _status() == 0


# --------------------------------------------------------------------------- edge cases of the MXFP4 entry points

def test_mxfp4_edge_cases(ops):
    e8 = getattr(torch, "float8_e8m0fnu", None)
    # one row, one group
    x = torch.randn((1, 32), device="cuda").bfloat16()
    q, s = ops.quantize_mx4(x)
    q_ref, s_ref = oracle.quantize_mx4(x.cpu(), 32, 4)
    assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu().view(torch.uint8), s_ref)
    # no rows at all: nothing to do, shapes right
    q0, s0 = ops.quantize_mx4(torch.empty((0, 64), device="cuda", dtype=torch.bfloat16))
    assert q0.shape == (0, 32) and s0.numel() == 0
    w = torch.randn((128, 64), device="cuda").bfloat16()
    wq, ws = ops.quantize_mx4(w)
    y0 = ops.f4f4bf16(q0, wq, s0, ws)
    assert y0.shape == (0, 128)
    # stacked quantizer with only empty segments: the scale buffer is all padding, all zero
    ms = torch.zeros(3, dtype=torch.int64, device="cuda")
    qs, ss = ops.quantize_mx4_stacked(ms, torch.empty((0, 128), device="cuda", dtype=torch.bfloat16))
    assert qs.shape == (0, 64) and ss.numel() == 3 * 127 * 4 and torch.count_nonzero(ss) == 0
    # grouped GEMM whose groups are all empty
    wq3, ws3 = ops.quantize_mx4(torch.randn((3, 128, 128), device="cuda").bfloat16())
    yg = ops.f4f4bf16_grouped_stacked(qs, wq3, ss, ws3.view(3, -1), ms)
    assert yg.shape == (0, 128)
    if e8 is not None:
        # K-grouped form with one tiny group and few rows
        xs, ws_, xqs, wqs, xss, wss, _ = _kgrouped_case(ops, 5, 16, [64], False, seed=1)
        offs = torch.tensor([64], dtype=torch.int32, device="cuda")
        out = ops.f4f4bf16_grouped_mm(xqs[0], wqs[0].transpose(-2, -1), xss[0].view(e8), wss[0].view(e8), offs)
        assert out.shape == (1, 5, 16)
        assert_sharp_bf16(out[0], oracle.gemm_mx4_torch(xqs[0], wqs[0], xss[0], wss[0], 32), "2D-2D 5x16x64")
        # offsets past the end of K: that group is rejected on the device, no out-of-bounds read
        bad = torch.tensor([128], dtype=torch.int32, device="cuda")
        out = ops.f4f4bf16_grouped_mm(xqs[0], wqs[0].transpose(-2, -1), xss[0].view(e8), wss[0].view(e8), bad)
        assert _status() & 0x400
    assert _status() == 0


@pytest.mark.parametrize("M,N,G", [(300, 272, 300), (512, 512, 200)])
def test_grouped_mm_2d2d_many_small_groups(ops, M, N, G):
    """Hundreds of K groups of 0..256 elements: the one-CTA kernel above 255 groups, CTA pairs below."""
    e8 = getattr(torch, "float8_e8m0fnu", None)
    if e8 is None:
        pytest.skip("this torch has no float8_e8m0fnu")
    g = torch.Generator().manual_seed(G)
    k_sizes = (torch.randint(0, 9, (G,), generator=g) * 32).tolist()
    xs, ws, xqs, wqs, xss, wss, _ = _kgrouped_case(ops, M, N, k_sizes, False, seed=G)
    xq, wq = torch.cat(xqs, dim=1).contiguous(), torch.cat(wqs, dim=1).contiguous()
    offs = torch.tensor(k_sizes, device="cuda").cumsum(0).to(torch.int32)
    out = ops.f4f4bf16_grouped_mm(xq, wq.transpose(-2, -1), torch.cat(xss).view(e8), torch.cat(wss).view(e8), offs)
    assert out.shape == (G, M, N)
    for i, kg in enumerate(k_sizes):
        if kg == 0:
            assert torch.count_nonzero(out[i]) == 0, i
        else:
            y_ref = oracle.gemm_mx4_torch(xqs[i], wqs[i], xss[i], wss[i], 32)
            assert torch.equal(out[i], y_ref.to(out.dtype)) or (out[i].float() - y_ref.float()).abs().max() <= 2 ** -7 * y_ref.float().abs().max(), i
    assert _status() == 0
