"""CPU tests: the oracle against fixtures produced by running the reference
(tests/golden/make_golden.py) and against torch's own conversions."""
import ctypes

import numpy as np
import pytest
import torch

import oracle
from helpers import bf16, fp8, load_golden, u8, randn_bf16
from golden.make_golden import (FP8_ROW_CASES, MX4_CASES, MX4_SEEDS, MX4_STACKED_STOCHASTIC_CASES, MX4_STOCHASTIC_CASES,
                                NVFP4_CASES, mx4_inputs)


def test_e4m3_encode_matches_torch_exhaustive_grid():
    # every e4m3 value, every midpoint between neighbours, and +-1 ulp(fp32) around both
    codes = torch.arange(0, 127, dtype=torch.uint8)
    vals = codes.view(torch.float8_e4m3fn).float()
    mids = (vals[:-1] + vals[1:]) / 2
    pts = torch.cat([vals, mids])
    pts = torch.cat([pts, torch.nextafter(pts, torch.tensor(1e9)), torch.nextafter(pts, torch.tensor(-1e9))])
    pts = torch.cat([pts, -pts])
    want = pts.to(torch.float8_e4m3fn).view(torch.uint8)
    L = oracle.lib()
    got = torch.tensor([L.oracle_f32_to_e4m3(ctypes.c_float(v)) for v in pts.tolist()], dtype=torch.uint8)
    assert torch.equal(got, want)
    # decode
    dec = torch.tensor([L.oracle_e4m3_to_f32(int(c)) for c in codes.tolist()])
    assert torch.equal(dec, vals)


def test_e4m3_saturates_finite():
    L = oracle.lib()
    for v, c in [(448.0, 0x7E), (463.9, 0x7E), (464.0, 0x7E), (1e30, 0x7E), (-1e30, 0xFE), (float("inf"), 0x7E)]:
        assert L.oracle_f32_to_e4m3(ctypes.c_float(v)) == c


def test_e2m1_rne_ties_to_even():
    L = oracle.lib()
    table = {0.0: 0, 0.25: 0, 0.26: 1, 0.5: 1, 0.75: 2, 1.0: 2, 1.25: 2, 1.5: 3, 1.75: 4, 2.0: 4,
             2.5: 4, 2.51: 5, 3.0: 5, 3.5: 6, 4.0: 6, 5.0: 6, 5.01: 7, 6.0: 7, 100.0: 7}
    for v, c in table.items():
        assert L.oracle_f32_to_e2m1(ctypes.c_float(v)) == c, v
        if v:
            assert L.oracle_f32_to_e2m1(ctypes.c_float(-v)) == (c | 8), v


def test_bf16_round_matches_torch():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(20000, generator=g) * 100
    x = torch.cat([x, torch.tensor([1.00390625, 1.01171875, 3.3895e38, 0.0, -0.0])])
    L = oracle.lib()
    got = torch.tensor([L.oracle_f32_to_bf16(ctypes.c_float(v)) for v in x.tolist()], dtype=torch.int32)
    want = x.to(torch.bfloat16).view(torch.int16).to(torch.int32) & 0xFFFF
    assert torch.equal(got, want)


def test_cpu_path_quantize_matches_reference_fixture():
    gold = load_golden("fp8_row_cpu_path.npz")
    assert gold is not None
    names = sorted({k.split(".")[0] for k in gold.files})
    assert len(names) >= 8
    for name in names:
        a = bf16(gold[f"{name}.a"])
        ub = torch.from_numpy(gold[f"{name}.ub"]) if f"{name}.ub" in gold.files else None
        q, s = oracle.quantize_fp8_row_cpu_path(a, ub)
        assert torch.equal(u8(q), torch.from_numpy(gold[f"{name}.q"])), name
        assert torch.equal(s.view(torch.int32), torch.from_numpy(gold[f"{name}.s"]).view(torch.int32)), name
        # and the torch statement used for CPU-baseline timing is the same arithmetic
        q2, s2 = oracle.quantize_fp8_row_cpu_path_torch(a, ub)
        assert torch.equal(u8(q2), u8(q)), name
        assert torch.equal(s2, s), name


def test_gpu_arithmetic_quantize_matches_torch_statement():
    # The C statement of the Triton arithmetic against the same formula written in torch
    # (fp32 IEEE division twice, clamp, RNE cast).
    for i, (name, shape, kw) in enumerate(FP8_ROW_CASES):
        if kw.get("jagged") or "permute" in kw:
            continue
        a = randn_bf16(shape, i, kw.get("scale", 1.0))
        ub = torch.tensor([kw["scale_ub"]]) if "scale_ub" in kw else None
        q, s = oracle.quantize_fp8_row(a, ub, None, kw.get("align_rows_to"))
        amax = a.abs().amax(dim=-1).float()
        cur = torch.clamp(amax, min=1.0 / 512.0)
        if ub is not None:
            cur = torch.clamp(cur, max=ub.item())
        sc = cur / 448.0
        qq = torch.clamp(a.float() / sc[..., None], -448, 448).to(torch.float8_e4m3fn)
        K = shape[-1]
        assert torch.equal(s, sc), name
        assert torch.equal(u8(q)[..., :K], u8(qq)), name
        assert (u8(q)[..., K:] == 0).all(), name


def test_triton_fixture_pins_gpu_arithmetic():
    gold = load_golden("fp8_row_triton_b200.npz")
    if gold is None:
        pytest.skip("fixture captured on a B200 not present yet")
    for i, (name, shape, kw) in enumerate(FP8_ROW_CASES):
        a = bf16(gold[f"{name}.a"])
        ub = torch.from_numpy(gold[f"{name}.ub"]) if f"{name}.ub" in gold.files else None
        zs = torch.from_numpy(gold[f"{name}.zs"]) if f"{name}.zs" in gold.files else None
        q, s = oracle.quantize_fp8_row(a, ub, zs, kw.get("align_rows_to"))
        assert torch.equal(s.reshape(-1).view(torch.int32),
                           torch.from_numpy(gold[f"{name}.s"]).reshape(-1).view(torch.int32)), name
        assert torch.equal(u8(q).reshape(-1), torch.from_numpy(gold[f"{name}.q"]).reshape(-1)), name


def test_gemm_oracles_agree_and_match_reference_cpu_fallback():
    gold = load_golden("fp8_gemm_cpu_path.npz")
    for name in sorted({k.split(".")[0] for k in gold.files}):
        xq, wq = fp8(gold[f"{name}.xq"]), fp8(gold[f"{name}.wq"])
        xs, ws = torch.from_numpy(gold[f"{name}.xs"]), torch.from_numpy(gold[f"{name}.ws"])
        y_ref = bf16(gold[f"{name}.y"])
        y_c = oracle.gemm_f8_rowwise(xq, wq, xs, ws)
        y_t = oracle.gemm_f8_rowwise_torch(xq, wq, xs, ws)
        # C (sequential fp32) vs torch (blocked fp32): same up to fp32 summation order
        torch.testing.assert_close(y_c.float(), y_t.float(), rtol=1.6e-2, atol=1e-2)
        # the reference's CPU fallback does a bf16 matmul: tolerance of its own tests
        torch.testing.assert_close(y_c.float(), y_ref.float(), rtol=1.6e-2, atol=3.5e-2)


def test_gemm_oracle_bias_kinds():
    x = randn_bf16((7, 64), 1)
    w = randn_bf16((9, 64), 2)
    xq, xs = oracle.quantize_fp8_row(x)
    wq, ws = oracle.quantize_fp8_row(w)
    for bias in (torch.randn(9), torch.randn(9).bfloat16()):
        y_c = oracle.gemm_f8_rowwise(xq, wq, xs, ws, bias)
        y_t = oracle.gemm_f8_rowwise_torch(xq, wq, xs, ws, bias)
        torch.testing.assert_close(y_c.float(), y_t.float(), rtol=1.6e-2, atol=1e-2)


def test_grouped_oracles_agree():
    ms = [3, 0, 5, 1]
    x = randn_bf16((sum(ms), 64), 3)
    w = randn_bf16((4, 6, 64), 4)
    xq, xs = oracle.quantize_fp8_row(x)
    wq, ws = oracle.quantize_fp8_row(w)
    y_c = oracle.gemm_f8_rowwise_grouped_stacked(xq, wq, xs, ws, ms)
    y_t = oracle.gemm_f8_rowwise_grouped_stacked_torch(xq, wq, xs, ws, ms)
    torch.testing.assert_close(y_c.float(), y_t.float(), rtol=1.6e-2, atol=1e-2)


def test_nvfp4_quantize_matches_reference_torch_fixture():
    gold = load_golden("nvfp4_torch_ref.npz")
    assert gold is not None
    for name, shape in NVFP4_CASES:
        x = bf16(gold[f"{name}.x"])
        gs = torch.from_numpy(gold[f"{name}.gs"])
        assert torch.equal(oracle.global_scale_nvfp4(x).reshape(1), gs), name
        q, s = oracle.quantize_nvfp4(x, gs)
        want_s = torch.from_numpy(gold[f"{name}.s_blocked"]).reshape(-1)
        assert torch.equal(u8(s).reshape(-1), want_s), name
        assert torch.equal(q, torch.from_numpy(gold[f"{name}.q"])), name
        # layout helpers
        s_plain = fp8(gold[f"{name}.s"])
        assert torch.equal(oracle.to_blocked(u8(s_plain)), want_s), name
        assert torch.equal(oracle.from_blocked(want_s, *s_plain.shape), u8(s_plain)), name


def test_nvfp4_triton_fixture():
    gold = load_golden("nvfp4_triton_b200.npz")
    if gold is None:
        pytest.skip("fixture captured on a B200 not present yet")
    for name, shape in NVFP4_CASES:
        x = bf16(gold[f"{name}.x"])
        gs = torch.from_numpy(gold[f"{name}.gs"])
        q, s = oracle.quantize_nvfp4(x, gs)
        assert torch.equal(u8(s).reshape(-1), torch.from_numpy(gold[f"{name}.s_blocked"]).reshape(-1)), name
        assert torch.equal(q, torch.from_numpy(gold[f"{name}.q"])), name


def test_nvfp4_f16_triton_fixture():
    """fp16 inputs: the reference's Triton quantizers (dense and stacked, with the per-group global scales) against the
    oracle, bit for bit except the approximate division of the group scales (a couple of ulps)."""
    from golden.make_golden import NVFP4_F16_CASES, STACKED_F16_CASE, nvfp4_f16_inputs, unswizzle_stacked_scales
    gold = load_golden("nvfp4_f16_triton_b200.npz")
    if gold is None:
        pytest.skip("fixture captured on a B200 not present yet")
    for i, (name, shape) in enumerate(NVFP4_F16_CASES):
        x = nvfp4_f16_inputs(shape, 800 + i)
        gs = torch.from_numpy(gold[f"{name}.gs"])
        q, s = oracle.quantize_nvfp4(x, gs)
        assert torch.equal(q, torch.from_numpy(gold[f"{name}.q"])), name
        assert torch.equal(u8(s).reshape(-1), torch.from_numpy(gold[f"{name}.s_blocked"]).view(torch.uint8).reshape(-1)), name
    name, m_sizes, K = STACKED_F16_CASE
    x = nvfp4_f16_inputs((sum(m_sizes), K), 850)
    gs = torch.from_numpy(gold[f"{name}.gs"])
    gs_or, idx_or = oracle.calculate_group_max(x, m_sizes)
    live = torch.tensor([m > 0 for m in m_sizes])
    assert torch.allclose(gs_or[live], gs[live], rtol=4e-7, atol=0.0)
    assert torch.equal(idx_or, torch.from_numpy(gold[f"{name}.idx"]))
    q, s, _ = oracle.nvfp4_quantize_stacked(m_sizes, x, gs)
    assert torch.equal(q, torch.from_numpy(gold[f"{name}.q"]))
    assert torch.equal(unswizzle_stacked_scales(s, m_sizes, K), torch.from_numpy(gold[f"{name}.s_rows"]))


def test_mx4_triton_fixture_pins_the_mx4_oracle():
    """Outputs of the reference's triton_quantize_mx4_unpack on a B200 (packed bytes and swizzled e8m0 scales, block
    sizes 32 and 16, floor / even / ceil rounding of the shared exponent) against the C restatement, bit for bit."""
    gold = load_golden("mx4_triton_b200.npz")
    if gold is None:
        pytest.skip("fixture captured on a B200 not present yet")
    for i, (name, shape, dtype) in enumerate(MX4_CASES):
        x = mx4_inputs(name, shape, dtype, 700 + i)
        for group in (32, 16):
            for mode in (4, 1, 2):
                q, s = oracle.quantize_mx4(x, group, mode)
                key = f"{name}.g{group}.m{mode}"
                assert torch.equal(q, torch.from_numpy(gold[key + ".q"])), key
                assert torch.equal(s.reshape(-1), torch.from_numpy(gold[key + ".s"]).reshape(-1)), key
            key = f"{name}.g{group}.m0"
            if key + ".s" in gold:
                # nearest: floor(log2(max) + 0.5); libm's log2f against the GPU's can move a maximum that sits on a
                # rounding boundary into the next binade, nothing else may differ
                q, s = oracle.quantize_mx4(x, group, 0)
                diff = s.reshape(-1) != torch.from_numpy(gold[key + ".s"]).reshape(-1)
                assert float(diff.float().mean()) < 1e-3, key


def test_mx4_stochastic_fixture_pins_the_oracle():
    """Rounding mode 3 of the reference's kernel captured on a B200 with fixed seeds (dense and stacked) against the C
    restatement with its own Philox, bit for bit."""
    gold = load_golden("mx4_triton_b200.npz")
    if gold is None or not any(".m3." in k for k in gold.keys()):
        pytest.skip("fixture of the stochastic mode not present")
    for i, (name, shape, dtype) in enumerate(MX4_CASES):
        if name not in MX4_STOCHASTIC_CASES:
            continue
        x = mx4_inputs(name, shape, dtype, 700 + i)
        for group in (32, 16):
            for seed in MX4_SEEDS:
                key = f"{name}.g{group}.m3.seed{seed}"
                q, s = oracle.quantize_mx4(x, group, 3, seed=seed)
                assert torch.equal(s.reshape(-1), torch.from_numpy(gold[key + ".s"]).reshape(-1)), key
                assert torch.equal(q, torch.from_numpy(gold[key + ".q"])), key
    for name, m_sizes, K in MX4_STACKED_STOCHASTIC_CASES:
        x = mx4_inputs(name, (sum(m_sizes), K), "bf16", 900 + K)
        gq, gs = torch.from_numpy(gold[f"{name}.m3.q"]), torch.from_numpy(gold[f"{name}.m3.s"]).reshape(-1)
        pc = (K // 32 + 3) // 4 * 4
        r = pad = 0
        for m in m_sizes:
            if m:
                rows = torch.arange(pad, pad + m, dtype=torch.int32)
                q, s = oracle.quantize_mx4(x[r:r + m], 32, 3, seed=MX4_SEEDS[0], stream_rows=rows)
                assert torch.equal(q, gq[r:r + m]), (name, r)
                assert torch.equal(s.reshape(-1), gs[pad * pc:pad * pc + s.numel()]), (name, r)
            r += m
            pad += (m + 127) // 128 * 128


# First output word of Philox-4x32 with 7 rounds for (seed, offset), computed with Triton's own tl.randint in its
# interpreter mode (no GPU needed); the test below recomputes them when Triton is importable.
PHILOX7_KNOWN = [(1234, 0xFFFFFFF9, 0xCCFEFD1A), (0x12345678, 0xFFFFFFF9, 0x89980EC0),
                 (0x7FFFFFFFFFFFFFF1, 0xFFFFFFF9, 0x018C5499)]

_PHILOX_SCRIPT = """
import os
os.environ["TRITON_INTERPRET"] = "1"
import torch, triton, triton.language as tl

@triton.jit
def k(out_ptr, seed, n: tl.constexpr):
    offs = tl.arange(0, n) * 1000003 - 7
    tl.store(out_ptr + tl.arange(0, n), tl.randint(seed, offs, n_rounds=7))

out = torch.zeros(16, dtype=torch.int32)
for seed in (1234, 0x12345678, 0x7FFFFFFFFFFFFFF1):
    k[(1,)](out, seed, 16)
    print(" ".join(str(int(v) & 0xFFFFFFFF) for v in out.tolist()))
"""


def test_philox_restatement_known_answers_and_triton_interpreter():
    import subprocess
    import sys
    L = oracle.lib()
    for seed, off, want in PHILOX7_KNOWN:
        assert L.oracle_philox7_first_word(seed, off) == want
    try:
        import triton  # noqa: F401
    except ImportError:
        return
    res = subprocess.run([sys.executable, "-c", _PHILOX_SCRIPT], capture_output=True, text=True, timeout=300)
    if res.returncode != 0:
        pytest.skip("Triton's interpreter mode did not run here: " + res.stderr[-200:])
    lines = res.stdout.strip().splitlines()[-3:]
    for seed, line in zip((1234, 0x12345678, 0x7FFFFFFFFFFFFFF1), lines):
        got = [int(v) for v in line.split()]
        mine = [L.oracle_philox7_first_word(seed, (i * 1000003 - 7) & 0xFFFFFFFF) for i in range(16)]
        assert got == mine, seed


def test_mx4_oracle_against_a_plain_statement():
    """Independent of the fixture: ceil rounding picks the smallest power of two 2^e with amax <= 6 * 2^e ... up to the
    reference's shift by two binades (e = ceil(log2(amax)) - 2), values are x * 2^-e rounded to e2m1 (ties to even)."""
    g = torch.Generator().manual_seed(5)
    x = (torch.randn((64, 256), generator=g) * torch.exp2(torch.randint(-20, 20, (64, 1), generator=g).float())).bfloat16()
    q, s = oracle.quantize_mx4(x, 32, 4)
    xf = x.float().reshape(64, 8, 32)
    amax = xf.abs().amax(dim=-1)
    e = torch.ceil(torch.log2(amax.double())).to(torch.int32) - 2
    e = e.clamp(-127, 125)
    # the scale bytes sit in 128-row x 4-column swizzled atoms: row r, column c -> (r % 32) * 16 + (r // 32) * 4 + c
    s = s.reshape(-1)
    for r in range(64):
        for c in range(8):
            atom = c // 4
            off = atom * 512 + (r % 32) * 16 + (r // 32) * 4 + (c % 4)
            assert int(s[off]) == int(e[r, c]) + 127, (r, c)
    grid = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
    scaled = (xf.double() * torch.exp2(-e.double()).unsqueeze(-1)).float().reshape(64, 256)
    lo = (q & 0xF).long()
    hi = (q >> 4).long()
    codes = torch.stack([lo, hi], dim=-1).reshape(64, 256)
    val = grid[codes & 7] * torch.where((codes & 8) != 0, -1.0, 1.0)
    # nearest grid point (ties checked by the e2m1 test above): no other grid value is strictly closer
    d = (scaled.unsqueeze(-1).abs().clamp(max=6.0) - grid).abs()
    assert torch.all((val.abs() - scaled.abs().clamp(max=6.0)).abs() <= d.min(dim=-1).values + 1e-7)


def test_nvfp4_gemm_oracles_agree_and_dequant_matches_reference():
    gold = load_golden("nvfp4_torch_ref.npz")
    name = "n128x64"
    x = bf16(gold[f"{name}.x"])
    gs = torch.from_numpy(gold[f"{name}.gs"])
    q, s = oracle.quantize_nvfp4(x, gs)
    # dequantize(x) as the reference does it equals fp4*scale/gs
    true_scale = oracle.from_blocked(u8(s).reshape(-1), 128, 4).view(torch.float8_e4m3fn).float() / gs
    deq = (oracle.fp4_to_float(q) * true_scale.repeat_interleave(16, 1)).to(torch.bfloat16)
    # value comparison: the reference's lookup table holds +0 for code 8 (-0)
    assert torch.equal(deq.float(), bf16(gold[f"{name}.deq"]).float())
    w = randn_bf16((48, 64), 9)
    gw = oracle.global_scale_nvfp4(w)
    wq, sw = oracle.quantize_nvfp4(w, gw)
    alpha = 1.0 / (gs * gw)
    y_c = oracle.gemm_nvfp4(q, wq, s, sw, alpha)
    y_t = oracle.gemm_nvfp4_torch(q, wq, s, sw, alpha)
    torch.testing.assert_close(y_c.float(), y_t.float(), rtol=1.6e-2, atol=1e-2)
    # sanity against the unquantized product: 4-bit error, so only a norm bound
    y_full = x.float() @ w.float().T
    assert (y_t.float() - y_full).norm() / y_full.norm() < 0.2


def test_fma_division_equals_ieee_division():
    # all bf16 magnitudes in the range that can round to a non-zero e4m3 x a spread of scales
    g = torch.Generator().manual_seed(0)
    bits = torch.arange(0x0080, 0x7F80, dtype=torch.int32)  # every positive normal bf16
    x = (bits << 16).view(torch.float32)
    total_bad = 0
    L = oracle.lib()
    for rep in range(24):
        amax = torch.exp(torch.rand(x.numel(), generator=g) * 40 - 20).to(torch.bfloat16).float()
        s = torch.clamp(amax, min=1 / 512) / 448.0
        keep = (x <= amax * 1.0) & (x / s > 2 ** -12)
        xs_, ss_ = x[keep].contiguous(), s[keep].contiguous()
        total_bad += L.oracle_check_fma_division(xs_.data_ptr(), ss_.data_ptr(), xs_.numel())
    assert total_bad == 0
    # fp32 inputs too
    xf = torch.randn(400000, generator=g).abs() + 1e-3
    sf = (torch.rand(400000, generator=g) * 8 + 1e-2) / 448
    assert L.oracle_check_fma_division(xf.data_ptr(), sf.data_ptr(), xf.numel()) == 0


def test_silu_mul_quant_oracle_against_torch_expression():
    # mslk/moe/activation.py:220-294 restated with exact expf; test/moe/activation_test.py:97-168 tolerance
    g = torch.Generator().manual_seed(5)
    x0 = torch.randn((37, 640), generator=g).to(torch.bfloat16)
    x1 = torch.randn((37, 640), generator=g).to(torch.bfloat16)
    ub = torch.tensor([1200.0])
    q, s = oracle.silu_mul_quant(x0, x1, ub, 20)
    ref = x0.float() * torch.sigmoid(x0.float()) * x1.float()
    torch.testing.assert_close(q[:20].float() * s[:20, None], ref[:20], rtol=1e-1, atol=1e-3)
    assert bool((q.view(torch.uint8)[20:] == 0).all()) and bool((s[20:] == 0).all())
    # inverse scale = row max / 448 up to two roundings; the largest element maps to +-448
    torch.testing.assert_close(s[:20], ref[:20].abs().amax(dim=1) / 448.0, rtol=1e-6, atol=0)
    assert bool((q[:20].float().abs().amax(dim=1) == 448.0).all())
    # the upper bound clamps the row maximum, the floor 1e-12 keeps an all-zero row finite
    q2, s2 = oracle.silu_mul_quant(x0, x1, torch.tensor([0.05]))
    torch.testing.assert_close(s2, torch.full((37,), 1.0 / (448.0 / 0.05)), rtol=1e-6, atol=0)
    z = torch.zeros((2, 64), dtype=torch.bfloat16)
    q3, s3 = oracle.silu_mul_quant(z, z)
    assert bool((q3.view(torch.uint8) == 0).all()) and bool(torch.isfinite(s3).all()) and bool((s3 > 0).all())
    torch.testing.assert_close(oracle.silu_mul(x0, x1), ref, rtol=1e-6, atol=1e-7)


def test_silu_mul_quant_triton_fixture_close_to_oracle():
    gold = load_golden("silu_mul_quant_triton_b200.npz")
    if gold is None:
        pytest.skip("fixture captured from the reference's Triton kernel not present")
    from golden.make_golden import SILU_CASES, silu_inputs
    for i, (name, T, D, ub, valid, contiguous) in enumerate(SILU_CASES):
        x = silu_inputs(name, T, D, 400 + i)
        n = T if valid is None else valid
        q, s = oracle.silu_mul_quant(x[:, :D], x[:, D:], None if ub is None else torch.tensor([ub]), valid)
        s_g = torch.from_numpy(gold[f"{name}.s"]).reshape(T)
        q_g = torch.from_numpy(gold[f"{name}.q"]).reshape(T, D)
        torch.testing.assert_close(s[:n], s_g[:n], rtol=2e-6, atol=0)
        a, b = q.view(torch.uint8)[:n].to(torch.int16), q_g[:n].to(torch.int16)
        oa = torch.where((a & 0x80) != 0, -(a & 0x7f), a & 0x7f)
        ob = torch.where((b & 0x80) != 0, -(b & 0x7f), b & 0x7f)
        d = (oa - ob).abs()
        assert int(d.max()) <= 1 and float((d != 0).float().mean()) < 2e-3, name


def test_gather_scatter_oracles_against_torch_expressions():
    # mslk/moe/gather_scatter.py:431-486, 489-526, 677-740 restated; test/moe/gather_scatter_test.py formulations
    from golden.make_golden import gather_inputs
    T, D, E = 48, 96, 4
    x, tok, ex, scores = gather_inputs(T, D, E, 3, False)
    o = oracle.gather_scale_dense_tokens(x, tok, ex, scores, 30)
    ref = x[tok.long()] * scores[tok.long(), ex].view(-1, 1)
    assert torch.equal(o[:30], ref[:30]) and bool((o[30:] == 0).all())
    q, s = oracle.gather_scale_quant_dense_tokens(x, tok, ex, scores, torch.tensor([1200.0]))
    torch.testing.assert_close(q.float() * s[:, None], ref.float(), atol=0.0625 * float(s.max()), rtol=0.125)
    prod = x[tok.long()].float() * scores[tok.long(), ex].float().view(-1, 1)      # unrounded fp32 product
    torch.testing.assert_close(s, prod.abs().amax(dim=1).clamp(min=1e-12) / 448.0, rtol=1e-6, atol=0)
    g = torch.Generator().manual_seed(1)
    for dtype in (torch.bfloat16, torch.int32, torch.float32):
        inn = (torch.randn((24, D), generator=g) * 4).to(dtype)
        out = (torch.randn((24, D), generator=g) * 4).to(dtype)
        ti = torch.randperm(24, generator=g).to(torch.int32)
        want = out.clone().scatter_add_(0, ti[:20].long().view(-1, 1).expand(-1, D), inn[:20])
        oracle.scatter_add_dense_tokens(out, inn, ti, 20)
        assert torch.equal(out, want)
    EP, TK = 2, 40
    inn = torch.randint(-9, 9, (EP, TK, D), generator=g, dtype=torch.int32)
    counts = torch.tensor([7, 0, 20, 5])
    ti = (torch.randperm(TK, generator=g) % 10).to(torch.int32)
    out = torch.zeros((10, D), dtype=torch.int32)
    oracle.scatter_add_padded_tokens(inn, counts, ti, out)
    want = torch.zeros((10, D), dtype=torch.int32)
    cs = [0, 7, 7, 27, 32]
    for rank in range(EP):
        s0, e0 = cs[2 * rank], cs[2 * rank + 2]
        want.scatter_add_(0, ti[s0:e0].long().view(-1, 1).expand(-1, D), inn[rank, s0:e0])
    assert torch.equal(out, want)


def test_gather_scale_quant_triton_fixture_close_to_oracle():
    gold = load_golden("gather_scale_quant_triton_b200.npz")
    if gold is None:
        pytest.skip("fixture captured from the reference's Triton kernel not present")
    from golden.make_golden import GATHER_CASES, gather_inputs
    for i, (name, T, D, E, ub, valid, rowmajor) in enumerate(GATHER_CASES):
        x, tok, ex, scores = gather_inputs(T, D, E, 500 + i, rowmajor)
        n = T if valid is None else valid
        q, s = oracle.gather_scale_quant_dense_tokens(x, tok, ex, scores, None if ub is None else torch.tensor([ub]), valid)
        s_g = torch.from_numpy(gold[f"{name}.s"]).reshape(T)
        q_g = torch.from_numpy(gold[f"{name}.q"]).reshape(T, D)
        torch.testing.assert_close(s[:n], s_g[:n], rtol=2e-6, atol=0)
        a, b = q.view(torch.uint8)[:n].to(torch.int16), q_g[:n].to(torch.int16)
        oa = torch.where((a & 0x80) != 0, -(a & 0x7f), a & 0x7f)
        ob = torch.where((b & 0x80) != 0, -(b & 0x7f), b & 0x7f)
        d = (oa - ob).abs()
        assert int(d.max()) <= 1 and float((d != 0).float().mean()) < 2e-3, name


def test_stacked_nvfp4_oracles_consistent_with_dense_oracle():
    # quantize_stacked.py:22-178 / global_scale.py:40-230 restated on top of the pinned dense NVFP4 oracle
    from golden.make_golden import STACKED_CASES, stacked_inputs, unswizzle_stacked_scales
    for i, (name, m_sizes, K) in enumerate(STACKED_CASES):
        x = stacked_inputs(m_sizes, K, 600 + i)
        gs, idx = oracle.calculate_group_max(x, m_sizes)
        q, s, starts = oracle.nvfp4_quantize_stacked(m_sizes, x, gs)
        assert starts[-1] == sum((m + 127) // 128 * 128 for m in m_sizes) and s.shape[0] == starts[-1]
        r = 0
        for g, m in enumerate(m_sizes):
            if m:
                amax = float(x[r:r + m].abs().max())
                assert float(gs[g]) == pytest.approx(2688.0 / (amax if amax else 1e-8), rel=1e-6)
                assert bool((idx[r:r + m] == g).all())
                qd, sd = oracle.quantize_nvfp4(x[r:r + m].contiguous(), gs[g:g + 1])
                assert torch.equal(q[r:r + m], qd)
                assert torch.equal(unswizzle_stacked_scales(s, m_sizes, K)[r:r + m],
                                   oracle.from_blocked(sd.view(torch.uint8).reshape(-1), m, K // 16))
            else:
                assert float(gs[g]) == torch.finfo(torch.float32).max
            r += m
    # grouped GEMM oracle = dense oracle per group
    m_sizes, N, K = [5, 0, 130], 48, 64
    g = torch.Generator().manual_seed(2)
    x = torch.randn((135, K), generator=g).to(torch.bfloat16)
    w = (torch.randn((3 * N, K), generator=g) * 0.1).to(torch.bfloat16)
    xgs, _ = oracle.calculate_group_max(x, m_sizes)
    wgs, _ = oracle.calculate_group_max(w, [N] * 3)
    xq, xs, starts = oracle.nvfp4_quantize_stacked(m_sizes, x, xgs)
    wq, ws, _ = oracle.nvfp4_quantize_stacked([N] * 3, w, wgs)
    alpha = 1.0 / (xgs * wgs)
    y = oracle.gemm_nvfp4_grouped_stacked(xq, wq.view(3, N, K // 2), xs, ws, m_sizes, alpha, starts)
    ref = torch.cat([x[:5].float() @ w[:N].float().T, x[5:].float() @ w[2 * N:].float().T])
    assert float((y.float() - ref).norm() / ref.norm()) < 0.2
