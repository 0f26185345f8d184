"""Generate the golden fixtures in this directory by RUNNING THE REFERENCE.

Two legs, both writing ``.npz`` files next to this script:

``--leg cpu``  (no GPU needed) imports the reference package from ``--ref-root``
    with ``MSLK_PYTHON_ONLY=1`` and records, on seeded inputs,
    * ``quantize_fp8_row`` on CPU tensors (its torch path,
      ``mslk/quantize/triton/fp8_quantize.py:356-378``),
    * ``matmul_fp8_row`` CPU fallback (``mslk/gemm/triton/fp8_gemm.py:1190-1201``),
    * the NVFP4 torch reference ``data_to_nvfp4_with_global_scale`` from the
      reference's own test (``test/quantize/triton/fp4_quantize_test.py:259-296``),
      ``_to_blocked``, ``global_scale_nvfp4`` and ``dequantize_nvfp4``.
``--leg gpu_silu``  (needs a B200) runs the reference's fused ``silu_mul_quant`` (``mslk/moe/activation.py``).
``--leg gpu_fp4_stacked``  (needs a B200) runs ``calculate_group_max`` and ``nvfp4_quantize_stacked``
    (``mslk/quantize/triton/legacy``); the scale bytes of the real rows are stored un-swizzled, the padding
    rows (which the reference leaves uninitialised) are not.
``--leg gpu_gather``  (needs a B200) runs the reference's ``gather_scale_quant_dense_tokens``
    (``mslk/moe/gather_scatter.py``).  These two legs store outputs only; the tests regenerate the
    seeded inputs with ``silu_inputs`` / ``gather_inputs`` (CPU generator, same torch build).
``--leg gpu_fp4_f16``  (needs a B200) runs the NVFP4 quantizers (dense, group maximum, stacked) on fp16 inputs.
``--leg gpu_mx4``  (needs a B200) runs the reference's MXFP4 quantizer ``quantize_mx4``
    (``mslk/quantize/triton/quantize_kernels/mx4.py``) for group sizes 32 / 16 and the floor / even / ceil rounding
    modes; outputs only (the tests regenerate the inputs with ``mx4_inputs``).
``--leg gpu``  (needs a B200) runs the reference's Triton kernels
    ``triton_quantize_fp8_row`` and ``triton_quantize_nvfp4`` on the same seeded
    inputs; these are the bit-level pins for the GPU arithmetic.

The inputs are stored with the outputs so the tests do not depend on torch's
random streams.  bf16 / fp8 tensors are stored as their raw integer views.

Usage:  python tests/golden/make_golden.py --leg cpu --ref-root <path to reference checkout>
"""

from __future__ import annotations

import argparse
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _raw(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype in (torch.float8_e4m3fn,):
        return t.view(torch.uint8).numpy()
    if hasattr(torch, "float4_e2m1fn_x2") and t.dtype == torch.float4_e2m1fn_x2:
        return t.view(torch.uint8).numpy()
    return t.numpy()


def _randn_bf16(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g, dtype=torch.float32) * scale).to(torch.bfloat16)


# (name, shape, kwargs) -- mirrors the case list of the reference's own test
# test/quantize/triton/fp8_quantize_test.py:145-220 at fixture-friendly sizes.
FP8_ROW_CASES = [
    ("r8x300", (8, 300), {}),
    ("r2x1", (2, 1), {}),
    ("r2x4101", (2, 4101), {}),
    ("r3x9000", (3, 9000), {}),                       # > 8192: the reference's two-pass branch
    ("r16x4096", (16, 4096), {}),
    ("r4x14336", (4, 14336), {}),
    ("b4x2x3", (4, 2, 3), {}),
    ("b4x2x13_align8", (4, 2, 13), {"align_rows_to": 8}),
    ("b4x2x8_align8", (4, 2, 8), {"align_rows_to": 8}),
    ("b6x4x2x3", (6, 4, 2, 3), {}),
    ("b4x2x3_perm", (4, 2, 3), {"permute": (2, 0, 1)}),
    ("b6x4x2x3_perm", (6, 4, 2, 3), {"permute": (0, 3, 2, 1)}),
    ("r2x3_ub", (2, 3), {"scale_ub": 1200.0}),
    ("r8x64_ub_small", (8, 64), {"scale_ub": 1.5}),
    ("r20x30_jag", (20, 30), {"jagged": True}),
    ("r20x30_jag_align16", (20, 30), {"jagged": True, "align_rows_to": 16}),
    ("b6x4x2x3_jag", (6, 4, 2, 3), {"jagged": True}),
    ("r4x256_tiny", (4, 256), {"scale": 1e-4}),        # amax below eps -> eps floor
    ("r4x256_zero", (4, 256), {"scale": 0.0}),
]

NVFP4_CASES = [
    # test/quantize/triton/fp4_quantize_test.py:198-212 (fixture-sized subset)
    ("n128x64", (128, 64)), ("n5x64", (5, 64)), ("n128x16", (128, 16)), ("n5x16", (5, 16)),
    ("n256x64", (256, 64)), ("n128x128", (128, 128)), ("n150x64", (150, 64)),
    ("n128x144", (128, 144)), ("n1x2048", (1, 2048)), ("n250x512", (250, 512)),
]


def _fp8_inputs(name, shape, kw, seed):
    a = _randn_bf16(shape, seed, kw.get("scale", 1.0))
    zs = None
    if kw.get("jagged"):
        g = torch.Generator().manual_seed(seed + 1000)
        grouped = a.view(-1, a.shape[-2], a.shape[-1])
        zs = torch.randint(0, grouped.shape[1] + 1, (grouped.shape[0],), generator=g)
        mask = torch.arange(grouped.shape[1]).expand(grouped.shape[0], grouped.shape[1]) >= zs[:, None]
        grouped[mask] = 0.0
    if "permute" in kw:
        a = a.permute(kw["permute"])
    ub = torch.tensor([kw["scale_ub"]], dtype=torch.float32) if "scale_ub" in kw else None
    return a, ub, zs


def _import_reference(ref_root: str):
    os.environ["MSLK_PYTHON_ONLY"] = "1"
    sys.path.insert(0, ref_root)
    # torch.testing._internal.common_quantized imports `expecttest`, which is not
    # installed; it only needs the name to exist.
    if "expecttest" not in sys.modules:
        stub = types.ModuleType("expecttest")
        stub.TestCase = __import__("unittest").TestCase
        sys.modules["expecttest"] = stub


def leg_cpu(ref_root: str):
    _import_reference(ref_root)
    from mslk.quantize.triton.fp8_quantize import quantize_fp8_row
    from mslk.gemm.triton.fp8_gemm import matmul_fp8_row
    from mslk.quantize.triton.legacy.fp4_utils import dequantize_nvfp4, global_scale_nvfp4
    from mslk.quantize.triton.legacy.primitives import _to_blocked

    out = {}
    for i, (name, shape, kw) in enumerate(FP8_ROW_CASES):
        if kw.get("jagged") or "align_rows_to" in kw or "permute" in kw:
            continue  # the reference's CPU path ignores these options
        a, ub, _ = _fp8_inputs(name, shape, kw, seed=i)
        q, s = quantize_fp8_row(a, scale_ub=ub, use_triton=False)
        out[f"{name}.a"] = _raw(a)
        out[f"{name}.q"] = _raw(q)
        out[f"{name}.s"] = _raw(s)
        if ub is not None:
            out[f"{name}.ub"] = _raw(ub)
    np.savez_compressed(os.path.join(HERE, "fp8_row_cpu_path.npz"), **out)

    # CPU GEMM fallback of the reference on reference-quantized inputs
    out = {}
    for name, (M, N, K), sw in [("g64x48x256", (64, 48, 256), 0.02), ("g5x33x128", (5, 33, 128), 1.0)]:
        x = _randn_bf16((M, K), 100)
        w = _randn_bf16((N, K), 101, sw)
        xq, xs = quantize_fp8_row(x, use_triton=False)
        wq, ws = quantize_fp8_row(w, use_triton=False)
        y = matmul_fp8_row(xq, wq, xs, ws)
        for k, v in dict(xq=xq, wq=wq, xs=xs, ws=ws, y=y).items():
            out[f"{name}.{k}"] = _raw(v)
    np.savez_compressed(os.path.join(HERE, "fp8_gemm_cpu_path.npz"), **out)

    # NVFP4 torch reference from the reference's own test module
    sys.path.insert(0, os.path.join(ref_root, "test", "quantize", "triton"))
    import importlib.util
    spec = importlib.util.spec_from_file_location(
        "_ref_fp4_test", os.path.join(ref_root, "test", "quantize", "triton", "fp4_quantize_test.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    out = {}
    for i, (name, shape) in enumerate(NVFP4_CASES):
        x = _randn_bf16(shape, 200 + i)
        gs = global_scale_nvfp4(x)
        q, s, s_dec = mod.data_to_nvfp4_with_global_scale(x, 16)
        s_blocked = _to_blocked(s)
        deq = dequantize_nvfp4(q.view(torch.uint8), s_blocked.view(torch.uint8), gs)
        out[f"{name}.x"] = _raw(x)
        out[f"{name}.gs"] = _raw(gs.reshape(1))
        out[f"{name}.q"] = _raw(q)
        out[f"{name}.s"] = _raw(s)
        out[f"{name}.s_blocked"] = _raw(s_blocked)
        out[f"{name}.deq"] = _raw(deq)
    np.savez_compressed(os.path.join(HERE, "nvfp4_torch_ref.npz"), **out)
    print("cpu leg written")


def leg_gpu(ref_root: str):
    _import_reference(ref_root)
    assert torch.cuda.is_available()
    from mslk.quantize.triton.fp8_quantize import triton_quantize_fp8_row
    from mslk.quantize.triton.quantize_kernels.nvfp4 import quantize_nvfp4
    from mslk.quantize.triton.legacy.fp4_utils import global_scale_nvfp4

    out = {}
    for i, (name, shape, kw) in enumerate(FP8_ROW_CASES):
        a, ub, zs = _fp8_inputs(name, shape, kw, seed=i)
        q, s = triton_quantize_fp8_row(
            a.cuda(), None if ub is None else ub.cuda(), None if zs is None else zs.cuda(),
            align_rows_to=kw.get("align_rows_to"))
        torch.cuda.synchronize()
        out[f"{name}.a"] = _raw(a.contiguous())          # logical (permuted) content, contiguous
        out[f"{name}.q"] = _raw(q)
        out[f"{name}.s"] = _raw(s)
        if ub is not None:
            out[f"{name}.ub"] = _raw(ub)
        if zs is not None:
            out[f"{name}.zs"] = _raw(zs)
    np.savez_compressed(os.path.join(HERE, "fp8_row_triton_b200.npz"), **out)

    out = {}
    for i, (name, shape) in enumerate(NVFP4_CASES):
        x = _randn_bf16(shape, 200 + i)
        gs = global_scale_nvfp4(x.cuda())
        q, s = quantize_nvfp4(x.cuda(), gs)
        torch.cuda.synchronize()
        out[f"{name}.x"] = _raw(x)
        out[f"{name}.gs"] = _raw(gs.reshape(1))
        out[f"{name}.q"] = _raw(q)
        out[f"{name}.s_blocked"] = _raw(s)
    np.savez_compressed(os.path.join(HERE, "nvfp4_triton_b200.npz"), **out)
    print("gpu leg written")


# (T, D, scale_ub, valid tokens or None, contiguous) -- after test/moe/activation_test.py:97-168
SILU_CASES = [
    ("s1x5120", 1, 5120, None, None, True),
    ("s32x5120", 32, 5120, None, None, True),
    ("s32x7168_ub", 32, 7168, 1200.0, None, True),
    ("s16x8192_strided", 16, 8192, None, None, False),
    ("s200x1024_partial", 200, 1024, None, 100, True),
    ("s16x14336_ub_small", 16, 14336, 0.05, None, True),
    ("s8x256_tiny", 8, 256, None, None, True),
    ("s32x2048_wide", 32, 2048, None, None, True),
]


def silu_inputs(name, T, D, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((T, 2 * D), generator=g, dtype=torch.float32).to(torch.bfloat16)
    if "tiny" in name:
        x = (x.float() * 1e-7).to(torch.bfloat16)      # row maxima below the 1e-12 floor of the scale
    elif "wide" in name:
        x = (x.float() * 60.0).to(torch.bfloat16)      # gate values below -87.3: exp(-x) beyond 2^126
    else:
        x = torch.sign(x) * torch.clamp(torch.abs(x), 0.01, 2.0)
    return x


def leg_gpu_silu(ref_root: str):
    """silu_mul_quant of the reference (Triton, mslk/moe/activation.py:72-294) on a B200."""
    _import_reference(ref_root)
    import importlib.util
    spec = importlib.util.spec_from_file_location("_ref_activation", os.path.join(ref_root, "mslk", "moe", "activation.py"))
    act = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(act)
    out = {}
    for i, (name, T, D, ub, valid, contiguous) in enumerate(SILU_CASES):
        x = silu_inputs(name, T, D, 400 + i).cuda()
        x0, x1 = x[:, :D], x[:, D:]
        if contiguous:
            x0, x1 = x0.contiguous(), x1.contiguous()
        ubt = None if ub is None else torch.tensor([ub], dtype=torch.float32, device="cuda")
        vt = None if valid is None else torch.tensor([valid], dtype=torch.int32, device="cuda")
        q, s = act.silu_mul_quant(x0, x1, ubt, vt)
        torch.cuda.synchronize()
        if valid is not None:          # rows past the count are never written: keep the file small
            q.view(torch.uint8)[valid:] = 0
            s[valid:] = 0
        # the inputs are not stored: silu_inputs() regenerates them from the seed
        out[f"{name}.q"] = _raw(q)
        out[f"{name}.s"] = _raw(s)
    np.savez_compressed(os.path.join(HERE, "silu_mul_quant_triton_b200.npz"), **out)
    print("gpu silu leg written")


# (name, T, D, E, scale_ub, valid rows, scores stored row-major)
GATHER_CASES = [
    ("g64x5120_e8", 64, 5120, 8, None, None, False),
    ("g128x2048_e2_ub_partial", 128, 2048, 2, 1200.0, 64, True),
    ("g32x1024_e4_ub_small", 32, 1024, 4, 0.05, None, False),
]


def gather_inputs(T, D, E, seed, rowmajor):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((T, D), generator=g, dtype=torch.float32).to(torch.bfloat16)
    token_indices = torch.randperm(T, generator=g).to(torch.int32)
    expert_indices = torch.randint(0, E, (T,), generator=g)
    scores = torch.randn((E, T), generator=g, dtype=torch.float32).to(torch.bfloat16).transpose(0, 1)
    if rowmajor:
        scores = scores.contiguous()
    return x, token_indices, expert_indices, scores


def leg_gpu_gather(ref_root: str):
    """gather_scale_quant_dense_tokens of the reference (Triton, mslk/moe/gather_scatter.py:96-169,537-655) on a B200."""
    _import_reference(ref_root)
    import importlib.util
    spec = importlib.util.spec_from_file_location("_ref_gather_scatter",
                                                  os.path.join(ref_root, "mslk", "moe", "gather_scatter.py"))
    gs = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gs)
    out = {}
    for i, (name, T, D, E, ub, valid, rowmajor) in enumerate(GATHER_CASES):
        x, tok, ex, scores = gather_inputs(T, D, E, 500 + i, rowmajor)
        scores_d = scores.cuda()          # a dense transposed view keeps its strides
        assert scores_d.stride() == scores.stride()
        ubt = None if ub is None else torch.tensor([ub], dtype=torch.float32, device="cuda")
        vt = None if valid is None else torch.tensor([valid], dtype=torch.int32, device="cuda")
        q, s = gs.gather_scale_quant_dense_tokens(x.cuda(), tok.cuda(), ex.cuda(), scores_d, ubt, vt)
        torch.cuda.synchronize()
        if valid is not None:
            q.view(torch.uint8)[valid:] = 0
            s[valid:] = 0
        out[f"{name}.q"] = _raw(q)
        out[f"{name}.s"] = _raw(s)
    np.savez_compressed(os.path.join(HERE, "gather_scale_quant_triton_b200.npz"), **out)
    print("gpu gather leg written")


# (name, rows per group, K): stacked NVFP4 quantization with one global scale per group
STACKED_CASES = [
    ("st_4g", [64, 232, 0, 600], 1024),
    ("st_1g", [300], 512),
    ("st_16g", [0, 129, 1, 128, 127, 0, 0, 256, 300, 5, 64, 0, 96, 33, 512, 7], 256),
]


def stacked_inputs(m_sizes, K, seed):
    g = torch.Generator().manual_seed(seed)
    parts = [torch.randn((m, K), generator=g, dtype=torch.float32) * (0.05 * (1 + 3 * i)) for i, m in enumerate(m_sizes)]
    if len(parts) > 2 and m_sizes[-1] > 0:
        parts[-1] = parts[-1] * 0.0          # an all-zero group: the 1e-8 stand-in of the global scale
    return torch.cat(parts, dim=0).to(torch.bfloat16)


def unswizzle_stacked_scales(scale_flat, m_sizes, K):
    """[sum m, K/16] scale bytes of the real rows, from the padded + swizzled buffer."""
    pc = (K // 16 + 3) // 4 * 4
    buf = scale_flat.reshape(-1).view(torch.uint8).cpu()
    rows, pr = [], 0
    for m in m_sizes:
        mp = (m + 127) // 128 * 128
        if m > 0:
            blk = buf[pr * pc:(pr + mp) * pc].reshape(mp // 128, pc // 4, 32, 4, 4)   # [rb, cb, r%32, r//32, c]
            un = blk.permute(0, 3, 2, 1, 4).reshape(mp, pc)                           # row = rb*128 + (r//32)*32 + r%32
            rows.append(un[:m, : K // 16])
        pr += mp
    return torch.cat(rows, dim=0) if rows else torch.zeros((0, K // 16), dtype=torch.uint8)


def leg_gpu_fp4_stacked(ref_root: str):
    """calculate_group_max + nvfp4_quantize_stacked of the reference (Triton) on a B200."""
    _import_reference(ref_root)
    from mslk.quantize.triton.legacy.global_scale import calculate_group_max
    from mslk.quantize.triton.legacy.quantize_stacked import nvfp4_quantize_stacked
    out = {}
    for i, (name, m_sizes, K) in enumerate(STACKED_CASES):
        x = stacked_inputs(m_sizes, K, 600 + i).cuda()
        ms = torch.tensor(m_sizes, dtype=torch.int64, device="cuda")
        gs, idx = calculate_group_max(x, ms)
        q, s = nvfp4_quantize_stacked(ms, x, gs)
        torch.cuda.synchronize()
        out[f"{name}.gs"] = _raw(gs)
        out[f"{name}.idx"] = _raw(idx)
        out[f"{name}.q"] = _raw(q.view(torch.uint8))
        out[f"{name}.s_rows"] = _raw(unswizzle_stacked_scales(s, m_sizes, K))
    np.savez_compressed(os.path.join(HERE, "nvfp4_stacked_triton_b200.npz"), **out)
    print("gpu fp4 stacked leg written")


# fp16 inputs of the NVFP4 quantizers (the reference's kernels take fp16 or bf16): dense cases and one stacked case
NVFP4_F16_CASES = [("h_r130_k256", (130, 256)), ("h_r5_k64", (5, 64)), ("h_r256_k1040", (256, 1040))]
STACKED_F16_CASE = ("h_st_5g", [64, 200, 0, 129, 7], 512)


def nvfp4_f16_inputs(shape, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g, dtype=torch.float32)
    x = x * torch.exp2(torch.randint(-6, 7, (shape[0], 1), generator=g).float())   # rows over a few binades of fp16
    return x.to(torch.float16)


def leg_gpu_fp4_f16(ref_root: str):
    """quantize_nvfp4, calculate_group_max and nvfp4_quantize_stacked of the reference (Triton) on a B200, fp16 inputs."""
    _import_reference(ref_root)
    from mslk.quantize.triton.quantize_kernels.nvfp4 import quantize_nvfp4
    from mslk.quantize.triton.legacy.global_scale import calculate_group_max
    from mslk.quantize.triton.legacy.quantize_stacked import nvfp4_quantize_stacked
    out = {}
    for i, (name, shape) in enumerate(NVFP4_F16_CASES):
        x = nvfp4_f16_inputs(shape, 800 + i).cuda()
        gs = (448.0 * 6.0) / x.abs().amax().float()     # global_scale_nvfp4 (legacy/fp4_utils.py:78-92) asserts bf16
        q, s = quantize_nvfp4(x, gs)
        torch.cuda.synchronize()
        out[f"{name}.gs"] = _raw(gs.reshape(1).float())
        out[f"{name}.q"] = _raw(q)
        out[f"{name}.s_blocked"] = _raw(s)
    name, m_sizes, K = STACKED_F16_CASE
    x = nvfp4_f16_inputs((sum(m_sizes), K), 850).cuda()
    ms = torch.tensor(m_sizes, dtype=torch.int64, device="cuda")
    gs, idx = calculate_group_max(x, ms)
    q, s = nvfp4_quantize_stacked(ms, x, gs)
    torch.cuda.synchronize()
    out[f"{name}.gs"] = _raw(gs)
    out[f"{name}.idx"] = _raw(idx)
    out[f"{name}.q"] = _raw(q.view(torch.uint8))
    out[f"{name}.s_rows"] = _raw(unswizzle_stacked_scales(s, m_sizes, K))
    np.savez_compressed(os.path.join(HERE, "nvfp4_f16_triton_b200.npz"), **out)
    print("gpu fp4 f16 leg written")


# (name, shape, dtype) of the MXFP4 quantizer cases: rows below / at / above the 128-row scale block, K with a partial
# group of four scales, fp16 input, values spanning many binades, an all-zero group and exact powers of two
MX4_CASES = [("r128_k64", (128, 64), "bf16"), ("r5_k128", (5, 128), "bf16"), ("r150_k1024", (150, 1024), "bf16"),
             ("r70_k3584", (70, 3584), "bf16"), ("r1_k5120", (1, 5120), "bf16"), ("r129_k96", (129, 96), "bf16"),
             ("r64_k512_f16", (64, 512), "f16"), ("r256_k256_wide", (256, 256), "bf16")]


MX4_NEAREST_CASES = ("r128_k64", "r129_k96", "r64_k512_f16", "r256_k256_wide")   # rounding mode 0 is captured for these


MX4_STOCHASTIC_CASES = ("r128_k64", "r129_k96", "r64_k512_f16", "r256_k256_wide")    # rounding mode 3 likewise
MX4_SEEDS = (0x12345678, (1 << 62) + 12345)
MX4_STACKED_STOCHASTIC_CASES = [("st_50_30_48", [50, 30, 48], 64), ("st_130_0_7", [130, 0, 7], 256)]


def mx4_inputs(name, shape, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g, dtype=torch.float32)
    if name.endswith("wide"):
        x = x * torch.exp2(torch.randint(-40, 40, (shape[0], 1), generator=g).float())
        x[0, :32] = 0.0                       # an all-zero group
        x[1, :32] = 4.0                       # exact powers of two: ceil and floor of log2 coincide
        x[2, :32] = 6.0
    return x.to(torch.bfloat16 if dtype == "bf16" else torch.float16)


def leg_gpu_mx4(ref_root: str):
    """quantize_mx4 of the reference (Triton) on a B200: group sizes 32 / 16, every rounding mode (stochastic with
    fixed seeds, dense and stacked)."""
    _import_reference(ref_root)
    from mslk.quantize.triton.quantize_kernels.mx4 import quantize_mx4
    out = {}
    for i, (name, shape, dtype) in enumerate(MX4_CASES):
        x = mx4_inputs(name, shape, dtype, 700 + i).cuda()
        for group in (32, 16):
            for mode in (4, 1, 2, 0):
                if mode == 0 and name not in MX4_NEAREST_CASES:
                    continue
                q, s = quantize_mx4(x, group_size=group, rounding_mode=mode)
                torch.cuda.synchronize()
                out[f"{name}.g{group}.m{mode}.q"] = _raw(q.view(torch.uint8))
                out[f"{name}.g{group}.m{mode}.s"] = _raw(s.view(torch.uint8))
            if name in MX4_STOCHASTIC_CASES:
                for seed in MX4_SEEDS:
                    q, s = quantize_mx4(x, group_size=group, rounding_mode=3, seed=seed)
                    torch.cuda.synchronize()
                    out[f"{name}.g{group}.m3.seed{seed}.q"] = _raw(q.view(torch.uint8))
                    out[f"{name}.g{group}.m3.seed{seed}.s"] = _raw(s.view(torch.uint8))
    # stacked segments with stochastic rounding: the random streams count rows of the padded scale matrix
    from mslk.quantize.triton.quantize_kernels.mx4_stacked import quantize_mx4_stacked
    for name, m_sizes, K in MX4_STACKED_STOCHASTIC_CASES:
        x = mx4_inputs(name, (sum(m_sizes), K), "bf16", 900 + K).cuda()
        ms = torch.tensor(m_sizes, dtype=torch.int64, device="cuda")
        q, s = quantize_mx4_stacked(ms, x, group_size=32, rounding_mode=3, seed=MX4_SEEDS[0])
        torch.cuda.synchronize()
        out[f"{name}.m3.q"] = _raw(q.view(torch.uint8))
        out[f"{name}.m3.s"] = _raw(s.view(torch.uint8))
    np.savez_compressed(os.path.join(HERE, "mx4_triton_b200.npz"), **out)
    print("gpu mx4 leg written")


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--leg", choices=["cpu", "gpu", "gpu_silu", "gpu_gather", "gpu_fp4_stacked", "gpu_mx4", "gpu_fp4_f16"], required=True)
    ap.add_argument("--ref-root", required=True)
    ap.add_argument("--out-dir", default=None, help="write here instead of beside this script")
    args = ap.parse_args()
    if args.out_dir:
        HERE = args.out_dir
        os.makedirs(HERE, exist_ok=True)
    {"cpu": leg_cpu, "gpu": leg_gpu, "gpu_silu": leg_gpu_silu, "gpu_gather": leg_gpu_gather,
     "gpu_fp4_stacked": leg_gpu_fp4_stacked, "gpu_mx4": leg_gpu_mx4, "gpu_fp4_f16": leg_gpu_fp4_f16}[args.leg](args.ref_root)
