"""Races this library's kernels against the reference's own sm_100 kernels on one B200.

    python baseline/race_ref_gpu.py [--quick] [--out <file>.jsonl]

Needs baseline/_ref/libmslk_ref_gpu.so (built by baseline/build_ref_gpu.py from the reference's sources at
stock CUTLASS) and, for the quantizer, baseline/_ref/pyref (the reference's Python package, `--python`).
For every case both sides get the same device tensors, are timed the same way (CUDA events around `iters`
back-to-back launches after warm-up, weights rotated through more than the L2 holds) and their outputs are
compared element by element in bf16 units in the last place.  Launches are replayed from CUDA graphs, the two
sides alternately (median of three rounds each).  One JSON line per case:
    {"case": ..., "ours_us": ..., "ref_us": ..., "ours_over_ref_speed": ref_us / ours_us,
     "max_ulp": ..., "frac_within_1ulp": ..., "frac_equal": ...}
"""

from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, ROOT)


def bf16_ulp_diff(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """|a - b| counted in bf16 steps (both tensors bf16): bit patterns mapped to a monotone integer line."""
    def key(t):
        i = t.contiguous().view(torch.int16).to(torch.int32)
        return torch.where(i < 0, -(i & 0x7fff), i)
    return (key(a) - key(b)).abs()


def compare(y, y_ref):
    d = bf16_ulp_diff(y, y_ref)
    n = d.numel()
    return {"max_ulp": int(d.max()), "frac_within_1ulp": float((d <= 1).sum()) / n, "frac_equal": float((d == 0).sum()) / n}


_NVML = None


def sm_clock_mhz():
    """Current SM clock of the device in use (read-only NVML query); None without NVML."""
    global _NVML
    try:
        import pynvml
        if _NVML is None:
            pynvml.nvmlInit()
            _NVML = pynvml.nvmlDeviceGetHandleByIndex(torch.cuda.current_device())
        return int(pynvml.nvmlDeviceGetClockInfo(_NVML, pynvml.NVML_CLOCK_SM))
    except Exception:
        return None


LAST_MHZ = [None]


def time_us(fn, n_variants, iters, warmup):
    """us per launch, `iters` launches replayed from one CUDA graph: both sides are then timed by the device, not
    by how fast their host paths (ctypes here, the torch dispatcher there) can issue short kernels.  The SM clock is
    sampled while the timed replay runs (LAST_MHZ): on a power-capped part the clock, not the kernel, can differ
    between two runs."""
    for i in range(warmup):
        fn(i % n_variants)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            for i in range(iters):
                fn(i % n_variants)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    mhz = []
    while not e1.query() and len(mhz) < 64:
        c = sm_clock_mhz()
        if c is None:
            break
        mhz.append(c)
    torch.cuda.synchronize()
    mhz.sort()
    LAST_MHZ[0] = mhz[len(mhz) // 2] if mhz else sm_clock_mhz()
    return e0.elapsed_time(e1) / iters * 1e3


def race_pair(ours_fn, ref_fn, n_variants, iters, warmup, rounds=5):
    """Median us per launch of both sides, measured alternately so that clock and temperature drift over the run
    hits both alike: the side that goes first changes every round, and a short idle gap in front of every
    measurement lets the power state of this 1000 W part settle the same way for both."""
    import time
    a, b = [], []
    for r in range(rounds):
        for side in ((0, 1) if r % 2 == 0 else (1, 0)):
            time.sleep(0.2)
            if side == 0:
                a.append((time_us(ours_fn, n_variants, iters, warmup), LAST_MHZ[0]))
            else:
                b.append((time_us(ref_fn, n_variants, iters, warmup), LAST_MHZ[0]))
    a.sort(key=lambda t: t[0])
    b.sort(key=lambda t: t[0])
    RACE_MHZ[:] = [a[len(a) // 2][1], b[len(b) // 2][1]]
    return a[len(a) // 2][0], b[len(b) // 2][0]


RACE_MHZ = [None, None]        # SM clock seen during the median run of each side of the last race_pair


def randn(shape, std=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda", dtype=torch.float32) * std).to(torch.bfloat16)


def variants(bytes_per_variant, rotate_mb=400.0):
    return max(1, min(8, math.ceil(rotate_mb * 1e6 / max(1, bytes_per_variant))))


def race_dense(ops, ref, M, N, K, iters, warmup, w_std=0.02):
    nv = variants(N * K)
    xq, xs = ops.quantize_fp8_row(randn((M, K), seed=1))
    ws = [ops.quantize_fp8_row(randn((N, K), w_std, seed=10 + i)) for i in range(nv)]
    y, y_ref = (torch.empty((M, N), dtype=torch.bfloat16, device="cuda") for _ in range(2))
    # the instance the reference's heuristic picks on sm_100 (csrc/gemm/cutlass/f8f8bf16_rowwise.cu:24-50)
    ref_fn = ref.f8f8bf16_rowwise_small if M <= 128 else ref.f8f8bf16_rowwise_large
    ours, theirs = race_pair(lambda i: ops.f8f8bf16_rowwise_out(xq, ws[i][0], xs, ws[i][1], y),
                             lambda i: ref_fn(xq, ws[i][0], xs, ws[i][1], y_ref), nv, iters, warmup)
    ops.f8f8bf16_rowwise_out(xq, ws[0][0], xs, ws[0][1], y)
    ref_fn(xq, ws[0][0], xs, ws[0][1], y_ref)
    torch.cuda.synchronize()
    flops = 2.0 * M * N * K
    return {"case": f"f8f8bf16_rowwise M={M} N={N} K={K}", "ours_us": ours, "ref_us": theirs,
            "ours_tflops": flops / ours / 1e6, "ref_tflops": flops / theirs / 1e6, "ours_over_ref_speed": theirs / ours,
            "ref_instance": "128_64_128_1_1_1" if M <= 128 else "128_256_128_2_1_1", **compare(y, y_ref)}


def race_grouped(ops, ref, E, tokens, N, K, iters, warmup, equal=False):
    from microbench import zipf_counts
    counts = torch.full((E,), tokens // E) if equal else zipf_counts(E, tokens)
    ms = counts.to(torch.int64).cuda()
    xq, xs = ops.quantize_fp8_row(randn((tokens, K), seed=2))
    wq, ws = ops.quantize_fp8_row(randn((E, N, K), 0.02, seed=3))
    y_ref = torch.empty((tokens * N,), dtype=torch.bfloat16, device="cuda")
    ours, theirs = race_pair(lambda i: ops.f8f8bf16_rowwise_grouped_stacked(xq, wq, xs, ws.view(-1), ms),
                             lambda i: ref.f8f8bf16_rowwise_grouped_stacked(xq, wq, xs, ws, ms, y_ref), 1, iters, warmup)
    y = ops.f8f8bf16_rowwise_grouped_stacked(xq, wq, xs, ws.view(-1), ms)
    yr = ref.f8f8bf16_rowwise_grouped_stacked(xq, wq, xs, ws, ms, y_ref)
    torch.cuda.synchronize()
    flops = 2.0 * tokens * N * K
    how = f"{tokens // E} tokens each" if equal else "Zipf 1.2, two empty experts"
    return {"case": f"f8f8bf16_rowwise_grouped_stacked E={E} tokens={tokens} N={N} K={K} ({how})",
            "ours_us": ours, "ref_us": theirs, "ours_tflops": flops / ours / 1e6, "ref_tflops": flops / theirs / 1e6,
            "ours_over_ref_speed": theirs / ours, "ref_instance": "grouped_256_256_128_2_1_1", **compare(y, yr)}


def race_nvfp4(ops, ref, M, N, K, iters, warmup):
    nv = variants(N * K // 2)
    x = randn((M, K), seed=4)
    gx = (448.0 * 6.0) / x.abs().amax().float()
    xq, sx = ops.quantize_nvfp4(x, gx)
    ws = []
    for i in range(nv):
        w = randn((N, K), seed=20 + i)
        gw = (448.0 * 6.0) / w.abs().amax().float()
        wq, sw = ops.quantize_nvfp4(w, gw)
        ws.append((wq, sw, (1.0 / (gx * gw)).reshape(1)))
    y, y_ref = (torch.empty((M, N), dtype=torch.bfloat16, device="cuda") for _ in range(2))
    # csrc/gemm/cutlass/f4f4bf16.cu:44-1266: 256_256_2_1_1 for 8192^3, 256_128_4_1_1 for M <= 64 at (28672, 8192)
    ref_fn = ref.f4f4bf16_small if M <= 128 else ref.f4f4bf16_large
    ours, theirs = race_pair(lambda i: ops.f4f4bf16(xq, ws[i][0], sx, ws[i][1], output=y, global_scale=ws[i][2]),
                             lambda i: ref_fn(xq, ws[i][0], sx, ws[i][1], y_ref, ws[i][2]), nv, iters, warmup)
    ops.f4f4bf16(xq, ws[0][0], sx, ws[0][1], output=y, global_scale=ws[0][2])
    ref_fn(xq, ws[0][0], sx, ws[0][1], y_ref, ws[0][2])
    torch.cuda.synchronize()
    flops = 2.0 * M * N * K
    return {"case": f"f4f4bf16 (NVFP4) M={M} N={N} K={K}", "ours_us": ours, "ref_us": theirs,
            "ours_tflops": flops / ours / 1e6, "ref_tflops": flops / theirs / 1e6, "ours_over_ref_speed": theirs / ours,
            "ref_instance": "256_128_4_1_1" if M <= 128 else "256_256_2_1_1", **compare(y, y_ref)}


def race_mxfp4(ops, ref, M, N, K, iters, warmup):
    nv = variants(N * K // 2)
    xq, sx = ops.quantize_mx4(randn((M, K), 0.1, seed=5), 32)
    ws = [ops.quantize_mx4(randn((N, K), 0.01, seed=40 + i), 32) for i in range(nv)]
    e8 = getattr(torch, "float8_e8m0fnu")
    f4 = getattr(torch, "float4_e2m1fn_x2")
    y, y_ref = (torch.empty((M, N), dtype=torch.bfloat16, device="cuda") for _ in range(2))
    rx, rsx = xq.view(f4), sx.view(e8)
    rws = [(w.view(f4), s.view(e8)) for w, s in ws]
    ours, theirs = race_pair(lambda i: ops.f4f4bf16(xq, ws[i][0], sx, ws[i][1], output=y),
                             lambda i: ref.f4f4bf16_large_mx(rx, rws[i][0], rsx, rws[i][1], y_ref), nv, iters, warmup)
    ops.f4f4bf16(xq, ws[0][0], sx, ws[0][1], output=y)
    ref.f4f4bf16_large_mx(rx, rws[0][0], rsx, rws[0][1], y_ref)
    torch.cuda.synchronize()
    flops = 2.0 * M * N * K
    return {"case": f"f4f4bf16 (MXFP4, block 32) M={M} N={N} K={K}", "ours_us": ours, "ref_us": theirs,
            "ours_tflops": flops / ours / 1e6, "ref_tflops": flops / theirs / 1e6, "ours_over_ref_speed": theirs / ours,
            "ref_instance": "256_256_2_1_1", **compare(y, y_ref)}


def race_grouped_fp4(ops, ref, E, tokens, N, K, mx, iters, warmup):
    """Grouped (stacked) FP4 GEMM, NVFP4 or MXFP4, against the reference instance its heuristic picks for these shapes
    (csrc/gemm/cutlass/f4f4bf16_grouped.cu:60-230 -> f4f4bf16_grouped_256_256_256_2_1_1)."""
    from microbench import zipf_counts
    counts = zipf_counts(E, tokens)
    ms = counts.to(torch.int64).cuda()
    w_ms = torch.full((E,), N, dtype=torch.int64, device="cuda")
    x, w = randn((tokens, K), 0.1, seed=6), randn((E * N, K), 0.01, seed=7)
    f4 = getattr(torch, "float4_e2m1fn_x2")
    starts = torch.zeros(E + 1, dtype=torch.int64)
    starts[1:] = torch.cumsum((counts.to(torch.int64) + 127) // 128 * 128, 0)
    starts = starts.cuda()
    if mx:
        e8 = getattr(torch, "float8_e8m0fnu")
        xq, sx = ops.quantize_mx4_stacked(ms, x)
        wq, sw = ops.quantize_mx4_stacked(w_ms, w)
        sw3 = sw[: E * N * (K // 32)].view(E, -1)
        gs = None
        r_sx, r_sw = sx.view(e8), sw3.view(e8)
    else:
        x_gs, _ = ops.calculate_group_max(x, ms)
        w_gs, _ = ops.calculate_group_max(w, w_ms)
        xq, sx = ops.nvfp4_quantize_stacked(ms, x, x_gs)
        wq, sw = ops.nvfp4_quantize_stacked(w_ms, w, w_gs)
        sw3 = sw[: E * N].view(E, N, -1)
        gs = torch.reciprocal(x_gs * w_gs)
        r_sx, r_sw = sx, sw3
    wq3 = wq.view(torch.uint8).view(E, N, K // 2)
    xq8 = xq.view(torch.uint8)
    y_ref = torch.empty((tokens, N), dtype=torch.bfloat16, device="cuda")
    ours_fn = lambda i: ops.f4f4bf16_grouped_stacked(xq8, wq3, sx, sw3, ms, gs, starts, use_mx=mx)
    ref_fn = lambda i: ref.f4f4bf16_grouped_stacked(xq8.view(f4), wq3.view(f4), r_sx, r_sw, ms, gs, starts, y_ref)
    ours, theirs = race_pair(ours_fn, ref_fn, 1, iters, warmup)
    y = ours_fn(0)
    ref_fn(0)
    torch.cuda.synchronize()
    flops = 2.0 * tokens * N * K
    return {"case": f"f4f4bf16_grouped_stacked ({'MXFP4' if mx else 'NVFP4'}) E={E} tokens={tokens} N={N} K={K} (Zipf 1.2, two empty experts)",
            "ours_us": ours, "ref_us": theirs, "ours_tflops": flops / ours / 1e6, "ref_tflops": flops / theirs / 1e6,
            "ours_over_ref_speed": theirs / ours, "ref_instance": "grouped_256_256_256_2_1_1", **compare(y, y_ref)}


def race_kgrouped_mxfp4(ops, ref, M, N, k_sizes, iters, warmup):
    """K-grouped ("2D-2D") MXFP4 GEMM against the same reference instance through its offsets path."""
    e8, f4 = getattr(torch, "float8_e8m0fnu"), getattr(torch, "float4_e2m1fn_x2")
    xqs, wqs, xss, wss = [], [], [], []
    for i, kg in enumerate(k_sizes):
        if kg == 0:
            continue
        q, s = ops.quantize_mx4(randn((M, kg), 0.1, seed=50 + i), 32)
        xqs.append(q)
        xss.append(s.view(torch.uint8).reshape(-1))
        q, s = ops.quantize_mx4(randn((N, kg), 0.01, seed=70 + i), 32)
        wqs.append(q)
        wss.append(s.view(torch.uint8).reshape(-1))
    xq, wq = torch.cat(xqs, dim=1).contiguous(), torch.cat(wqs, dim=1).contiguous()
    sx, sw = torch.cat(xss).view(e8), torch.cat(wss).view(e8)
    offs = torch.tensor(k_sizes, device="cuda").cumsum(0).to(torch.int32)
    G = len(k_sizes)
    y = torch.empty((G, M, N), dtype=torch.bfloat16, device="cuda")
    y_ref = torch.zeros((G, M, N), dtype=torch.bfloat16, device="cuda")
    ours_fn = lambda i: ops.f4f4bf16_grouped_mm(xq, wq.transpose(-2, -1), sx, sw, offs, y)
    ref_fn = lambda i: ref.f4f4bf16_grouped_mm(xq.view(f4), wq.view(f4), sx, sw, offs, None, y_ref)
    ours, theirs = race_pair(ours_fn, ref_fn, 1, iters, warmup)
    ours_fn(0)
    ref_fn(0)
    torch.cuda.synchronize()
    live = [g for g, kg in enumerate(k_sizes) if kg]          # the reference leaves the output of an empty group untouched
    flops = 2.0 * M * N * sum(k_sizes)
    return {"case": f"f4f4bf16_grouped_mm 2D-2D (MXFP4) M={M} N={N} K groups={k_sizes}", "ours_us": ours, "ref_us": theirs,
            "ours_tflops": flops / ours / 1e6, "ref_tflops": flops / theirs / 1e6, "ours_over_ref_speed": theirs / ours,
            "ref_instance": "grouped_256_256_256_2_1_1", **compare(y[live], y_ref[live])}


def race_quantize(ops, ref_quant, M, K, iters, warmup):
    nv = variants(M * K * 2)
    xs = [randn((M, K), seed=30 + i) for i in range(nv)]
    ours, theirs = race_pair(lambda i: ops.quantize_fp8_row(xs[i]), lambda i: ref_quant(xs[i]), nv, iters, warmup)
    q, s = ops.quantize_fp8_row(xs[0])
    qr, sr = ref_quant(xs[0])
    byts = 3.0 * M * K + 4.0 * M
    return {"case": f"quantize_fp8_row M={M} K={K} bf16", "ours_us": ours, "ref_us": theirs, "ours_gbs": byts / ours / 1e3,
            "ref_gbs": byts / theirs / 1e3, "ours_over_ref_speed": theirs / ours,
            "bytes_equal": bool(torch.equal(q.view(torch.uint8), qr.view(torch.uint8))), "scales_equal": bool(torch.equal(s, sr)),
            "ref_kernel": "triton_quantize_fp8_row (mslk/quantize/triton/fp8_quantize.py:210-316)"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--quick", action="store_true", help="headline shapes only")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    lib = os.path.join(HERE, "_ref", "libmslk_ref_gpu.so")
    if not os.path.exists(lib):
        print(json.dumps({"unavailable": f"{lib} is missing: run baseline/build_ref_gpu.py"}))
        return
    from mslk_b200 import ops
    torch.ops.load_library(lib)
    ref = torch.ops.mslk_ref
    lines = []

    def emit(r):
        r["ours_sm_mhz"], r["ref_sm_mhz"] = RACE_MHZ
        lines.append(r)
        print(json.dumps(r), flush=True)

    llama = [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)]
    emit(race_dense(ops, ref, 8192, 8192, 8192, args.iters, args.warmup))
    for M in ((8192,) if args.quick else (8192, 2048, 128, 16, 1)):
        for N, K in llama:
            emit(race_dense(ops, ref, M, N, K, args.iters if M >= 2048 else 4 * args.iters, args.warmup))
    if not args.quick:
        emit(race_dense(ops, ref, 4096, 4096, 4096, args.iters, args.warmup))
        for N, K in ((57344 // 8, 8192), (8192, 28672 // 8)):
            emit(race_dense(ops, ref, 8192, N, K, args.iters, args.warmup, w_std=0.01))
    for N, K in ((16384, 5120), (5120, 8192)):
        emit(race_grouped(ops, ref, 16, 16384, N, K, args.iters, args.warmup))
    if not args.quick:
        # many small experts: equal groups of one 256-row tile, and groups far below a tile
        emit(race_grouped(ops, ref, 128, 128 * 256, 4096, 4096, args.iters, args.warmup, equal=True))
        emit(race_grouped(ops, ref, 128, 128 * 64, 4096, 4096, args.iters, args.warmup, equal=True))
    emit(race_nvfp4(ops, ref, 8192, 8192, 8192, args.iters, args.warmup))
    for M in (1, 32):
        emit(race_nvfp4(ops, ref, M, 28672, 8192, 4 * args.iters, args.warmup))
    if hasattr(ref, "f4f4bf16_large_mx") and hasattr(torch, "float8_e8m0fnu"):
        emit(race_mxfp4(ops, ref, 8192, 8192, 8192, args.iters, args.warmup))
    if hasattr(ref, "f4f4bf16_grouped_stacked") and hasattr(torch, "float8_e8m0fnu"):
        for mx in (False, True):
            emit(race_grouped_fp4(ops, ref, 16, 16384, 16384, 5120, mx, args.iters, args.warmup))
        emit(race_kgrouped_mxfp4(ops, ref, 5120, 8192, [4096] * 4, args.iters, args.warmup))
        emit(race_kgrouped_mxfp4(ops, ref, 2048, 2048, [2048, 0, 6144, 992, 8192], args.iters, args.warmup))
    pyref = os.path.join(HERE, "_ref", "pyref")
    if os.path.isdir(pyref):
        os.environ["MSLK_PYTHON_ONLY"] = "1"
        sys.path.insert(0, pyref)
        for name in [m for m in sys.modules if m == "mslk" or m.startswith("mslk.")]:
            del sys.modules[name]
        from mslk.quantize.triton.fp8_quantize import triton_quantize_fp8_row
        for M, K in ((8192, 4096), (8192, 14336), (8192, 8192), (8192, 28672), (16384, 5120)):
            emit(race_quantize(ops, triton_quantize_fp8_row, M, K, args.iters, args.warmup))
    if args.out:
        os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
        with open(args.out, "w") as f:
            for r in lines:
                f.write(json.dumps(r) + "\n")
        with open(os.path.splitext(args.out)[0] + "_table.md", "w") as f:
            f.write("| case | this library | reference | speed ratio (>1: this library faster) | SM MHz (ours / ref) | output difference |\n")
            f.write("|---|---|---|---|---|---|\n")
            for r in lines:
                if "max_ulp" in r:
                    diff = "bit-identical" if r["max_ulp"] == 0 else \
                        f"max {r['max_ulp']} bf16 ulp, {100 * r['frac_equal']:.3f} % identical"
                else:
                    diff = "bytes and scales bit-identical" if r["bytes_equal"] and r["scales_equal"] else "DIFFERENT"
                inst = r.get("ref_instance") or r.get("ref_kernel", "").split(" ")[0]
                f.write(f"| {r['case']} | {r['ours_us']:.1f} us | {r['ref_us']:.1f} us (`{inst}`) | "
                        f"{r['ours_over_ref_speed']:.2f} | {r['ours_sm_mhz']} / {r['ref_sm_mhz']} | {diff} |\n")


if __name__ == "__main__":
    main()
