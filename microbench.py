"""Shape-level micro-benchmarks of the individual kernels (one JSON line per case).

    python microbench.py quantize_fp8_row --shape 8192,4096
    python microbench.py f8f8bf16_rowwise --shape 8192,8192,8192
    python microbench.py decode --graph                            # M = 1, 16, 32: general vs split-K kernel
    python microbench.py batched --shape 8,2048,4096,4096          # B,M,N,K
    python microbench.py grouped --experts 16 --tokens 16384 --shape 16384,5120   # N,K per expert
    python microbench.py f4f4bf16_grouped --experts 16 --tokens 16384 --shape 16384,5120   # N,K per expert
    python microbench.py f4f4bf16 --shape 8192,8192,8192
    python microbench.py quantize_nvfp4 --shape 8192,8192
    python microbench.py moe_gather_scatter --tokens 16384 --shape 5120,16,2      # D,E,top-k
    python microbench.py silu_mul_quant --shape 16384,14336      # T,D; also times the unfused pair
    python microbench.py sweep          # the Llama-3-8B sweep: M x (N,K), quantize + GEMM

Timing: CUDA events around `--iters` launches after `--warmup` launches, on torch's current
stream.  Inputs rotate through enough buffers to exceed the 126 MB L2 (`--rotate-mb`, default 512).
With `--graph` the launches are captured in one CUDA graph first, which removes the host launch
cost from small cases.  `--iters 1 --warmup 0 --rotate-mb 0` gives a minimal run to profile.
Synthetic data: activations bf16 ~N(0,1), weights ~N(0, --w-std).
"""

from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def _time(fn, n_variants, iters, warmup, graph):
    for i in range(warmup):
        fn(i % n_variants)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph:
        g = torch.cuda.CUDAGraph()
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            with torch.cuda.graph(g, stream=s):
                for i in range(iters):
                    fn(i % n_variants)
        g.replay()
        torch.cuda.synchronize()
        e0.record()
        g.replay()
        e1.record()
    else:
        e0.record()
        for i in range(iters):
            fn(i % n_variants)
        e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e-3  # seconds per launch


def _variants(bytes_per_variant, rotate_mb):
    if rotate_mb <= 0:
        return 1
    return max(1, min(16, math.ceil(rotate_mb * 1e6 / max(1, bytes_per_variant))))


def _randn(shape, std=1.0):
    return (torch.randn(shape, device="cuda", dtype=torch.float32) * std).to(torch.bfloat16)


def bench_quantize_fp8_row(ops, M, K, args):
    nv = _variants(M * K * 2, args.rotate_mb)
    xs = [_randn((M, K)) for _ in range(nv)]
    sec = _time(lambda i: ops.quantize_fp8_row(xs[i]), nv, args.iters, args.warmup, args.graph)
    byts = 3.0 * M * K + 4.0 * M
    return {"op": "quantize_fp8_row", "M": M, "K": K, "us": sec * 1e6, "GBps": byts / sec / 1e9, "bytes": byts}


def bench_f8f8bf16_rowwise(ops, M, N, K, args):
    nv = _variants(N * K, args.rotate_mb)
    xq, xs = ops.quantize_fp8_row(_randn((M, K)))
    ws = [ops.quantize_fp8_row(_randn((N, K), args.w_std)) for _ in range(nv)]
    y = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    sec = _time(lambda i: ops.f8f8bf16_rowwise_out(xq, ws[i][0], xs, ws[i][1], y), nv, args.iters, args.warmup, args.graph)
    flops = 2.0 * M * N * K
    byts = M * K + N * K + 2.0 * M * N + 4.0 * (M + N)
    return {"op": "f8f8bf16_rowwise", "M": M, "N": N, "K": K, "us": sec * 1e6, "TFLOPs": flops / sec / 1e12,
            "GBps": byts / sec / 1e9}


def bench_moe_gather_scatter(ops, T, D, E, topk, args):
    """Dispatch / combine around the grouped GEMM: a = T * topk rows gathered from T tokens, and added back."""
    a = T * topk
    g = torch.Generator(device="cuda").manual_seed(0)
    x = _randn((T, D))
    scores = torch.rand((T, E), generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    tok = (torch.randperm(a, generator=g, device="cuda") % T).to(torch.int32)
    ex = torch.randint(0, E, (a,), generator=g, device="cuda")
    out = []
    sec = _time(lambda i: ops.gather_scale_dense_tokens(x, tok, ex, scores), 1, args.iters, args.warmup, args.graph)
    out.append({"op": "gather_scale_dense_tokens", "T": T, "D": D, "a": a, "us": sec * 1e6, "GBps": 4.0 * a * D / sec / 1e9})
    sec = _time(lambda i: ops.gather_scale_quant_dense_tokens(x, tok, ex, scores), 1, args.iters, args.warmup, args.graph)
    out.append({"op": "gather_scale_quant_dense_tokens", "T": T, "D": D, "a": a, "us": sec * 1e6,
                "GBps": 3.0 * a * D / sec / 1e9})
    y = _randn((a, D))
    acc = torch.zeros((T, D), dtype=torch.bfloat16, device="cuda")
    sec = _time(lambda i: ops.scatter_add_dense_tokens(acc, y, tok), 1, args.iters, args.warmup, args.graph)
    # bytes: the rows read plus a read-modify-write of the destination rows
    out.append({"op": "scatter_add_dense_tokens", "T": T, "D": D, "a": a, "us": sec * 1e6,
                "GBps": (2.0 * a * D + 4.0 * a * D) / sec / 1e9})
    return out


def bench_silu_mul_quant(ops, T, D, args):
    nv = _variants(T * D * 4, args.rotate_mb)
    xs = [_randn((T, 2 * D)) for _ in range(nv)]
    sec = _time(lambda i: ops.silu_mul_quant(xs[i][:, :D], xs[i][:, D:]), nv, args.iters, args.warmup, args.graph)
    sec_unfused = _time(lambda i: ops.quantize_fp8_row(ops.silu_mul(xs[i][:, :D], xs[i][:, D:])), nv, args.iters,
                        args.warmup, args.graph)
    byts = 5.0 * T * D + 4.0 * T
    return {"op": "silu_mul_quant", "T": T, "D": D, "us": sec * 1e6, "GBps": byts / sec / 1e9, "bytes": byts,
            "unfused_silu_mul_then_quantize_us": sec_unfused * 1e6}


def bench_batched(ops, B, M, N, K, args):
    xq, xs = ops.quantize_fp8_row(_randn((B, M, K)))
    nv = _variants(B * N * K, args.rotate_mb)
    ws = [ops.quantize_fp8_row(_randn((B, N, K), args.w_std)) for _ in range(nv)]
    y = torch.empty((B, M, N), dtype=torch.bfloat16, device="cuda")
    sec = _time(lambda i: ops.f8f8bf16_rowwise_batched(xq, ws[i][0], xs, ws[i][1], output=y), nv, args.iters,
                args.warmup, args.graph)

    def loop(i):
        for b in range(B):
            ops.f8f8bf16_rowwise_out(xq[b], ws[i][0][b], xs[b], ws[i][1][b], y[b])
    sec_loop = _time(loop, nv, args.iters, args.warmup, args.graph)
    flops = 2.0 * B * M * N * K
    return {"op": "f8f8bf16_rowwise_batched", "B": B, "M": M, "N": N, "K": K, "us": sec * 1e6,
            "TFLOPs": flops / sec / 1e12, "loop_over_dense_us": sec_loop * 1e6,
            "loop_over_dense_TFLOPs": flops / sec_loop / 1e12}


def bench_decode(ops, M, N, K, args):
    """Few-token GEMM: the general kernel against the split-K weight-streaming kernel (caller-provided workspace)."""
    from mslk_b200._lib import check, lib
    nv = _variants(N * K, args.rotate_mb)
    xq, xs = ops.quantize_fp8_row(_randn((M, K)))
    ws = [ops.quantize_fp8_row(_randn((N, K), args.w_std)) for _ in range(nv)]
    y = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    sec = _time(lambda i: ops.f8f8bf16_rowwise_out(xq, ws[i][0], xs, ws[i][1], y), nv, args.iters, args.warmup, args.graph)
    nbytes = lib.mslk_b200_f8f8bf16_rowwise_workspace_bytes(M, N, K)
    work = torch.zeros((max(nbytes, 16),), dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream

    def split(i):
        check(lib.mslk_b200_f8f8bf16_rowwise_ws(xq.data_ptr(), ws[i][0].data_ptr(), xs.data_ptr(), ws[i][1].data_ptr(), None,
                                                0, y.data_ptr(), M, N, K, work.data_ptr(), nbytes, stream().cuda_stream),
              "f8f8bf16_rowwise_ws")
    sec_ws = _time(split, nv, args.iters, args.warmup, args.graph)
    byts = N * K + M * K + 2.0 * M * N
    return {"op": "f8f8bf16_rowwise few tokens", "M": M, "N": N, "K": K, "general_us": sec * 1e6,
            "general_GBps": byts / sec / 1e9, "split_k_us": sec_ws * 1e6, "split_k_GBps": byts / sec_ws / 1e9,
            "workspace_bytes": nbytes}


def zipf_counts(experts, tokens, seed=0, s=1.2, n_empty=2):
    """Per-expert token counts: top-1 routing with Zipf(s) expert popularity, the `n_empty` least popular
    experts forced to zero tokens (their tokens go to the most popular one)."""
    g = torch.Generator().manual_seed(seed)
    p = (torch.randperm(experts, generator=g).float() + 1) ** -s
    counts = torch.bincount(torch.multinomial(p / p.sum(), tokens, replacement=True, generator=g), minlength=experts)
    low = torch.argsort(p)[:n_empty]
    counts[torch.argmax(counts)] += counts[low].sum()
    counts[low] = 0
    return counts


def bench_grouped(ops, E, tokens, N, K, args):
    counts = zipf_counts(E, tokens)
    xq, xs = ops.quantize_fp8_row(_randn((tokens, K)))
    wq, ws = ops.quantize_fp8_row(_randn((E, N, K), args.w_std))
    ms = counts.to(torch.int64).cuda()
    sec = _time(lambda i: ops.f8f8bf16_rowwise_grouped_stacked(xq, wq, xs, ws.view(-1), ms), 1, args.iters,
                args.warmup, args.graph)
    # the same product with the combine fused in: rows added to a top-2 style destination
    g = torch.Generator(device="cuda").manual_seed(1)
    idx = (torch.randperm(tokens, generator=g, device="cuda") % max(tokens // 2, 1)).to(torch.int32)
    acc = torch.zeros((max(tokens // 2, 1), N), dtype=torch.bfloat16, device="cuda")
    sec_sc = _time(lambda i: ops.f8f8bf16_rowwise_grouped_stacked_scatter_add(xq, wq, xs, ws.view(-1), ms, acc, idx), 1,
                   args.iters, args.warmup, args.graph)
    flops = 2.0 * tokens * N * K
    return {"op": "f8f8bf16_rowwise_grouped_stacked", "E": E, "tokens": tokens, "N": N, "K": K,
            "counts": counts.tolist(), "us": sec * 1e6, "TFLOPs": flops / sec / 1e12,
            "with_scatter_add_us": sec_sc * 1e6, "with_scatter_add_TFLOPs": flops / sec_sc / 1e12}


def bench_f4f4bf16_grouped(ops, E, tokens, N, K, args):
    counts = zipf_counts(E, tokens)
    ms = counts.to(torch.int64).cuda()
    x = _randn((tokens, K))
    w = _randn((E * N, K), args.w_std)
    w_ms = torch.full((E,), N, dtype=torch.int64, device="cuda")
    x_gs, _ = ops.calculate_group_max(x, ms)
    w_gs, _ = ops.calculate_group_max(w, w_ms)
    sec_q = _time(lambda i: ops.nvfp4_quantize_stacked(ms, x, x_gs), 1, args.iters, args.warmup, args.graph)
    xq, xs = ops.nvfp4_quantize_stacked(ms, x, x_gs)
    wq, ws2 = ops.nvfp4_quantize_stacked(w_ms, w, w_gs)
    padded_n = (N + 127) // 128 * 128
    ws = ws2[: E * padded_n].view(E, padded_n, -1)
    alpha = torch.reciprocal(x_gs * w_gs)
    wq3 = wq.view(E, N, K // 2)
    sec = _time(lambda i: ops.f4f4bf16_grouped_stacked(xq, wq3, xs, ws, ms, alpha, None, use_mx=False), 1, args.iters,
                args.warmup, args.graph)
    flops = 2.0 * tokens * N * K
    return {"op": "f4f4bf16_grouped_stacked", "E": E, "tokens": tokens, "N": N, "K": K, "us": sec * 1e6,
            "TFLOPs": flops / sec / 1e12, "quantize_stacked_us": sec_q * 1e6,
            "quantize_stacked_GBps": tokens * K * 2.5625 / sec_q / 1e9, "counts": counts.tolist()}


def bench_quantize_nvfp4(ops, M, K, args):
    nv = _variants(M * K * 2, args.rotate_mb)
    xs = [_randn((M, K)) for _ in range(nv)]
    gs = (448.0 * 6.0) / xs[0].abs().amax().float()
    sec = _time(lambda i: ops.quantize_nvfp4(xs[i], gs), nv, args.iters, args.warmup, args.graph)
    byts = 2.0 * M * K + M * K / 2 + M * K / 16
    return {"op": "quantize_nvfp4", "M": M, "K": K, "us": sec * 1e6, "GBps": byts / sec / 1e9}


def bench_quantize_mx4(ops, M, K, args):
    nv = _variants(M * K * 2, args.rotate_mb)
    xs = [_randn((M, K)) for _ in range(nv)]
    out = []
    for group in (32, 16):
        sec = _time(lambda i: ops.quantize_mx4(xs[i], group), nv, args.iters, args.warmup, args.graph)
        byts = 2.0 * M * K + M * K / 2 + M * K / group
        out.append({"op": "quantize_mx4", "group": group, "M": M, "K": K, "us": sec * 1e6, "GBps": byts / sec / 1e9})
    return out


def bench_f4f4bf16_mx(ops, M, N, K, args):
    nv = _variants(N * K // 2, args.rotate_mb)
    xq, sx = ops.quantize_mx4(_randn((M, K)), 32)
    ws = [ops.quantize_mx4(_randn((N, K)), 32) for _ in range(nv)]
    y = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    sec = _time(lambda i: ops.f4f4bf16(xq, ws[i][0], sx, ws[i][1], output=y), nv, args.iters, args.warmup, args.graph)
    flops = 2.0 * M * N * K
    return {"op": "f4f4bf16 (MXFP4, block 32)", "M": M, "N": N, "K": K, "us": sec * 1e6, "TFLOPs": flops / sec / 1e12}


def bench_f4f4bf16(ops, M, N, K, args):
    nv = _variants(N * K // 2, args.rotate_mb)
    x = _randn((M, K))
    gx = (448.0 * 6.0) / x.abs().amax().float()
    xq, sx = ops.quantize_nvfp4(x, gx)
    ws = []
    for _ in range(nv):
        w = _randn((N, K))
        gw = (448.0 * 6.0) / w.abs().amax().float()
        wq, sw = ops.quantize_nvfp4(w, gw)
        ws.append((wq, sw, (1.0 / (gx * gw)).reshape(1)))
    y = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    sec = _time(lambda i: ops.f4f4bf16(xq, ws[i][0], sx, ws[i][1], output=y, global_scale=ws[i][2]), nv, args.iters,
                args.warmup, args.graph)
    flops = 2.0 * M * N * K
    byts = M * K / 2 + N * K / 2 + (M + N) * K / 16 + 2.0 * M * N
    return {"op": "f4f4bf16", "M": M, "N": N, "K": K, "us": sec * 1e6, "TFLOPs": flops / sec / 1e12,
            "GBps": byts / sec / 1e9}


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("op", choices=["quantize_fp8_row", "f8f8bf16_rowwise", "decode", "batched", "grouped", "f4f4bf16", "f4f4bf16_grouped", "moe_gather_scatter", "quantize_nvfp4", "quantize_mx4", "f4f4bf16_mx", "silu_mul_quant",
                                   "sweep"])
    ap.add_argument("--shape", default=None, help="comma-separated sizes (see module docstring)")
    ap.add_argument("--experts", type=int, default=16)
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--rotate-mb", type=float, default=512.0)
    ap.add_argument("--w-std", type=float, default=0.02)
    ap.add_argument("--graph", action="store_true")
    args = ap.parse_args()
    from mslk_b200 import ops
    from mslk_b200._lib import device_status
    shape = [int(v) for v in args.shape.split(",")] if args.shape else None
    out = []
    if args.op == "quantize_fp8_row":
        out.append(bench_quantize_fp8_row(ops, *(shape or [8192, 4096]), args))
    elif args.op == "f8f8bf16_rowwise":
        out.append(bench_f8f8bf16_rowwise(ops, *(shape or [8192, 8192, 8192]), args))
    elif args.op == "decode":
        for M in ((shape[0],) if shape else (1, 16, 32)):
            for N, K in (((shape[1], shape[2]),) if shape else ((6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336))):
                out.append(bench_decode(ops, M, N, K, args))
    elif args.op == "batched":
        out.append(bench_batched(ops, *(shape or [8, 2048, 4096, 4096]), args))
    elif args.op == "grouped":
        out.append(bench_grouped(ops, args.experts, args.tokens, *(shape or [16384, 5120]), args))
    elif args.op == "quantize_nvfp4":
        out.append(bench_quantize_nvfp4(ops, *(shape or [8192, 8192]), args))
    elif args.op == "quantize_mx4":
        out.extend(bench_quantize_mx4(ops, *(shape or [8192, 8192]), args))
    elif args.op == "f4f4bf16_grouped":
        out.append(bench_f4f4bf16_grouped(ops, args.experts, args.tokens, *(shape or [16384, 5120]), args))
    elif args.op == "moe_gather_scatter":
        out.extend(bench_moe_gather_scatter(ops, args.tokens, *(shape or [5120, 16, 2]), args))
    elif args.op == "silu_mul_quant":
        out.append(bench_silu_mul_quant(ops, *(shape or [16384, 14336]), args))
    elif args.op == "f4f4bf16_mx":
        out.append(bench_f4f4bf16_mx(ops, *(shape or [8192, 8192, 8192]), args))
    elif args.op == "f4f4bf16":
        out.append(bench_f4f4bf16(ops, *(shape or [8192, 8192, 8192]), args))
    else:
        for M in (1, 16, 128, 2048, 8192):
            for N, K in ((6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)):
                out.append(bench_quantize_fp8_row(ops, M, K, args))
                out.append(bench_f8f8bf16_rowwise(ops, M, N, K, args))
    status = device_status()
    for r in out:
        r["device_status"] = status
        print(json.dumps(r), flush=True)


if __name__ == "__main__":
    main()
