"""Multi-GPU benchmark of the sharded configurations (one process per GPU, NCCL).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node P --master-addr 127.0.0.1 --master-port 29511 \
        -m mslk_b200.tp_bench [--workload ffn70b|moe|all] [--steps K] [--warmup W] [--chunks C]

ffn70b  Llama-3-70B FFN at M = 8192 tokens: gate+up (N = 57344, K = 8192) with the weight rows sharded
        and an all-gather of the bf16 output; down (N = 8192, K = 28672) with K sharded and a
        reduce-scatter of the partial products.  Reported: TFLOP/s of the GEMMs alone and of GEMM +
        collective (whole job: 2*M*N*K of the unsharded problem / max-over-ranks time).
moe     16 experts (hidden 5120, FFN 8192), 16384 tokens with Zipf(1.2) counts; experts sharded
        contiguously over the ranks, no collective; whole-job TFLOP/s = total flops / slowest rank.

Times are CUDA events on each rank, maximum over ranks.  Synthetic seeded data.  With P = 1 the same
code runs unsharded (no collective).
"""

from __future__ import annotations

import argparse
import json
import os

os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer stores only; no multicast binding

import torch
import torch.distributed as dist

M_TOKENS = 8192


def _max_ms(ms: float, device) -> float:
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _timed(fn, steps, warmup, device):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if dist.is_initialized():
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return _max_ms(e0.elapsed_time(e1) / steps, device)


def _randn(shape, gen, std=1.0):
    return (torch.randn(shape, generator=gen, device=gen.device, dtype=torch.float32) * std).to(torch.bfloat16)


def bench_ffn70b(ops, par, rank, world, device, args):
    g = torch.Generator(device=device).manual_seed(0)      # same seed on every rank: replicated activations
    out = {}
    # ---- gate+up: N-sharded, all-gather of the output
    N, K = 57344, 8192
    x = _randn((M_TOKENS, K), g)
    xq, xs = ops.quantize_fp8_row(x)
    n0, n1 = par.shard_range(N, rank, world)
    gw = torch.Generator(device=device).manual_seed(100 + rank)
    wq, ws = ops.quantize_fp8_row(_randn((n1 - n0, K), gw, 0.01))
    col = par.ColumnParallelLinear(wq, ws, ops.f8f8bf16_rowwise, chunks=args.chunks)
    flops = 2.0 * M_TOKENS * N * K
    ms_gemm = _timed(lambda: col.local(xq, xs), args.steps, args.warmup, device)
    ms_full = _timed(lambda: col.forward(xq, xs), args.steps, args.warmup, device)
    out["gate_up"] = {"N": N, "K": K, "sharding": f"N/{world} + all-gather", "gemm_ms": ms_gemm,
                      "gemm_tflops": flops / ms_gemm / 1e9, "with_collective_ms": ms_full,
                      "with_collective_tflops": flops / ms_full / 1e9, "chunks": args.chunks,
                      "gathered_bytes_per_gpu": (world - 1) * M_TOKENS * (N // world) * 2}
    # ---- same, fused: the GEMM epilogue stores its column block into every rank's output buffer
    if world > 1:
        import torch.distributed._symmetric_memory as symm_mem
        y_ref = col.forward(xq, xs).clone()
        y_sym = symm_mem.empty((M_TOKENS, N), dtype=torch.bfloat16, device=device)
        hdl = symm_mem.rendezvous(y_sym, dist.group.WORLD)
        ptrs = list(hdl.buffer_ptrs)

        def fused():
            ops.f8f8bf16_rowwise_allgather(xq, wq, xs, ws, ptrs, rank, y_sym)
            hdl.barrier()          # all ranks' stores have landed before anyone reads

        y_sym.zero_()
        hdl.barrier()
        fused()
        torch.cuda.synchronize()
        same = bool(torch.equal(y_sym, y_ref))
        ms_fused = _timed(fused, args.steps, args.warmup, device)
        out["gate_up"].update({"fused_epilogue_allgather_ms": ms_fused,
                               "fused_epilogue_allgather_tflops": flops / ms_fused / 1e9,
                               "fused_matches_nccl_path": same})
        del y_sym, hdl, y_ref
    del col, wq, ws, x, xq
    torch.cuda.empty_cache()
    # ---- down: K-sharded, reduce-scatter of the partials
    N, K = 8192, 28672
    x = _randn((M_TOKENS, K), g)
    xq, xs = ops.quantize_fp8_row(x)                        # scales over the FULL row
    xq_k = par.shard_k(xq, rank, world)
    del x, xq
    gw = torch.Generator(device=device).manual_seed(200)    # full weight on every rank, then sharded over K
    k0, k1 = par.shard_range(K, rank, world)
    w = _randn((N, K), gw, 0.01)
    wq, ws = ops.quantize_fp8_row(w)
    del w
    wq_k = wq[:, k0:k1].contiguous()
    del wq
    row = par.RowParallelLinear(wq_k, ws, ops.f8f8bf16_rowwise)
    flops = 2.0 * M_TOKENS * N * K
    ms_gemm = _timed(lambda: row.local(xq_k, xs), args.steps, args.warmup, device)
    ms_full = _timed(lambda: row.forward(xq_k, xs), args.steps, args.warmup, device)
    out["down"] = {"N": N, "K": K, "sharding": f"K/{world} + reduce-scatter (bf16 partials)", "gemm_ms": ms_gemm,
                   "gemm_tflops": flops / ms_gemm / 1e9, "with_collective_ms": ms_full,
                   "with_collective_tflops": flops / ms_full / 1e9,
                   "scattered_bytes_per_gpu": (world - 1) * (M_TOKENS // world) * N * 2}
    # ---- same, fused: partial rows leave the epilogue straight into the owners' staging slots
    if world > 1:
        import torch.distributed._symmetric_memory as symm_mem
        rows = M_TOKENS // world
        # fp32 reference of the unsharded product for this rank's rows: all-reduce of fp32 partials
        ref = (xq_k.float() @ wq_k.float().T) * xs[:, None] * ws[None, :]
        dist.all_reduce(ref)
        ref = ref[rank * rows:(rank + 1) * rows]
        y_nccl = row.forward(xq_k, xs).float()
        # two staging buffers used alternately: one cross-rank barrier per call is then enough (a slot
        # is rewritten two calls later, after its owner's reduction has been passed by a barrier)
        stages, handles = [], []
        for _ in range(2):
            st = symm_mem.empty((world, rows, N), dtype=torch.bfloat16, device=device)
            handles.append(symm_mem.rendezvous(st, dist.group.WORLD))
            stages.append(st)
        y_out = torch.empty((rows, N), dtype=torch.bfloat16, device=device)
        turn = [0]

        def fused():
            i = turn[0] & 1
            turn[0] += 1
            ops.f8f8bf16_rowwise_scatter(xq_k, wq_k, xs, ws, list(handles[i].buffer_ptrs), rank)
            handles[i].barrier()                # every rank's partial rows have landed
            ops.reduce_slots(stages[i], y_out)

        fused()
        torch.cuda.synchronize()
        scale = max(1.0, float(ref.std()))
        ms_fused = _timed(fused, args.steps, args.warmup, device)
        torch.cuda.synchronize()
        out["down"].update({
            "fused_epilogue_scatter_ms": ms_fused, "fused_epilogue_scatter_tflops": flops / ms_fused / 1e9,
            "fused_within_tolerance_of_fp32_reference": bool(torch.allclose(y_out.float(), ref, rtol=1.6e-2, atol=1e-2 * scale)),
            "max_abs_err_vs_fp32_reference": {"fused": float((y_out.float() - ref).abs().max()),
                                              "nccl_bf16_reduce_scatter": float((y_nccl - ref).abs().max())}})
        del stages, handles, ref
    return out


def bench_moe(ops, par, rank, world, device, args):
    from .microbench import zipf_counts
    E, tokens = 16, 16384
    counts = zipf_counts(E, tokens).tolist()
    row0, row1, (e0, e1) = par.expert_token_range(counts, rank, world)
    g = torch.Generator(device=device).manual_seed(300 + rank)
    ms_local = torch.tensor(counts[e0:e1], dtype=torch.int64, device=device)
    out = {"counts": counts, "experts_per_gpu": e1 - e0, "tokens_this_rank0": row1 - row0 if rank == 0 else None}
    for name, N, K in (("gate_up", 16384, 5120), ("down", 5120, 8192)):
        xq, xs = ops.quantize_fp8_row(_randn((max(row1 - row0, 1), K), g))
        xq, xs = xq[: row1 - row0], xs[: row1 - row0]
        wq, ws = ops.quantize_fp8_row(_randn((e1 - e0, N, K), g, 0.02))
        ms = _timed(lambda: ops.f8f8bf16_rowwise_grouped_stacked(xq, wq, xs, ws.view(-1), ms_local),
                    args.steps, args.warmup, device)
        flops = 2.0 * tokens * N * K
        out[name] = {"N": N, "K": K, "ms_slowest_rank": ms, "tflops_whole_job": flops / ms / 1e9}
        del xq, wq
        torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", choices=["ffn70b", "moe", "all"], default="all")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--chunks", type=int, default=4)
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    from . import ops, parallel as par
    from ._lib import device_status
    res = {"n_gpus": world, "tokens": M_TOKENS, "steps": args.steps, "warmup": args.warmup, "data": "synthetic"}
    if args.workload in ("ffn70b", "all"):
        res["ffn70b"] = bench_ffn70b(ops, par, rank, world, device, args)
    if args.workload in ("moe", "all"):
        res["moe"] = bench_moe(ops, par, rank, world, device, args)
    res["device_status"] = device_status()
    if rank == 0:
        print(json.dumps(res), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
