#!/usr/bin/env python
"""Benchmark of the FP8-rowwise hot path (per-row quantize -> rowwise-scaled FP8 GEMM) on 1..8 B200s.

Headline workload at every GPU count: the Llama-3-70B FFN projections at M = 8192 tokens, tensor-parallel
over the N GPUs of one node (one process per GPU, NCCL / NVLink):

  gate+up  (N = 57344, K = 8192): the bf16 activation is quantized per row (replicated on every rank), the
           weight rows are sharded over the ranks, every rank multiplies its [57344/P, 8192] shard and the
           bf16 outputs are all-gathered, so every rank ends with the full [8192, 57344] result;
  down     (N = 8192, K = 28672): K is sharded -- the activation is quantized over the FULL rows beforehand
           and every rank holds its [:, K/P] byte slices (input preparation, as the weights) -- every rank
           multiplies its slices and the scaled partial products are reduce-scattered over the token
           dimension, so rank r ends with rows [r*M/P, (r+1)*M/P) of the sum.

`value` = flops of the UNSHARDED problem (2*M*N*K of both projections) / time of a step on the slowest
rank: strong scaling.  The collectives are part of the step.  By default the step uses this library's
fused epilogues where they are faster than NCCL (the GEMM's epilogue stores its tiles into the peers'
buffers over NVLink while the tensor cores work) and NCCL elsewhere; the same step with the plain NCCL
collectives (`all_gather_into_tensor`, `reduce_scatter_tensor`) and the GEMMs alone are reported beside it
under `tp`.  At N = 1 the step is the two unsharded GEMMs (+ the quantizer).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

prints ONE JSON line (rank 0).  `--impl reference` times the reference's CPU path (torch per-row quantize +
dequantize / fp32 matmul, as its tests do) on the host cores, on a bounded sample of the same workload.
Extra sections: `roofline` (dominant kernel = the tcgen05 GEMM), `e2e`, `clocks`, `tp`, `moe_expert_sharded`,
and at N = 1 `cpu_baseline`, `sustained`, `llama3_8b_step`, `configs` (the other BASELINE configurations,
each with its own roofline) and `reference_gpu` (the reference's own sm_100 kernels when baseline/_ref holds them).
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time

os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # peer traffic = plain stores; nothing binds a multicast object

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FFN_TOKENS = 8192
GATE_UP = (57344, 8192)
DOWN = (8192, 28672)
CPU_SAMPLE_TOKENS = 256
LLAMA8B_PROJECTIONS = [("qkv", 6144, 4096), ("o", 4096, 4096), ("gate_up", 28672, 4096), ("down", 4096, 14336)]
SM_INGEST_TBS = 13.0           # TB/s from L2 into the SMs: what ncu counted on the FP8 and both FP4 pair kernels at 8192^3
NOMINAL_FP8_TFLOPS = 4500.0
NOMINAL_FP4_TFLOPS = 9000.0
NOMINAL_HBM_GBS = 8000.0
NVLINK_PEER_GBS = 770.0        # measured peer-copy rate per direction per GPU on this pool


def ffn_flops(tokens=FFN_TOKENS):
    return 2.0 * tokens * (GATE_UP[0] * GATE_UP[1] + DOWN[0] * DOWN[1])


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_burst": float(p["bf16_tflops"]),
                "bf16_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


def load_traffic():
    """DRAM bytes per launch of the headline GEMM launches, from the ncu capture summarised under profiles/
    (`key = value` lines); {} when the summary is absent."""
    path = os.path.join(ROOT, "profiles", "bench_gemm_dram_traffic__ffn70b_step.txt")
    out = {}
    if os.path.exists(path):
        for line in open(path):
            if "=" in line and not line.lstrip().startswith("#"):
                k, v = line.split("=", 1)
                try:
                    out[k.strip()] = float(v.split()[0])
                except (ValueError, IndexError):
                    pass
    return out


class ClockSampler:
    """Samples SM clock, power and throttle reasons of one GPU with `nvidia-smi -lms` in a child
    process while the timed region runs (a thread in this process would be starved by the launch loop)."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None

    def start(self):
        import subprocess
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            # the child needs up to a few seconds to open NVML on a box with eight GPUs: wait for its first line, so
            # that it is sampling when the timed region starts
            import select
            self.first = ""
            if select.select([self.proc.stdout], [], [], 8.0)[0]:
                self.first = self.proc.stdout.readline()
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            out = self.proc.communicate(timeout=5)[0]
        except Exception:
            out = ""
        clocks, powers, reasons, max_mhz = [], [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in (getattr(self, "first", "") + out).strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                clocks.append(int(float(f[0])))
                max_mhz = int(float(f[1]))
                powers.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v == "Active":
                    reasons.add(n)
        # "under load" = samples whose power draw is above half of the largest seen
        busy = [c for c, p in zip(clocks, powers) if powers and p >= 0.5 * max(powers)]
        busy.sort()
        return {"sm_mhz": (busy[len(busy) // 2] if busy else None), "sm_max_mhz": max_mhz,
                "reasons": sorted(reasons), "samples": len(clocks), "samples_under_load": len(busy),
                "power_w_max": (max(powers) if powers else None)}


def _randn(shape, gen, std=1.0):
    return (torch.randn(shape, generator=gen, device=gen.device, dtype=torch.float32) * std).to(torch.bfloat16)


def _ev():
    return torch.cuda.Event(enable_timing=True)


class Dist:
    """The little of torch.distributed the benchmark needs, degenerate at world size 1."""

    def __init__(self, world, device):
        self.world, self.device = world, device

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def max(self, value: float) -> float:
        if self.world == 1:
            return float(value)
        import torch.distributed as dist
        t = torch.tensor([value], dtype=torch.float64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(self, fn, steps, warmup):
        """ms per call of `fn`: CUDA events on the current stream, barrier + synchronize on both sides, max over ranks."""
        for _ in range(warmup):
            fn()
        self.barrier()
        e0, e1 = _ev(), _ev()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        self.barrier()
        return self.max(e0.elapsed_time(e1) / steps)


class FfnTensorParallel:
    """Operands, buffers and the step variants of the tensor-parallel Llama-3-70B FFN projections."""

    def __init__(self, ops, par, rank, world, device):
        import torch.distributed as dist
        self.ops, self.par, self.rank, self.world, self.device = ops, par, rank, world, device
        M, P = FFN_TOKENS, world
        g = torch.Generator(device=device).manual_seed(0)         # same seed on every rank: replicated activations
        # ---- gate+up: replicated bf16 activation, weight rows sharded
        N, K = GATE_UP
        self.x1 = _randn((M, K), g)
        n0, n1 = par.shard_range(N, rank, world)
        gw = torch.Generator(device=device).manual_seed(100 + rank)
        self.wq1, self.ws1 = ops.quantize_fp8_row(_randn((n1 - n0, K), gw, 0.01))
        # ---- down: activation quantized over the full rows, then the byte slices of this rank
        N2, K2 = DOWN
        xq2, self.xs2 = ops.quantize_fp8_row(_randn((M, K2), g))
        self.xq2_k = par.shard_k(xq2, rank, world)
        del xq2
        gw2 = torch.Generator(device=device).manual_seed(200)     # the full weight on every rank, then its K slice
        wq2, self.ws2 = ops.quantize_fp8_row(_randn((N2, K2), gw2, 0.01))
        self.wq2_k = par.shard_k(wq2, rank, world)
        del wq2
        torch.cuda.empty_cache()
        self.rows = M // P
        self.col = par.ColumnParallelLinear(self.wq1, self.ws1, ops.f8f8bf16_rowwise, chunks=1)
        self.row = par.RowParallelLinear(self.wq2_k, self.ws2, ops.f8f8bf16_rowwise)
        self.y2 = torch.empty((self.rows, N2), dtype=torch.bfloat16, device=device)
        self.partial = torch.empty((M, N2), dtype=torch.bfloat16, device=device)
        self.fused_down = False
        if P > 1:
            import torch.distributed._symmetric_memory as symm_mem
            self.y1 = symm_mem.empty((M, N), dtype=torch.bfloat16, device=device)
            self.h1 = symm_mem.rendezvous(self.y1, dist.group.WORLD)
            self.p1 = list(self.h1.buffer_ptrs)
            # two staging buffers used alternately: one cross-rank barrier per call is then enough (a slot is
            # rewritten two calls later, after its owner's reduction has been passed by a barrier)
            self.stages, self.hs = [], []
            for _ in range(2):
                st = symm_mem.empty((P, self.rows, N2), dtype=torch.bfloat16, device=device)
                self.hs.append(symm_mem.rendezvous(st, dist.group.WORLD))
                self.stages.append(st)
            self.turn = 0
            self.gathered = torch.empty((P * M, n1 - n0), dtype=torch.bfloat16, device=device)
            self.y_local = torch.empty((M, n1 - n0), dtype=torch.bfloat16, device=device)
        else:
            self.y1 = torch.empty((M, N), dtype=torch.bfloat16, device=device)
            self.y_local = self.y1

    # ---------------------------------------------------------------- pieces
    def quantize(self):
        return self.ops.quantize_fp8_row(self.x1)

    def gate_up_gemm_only(self, xq, xs):
        self.ops.f8f8bf16_rowwise_out(xq, self.wq1, xs, self.ws1, self.y_local)
        return self.y_local

    def gate_up_fused(self, xq, xs):
        if self.world == 1:
            self.ops.f8f8bf16_rowwise_out(xq, self.wq1, xs, self.ws1, self.y1)
        else:
            self.ops.f8f8bf16_rowwise_allgather(xq, self.wq1, xs, self.ws1, self.p1, self.rank, self.y1)
            self.h1.barrier()          # every rank's column blocks have landed before anyone reads them
        return self.y1

    def gate_up_nccl(self, xq, xs):
        import torch.distributed as dist
        if self.world == 1:
            self.ops.f8f8bf16_rowwise_out(xq, self.wq1, xs, self.ws1, self.y1)
            return self.y1
        M, P, nl = xq.shape[0], self.world, self.wq1.shape[0]
        dist.all_gather_into_tensor(self.gathered, self.gate_up_gemm_only(xq, xs))
        # [P, M, N/P] rank-major -> columns of the row-major [M, N] result
        self.y1.view(M, P, nl).copy_(self.gathered.view(P, M, nl).permute(1, 0, 2))
        return self.y1

    def down_gemm_only(self):
        self.ops.f8f8bf16_rowwise_out(self.xq2_k, self.wq2_k, self.xs2, self.ws2, self.partial)
        return self.partial

    def down_fused(self):
        if self.world == 1:
            self.ops.f8f8bf16_rowwise_out(self.xq2_k, self.wq2_k, self.xs2, self.ws2, self.y2)
            return self.y2
        i = self.turn & 1
        self.turn += 1
        self.ops.f8f8bf16_rowwise_scatter(self.xq2_k, self.wq2_k, self.xs2, self.ws2, list(self.hs[i].buffer_ptrs), self.rank)
        self.hs[i].barrier()                 # every rank's partial rows have landed
        self.ops.reduce_slots(self.stages[i], self.y2)
        return self.y2

    def down_nccl(self):
        import torch.distributed as dist
        if self.world == 1:
            self.ops.f8f8bf16_rowwise_out(self.xq2_k, self.wq2_k, self.xs2, self.ws2, self.y2)
            return self.y2
        self.down_gemm_only()
        dist.reduce_scatter_tensor(self.y2, self.partial, op=dist.ReduceOp.SUM)
        return self.y2

    # ---------------------------------------------------------------- steps
    def step(self, ev=None):
        """The product path: quantize, gate+up with the fused all-gather, down with the faster of the fused
        scatter + slot sum and NCCL's reduce-scatter (chosen once from a timing at set-up)."""
        xq, xs = self.quantize()
        if ev is not None:
            ev[0].record()
        self.gate_up_fused(xq, xs)
        if ev is not None:
            ev[1].record()
        if self.fused_down:
            self.down_fused()
        else:
            self.down_nccl()
        if ev is not None:
            ev[2].record()

    def step_nccl(self):
        xq, xs = self.quantize()
        self.gate_up_nccl(xq, xs)
        self.down_nccl()

    def step_gemm_only(self):
        xq, xs = self.quantize()
        self.gate_up_gemm_only(xq, xs)
        self.down_gemm_only()

    def launches_per_step(self):
        # this library's kernels: quantize, gate+up GEMM, down GEMM (+ the slot sum of the fused reduce-scatter)
        return 3 + (1 if (self.world > 1 and self.fused_down) else 0)


def tp_breakdown(tp, dd, steps, warmup):
    """GEMM alone / with NCCL / with the fused epilogue for both projections (ms = slowest rank), bytes that
    cross NVLink per GPU, and the NVLink roofline of the fused kernels."""
    M, P = FFN_TOKENS, tp.world
    xq, xs = tp.quantize()
    out = {}
    f1 = 2.0 * M * GATE_UP[0] * GATE_UP[1]
    f2 = 2.0 * M * DOWN[0] * DOWN[1]
    g1 = dd.timed(lambda: tp.gate_up_gemm_only(xq, xs), steps, warmup)
    g2 = dd.timed(tp.down_gemm_only, steps, warmup)
    out["gate_up"] = {"sharding": f"N/{P}" + (" + all-gather of the bf16 output" if P > 1 else ""),
                      "gemm_only_ms": g1, "gemm_only_tflops": f1 / g1 / 1e9}
    out["down"] = {"sharding": f"K/{P}" + (" + reduce-scatter of the bf16 partial products" if P > 1 else ""),
                   "gemm_only_ms": g2, "gemm_only_tflops": f2 / g2 / 1e9}
    if P > 1:
        n1 = dd.timed(lambda: tp.gate_up_nccl(xq, xs), steps, warmup)
        u1 = dd.timed(lambda: tp.gate_up_fused(xq, xs), steps, warmup)
        n2 = dd.timed(tp.down_nccl, steps, warmup)
        u2 = dd.timed(tp.down_fused, steps, warmup)
        ag_bytes = (P - 1) * M * (GATE_UP[0] // P) * 2        # sent (and received) per GPU
        rs_bytes = (P - 1) * (M // P) * DOWN[0] * 2
        peaks = load_peaks()
        t_flops1 = f1 / P / (2.0 * peaks["bf16_burst"] * 1e12) * 1e3
        t_link1 = ag_bytes / (NVLINK_PEER_GBS * 1e9) * 1e3
        t_flops2 = f2 / P / (2.0 * peaks["bf16_burst"] * 1e12) * 1e3
        t_link2 = rs_bytes / (NVLINK_PEER_GBS * 1e9) * 1e3
        out["gate_up"].update({
            "nccl_all_gather_ms": n1, "nccl_all_gather_tflops": f1 / n1 / 1e9,
            "fused_epilogue_ms": u1, "fused_epilogue_tflops": f1 / u1 / 1e9,
            "nvlink_bytes_per_gpu": ag_bytes, "fused_nvlink_gbs_per_gpu": ag_bytes / u1 / 1e6,
            "roofline_ms": max(t_flops1, t_link1), "roofline_frac": max(t_flops1, t_link1) / u1,
            "limiter": "NVLink ingress/egress of the all-gather" if t_link1 > t_flops1 else "tensor cores"})
        out["down"].update({
            "nccl_reduce_scatter_ms": n2, "nccl_reduce_scatter_tflops": f2 / n2 / 1e9,
            "fused_epilogue_ms": u2, "fused_epilogue_tflops": f2 / u2 / 1e9,
            "nvlink_bytes_per_gpu": rs_bytes, "fused_nvlink_gbs_per_gpu": rs_bytes / u2 / 1e6,
            "roofline_ms": max(t_flops2, t_link2), "roofline_frac": max(t_flops2, t_link2) / min(u2, n2),
            "limiter": "NVLink" if t_link2 > t_flops2 else "tensor cores (+ launch latency of the dependent steps)"})
        # the fused placements must reproduce the NCCL path: bit-identical for the all-gather (same kernel, other
        # addresses); the reduce-scatter sums bf16 partials in fp32 in rank order, NCCL in bf16 in ring order
        y_n = tp.gate_up_nccl(xq, xs).clone()
        y_f = tp.gate_up_fused(xq, xs)
        torch.cuda.synchronize()
        out["gate_up"]["fused_matches_nccl_path"] = bool(torch.equal(y_n, y_f))
        del y_n
        d_n = tp.down_nccl().float().clone()
        d_f = tp.down_fused().float()
        torch.cuda.synchronize()
        # both paths add P bf16 partial products; NCCL's ring rounds to bf16 after every hop, so two correct results
        # differ by up to P roundings at the magnitude of the partial sums: P * 2^-8 * max|partial| (+ 2^-7 relative)
        pmax = dd.max(float(tp.partial.abs().max()))
        atol = P * 2.0 ** -8 * pmax
        out["down"]["fused_within_tolerance_of_nccl_path"] = bool(torch.allclose(d_f, d_n, rtol=2.0 ** -7, atol=atol))
        out["down"]["fused_max_abs_diff_vs_nccl"] = float((d_f - d_n).abs().max())
        out["down"]["tolerance_abs"] = atol
    return out


def moe_expert_sharded(ops, par, dd, rank, world, device, steps, warmup):
    """configs: 16 experts (hidden 5120, FFN 8192), 16384 tokens, Zipf(1.2) counts with empty experts; experts
    sharded over the ranks, tokens bucketed per rank, no collective.  Whole-job TFLOP/s = total flops / slowest
    rank, for contiguous expert ranges and for the token-count-aware placement."""
    from microbench import zipf_counts
    E, tokens = 16, 16384
    counts = zipf_counts(E, tokens).tolist()
    placements = {"contiguous": [list(range(*par.expert_slice(E, r, world))) for r in range(world)]}
    if world > 1:
        placements["balanced"] = par.balanced_expert_assignment(counts, world)[0]
    out = {"counts": counts, "experts": E, "tokens": tokens}
    for pname, experts_of in placements.items():
        mine = experts_of[rank]
        loads = [sum(counts[e] for e in ex) for ex in experts_of]
        n_tok = loads[rank]
        ms_local = torch.tensor([counts[e] for e in mine] or [0], dtype=torch.int64, device=device)
        g = torch.Generator(device=device).manual_seed(300 + rank)
        res = {"experts_of_rank": experts_of, "tokens_of_rank": loads,
               "bound_tokens_on_one_rank": max(max(counts), -(-tokens // world)),
               "efficiency_bound": tokens / (world * max(max(counts), -(-tokens // world)))}
        for name, N, K in (("gate_up", 16384, 5120), ("down", 5120, 8192)):
            xq, xs = ops.quantize_fp8_row(_randn((max(n_tok, 1), K), g))
            xq, xs = xq[:n_tok], xs[:n_tok]
            wq, ws = ops.quantize_fp8_row(_randn((max(len(mine), 1), N, K), g, 0.02))
            if n_tok == 0:
                fn = lambda: None
            else:
                fn = lambda: ops.f8f8bf16_rowwise_grouped_stacked(xq, wq, xs, ws.view(-1), ms_local)
            ms = dd.timed(fn, steps, warmup)
            res[name] = {"N": N, "K": K, "ms_slowest_rank": ms, "tflops_whole_job": 2.0 * tokens * N * K / ms / 1e9}
            del xq, wq
            torch.cuda.empty_cache()
        out[pname] = res
    return out


# ----------------------------------------------------------------------------- N = 1 extras

def llama3_8b_step(ops, device, steps, warmup):
    """The Llama-3-8B layer projections at M = 8192 (quantize_fp8_row + f8f8bf16_rowwise for each of the four)."""
    M = 8192
    g = torch.Generator(device=device).manual_seed(0)
    layers = []
    for name, n, k in LLAMA8B_PROJECTIONS:
        x = _randn((M, k), g)
        wq, ws = ops.quantize_fp8_row(_randn((n, k), g, 0.02))
        layers.append({"name": name, "n": n, "k": k, "x": x, "wq": wq, "ws": ws,
                       "y": torch.empty((M, n), dtype=torch.bfloat16, device=device)})

    def step(ev=None):
        for i, L in enumerate(layers):
            if ev is not None:
                ev[i][0].record()
            xq, xs = ops.quantize_fp8_row(L["x"])
            if ev is not None:
                ev[i][1].record()
            ops.f8f8bf16_rowwise_out(xq, L["wq"], xs, L["ws"], L["y"])
            if ev is not None:
                ev[i][2].record()

    for _ in range(max(warmup, 3)):
        step()
    torch.cuda.synchronize()
    ev = [[[_ev() for _ in range(3)] for _ in layers] for _ in range(steps)]
    e0, e1 = _ev(), _ev()
    e0.record()
    for s in range(steps):
        step(ev[s])
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    flops = sum(2.0 * M * L["n"] * L["k"] for L in layers)
    q_ms = [sum(ev[s][i][0].elapsed_time(ev[s][i][1]) for s in range(steps)) / steps for i in range(len(layers))]
    g_ms = [sum(ev[s][i][1].elapsed_time(ev[s][i][2]) for s in range(steps)) / steps for i in range(len(layers))]
    return {"workload": "llama3-8b layer projections, M=8192: quantize_fp8_row + f8f8bf16_rowwise for (N,K) in "
                        "(6144,4096),(4096,4096),(28672,4096),(4096,14336)",
            "tflops": flops / ms / 1e9, "ms_per_step": ms, "gemm_kernels_tflops": flops / sum(g_ms) / 1e9,
            "step_over_gemm_kernels": sum(g_ms) / ms,
            "shapes": [{"name": L["name"], "N": L["n"], "K": L["k"], "gemm_ms": g_ms[i],
                        "gemm_tflops": 2.0 * M * L["n"] * L["k"] / g_ms[i] / 1e9, "quant_ms": q_ms[i]}
                       for i, L in enumerate(layers)]}


def _time_graph(fn, rounds):
    """ms per call of `fn` replayed `rounds` times from one CUDA graph (removes the host's launch gaps)."""
    fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(rounds):
            fn()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = _ev(), _ev()
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / rounds


def _time_plain(fn, iters, warmup=3):
    """ms per call over `iters` launches after `warmup`; half a second of idle first, so that every extra configuration
    starts from the same power state instead of inheriting the throttled clock of the one measured before it."""
    torch.cuda.synchronize()
    time.sleep(0.5)
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = _ev(), _ev()
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def other_configs(ops, device, peaks):
    """The other BASELINE configurations on one GPU, each with its own roofline object."""
    out = {}
    fp8_peak = 2.0 * peaks["bf16_burst"]
    g = torch.Generator(device=device).manual_seed(0)

    def tensor_roof(flops, ms, peak, nominal):
        a = flops / ms / 1e9
        return {"bound": "tensor", "achieved": a, "peak": peak, "unit": "TFLOP/s", "frac": a / peak,
                "frac_of_nominal": a / nominal, "nominal": nominal, "ms": ms}

    def hbm_roof(byts, ms):
        a = byts / ms / 1e6
        return {"bound": "hbm", "achieved": a, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": a / peaks["hbm_gbs"],
                "frac_of_nominal": a / NOMINAL_HBM_GBS, "nominal": NOMINAL_HBM_GBS, "ms": ms, "bytes": byts}

    # ---- configs[0]: 4096^3, quantize + GEMM
    a, w = _randn((4096, 4096), g), _randn((4096, 4096), g)
    wq, ws = ops.quantize_fp8_row(w)
    y = torch.empty((4096, 4096), dtype=torch.bfloat16, device=device)
    xq, xs = ops.quantize_fp8_row(a)
    q_ms = _time_graph(lambda: ops.quantize_fp8_row(a), 20)
    g_ms = _time_plain(lambda: ops.f8f8bf16_rowwise_out(xq, wq, xs, ws, y), 30)
    out["fp8_4096_cubed"] = {"quantize": hbm_roof(3.0 * 4096 * 4096 + 4.0 * 4096, q_ms),
                             "gemm": tensor_roof(2.0 * 4096 ** 3, g_ms, fp8_peak, NOMINAL_FP8_TFLOPS),
                             "note": "50 MB of quantizer traffic fits the 126 MB L2: the quantize figure is an L2 figure"}
    # ---- 8192^3 FP8 (the north-star shape)
    xq, xs = ops.quantize_fp8_row(_randn((8192, 8192), g))
    wq, ws = ops.quantize_fp8_row(_randn((8192, 8192), g, 0.02))
    y = torch.empty((8192, 8192), dtype=torch.bfloat16, device=device)
    ms = _time_plain(lambda: ops.f8f8bf16_rowwise_out(xq, wq, xs, ws, y), 30)
    out["fp8_8192_cubed"] = tensor_roof(2.0 * 8192 ** 3, ms, fp8_peak, NOMINAL_FP8_TFLOPS)
    out["fp8_8192_cubed"]["frac_of_nominal_4500"] = out["fp8_8192_cubed"]["frac_of_nominal"]
    # ---- few-token Llama-3-8B shapes (weight streaming: HBM-bound)
    few = []
    for M in (1, 16, 128):
        for N, K in ((28672, 4096), (4096, 14336)):
            xq, xs = ops.quantize_fp8_row(_randn((M, K), g))
            ws_ = [ops.quantize_fp8_row(_randn((N, K), g, 0.02)) for _ in range(3)]     # 3 x 117 MB > L2
            y = torch.empty((M, N), dtype=torch.bfloat16, device=device)
            it = [0]

            def f():
                i = it[0] % 3
                it[0] += 1
                ops.f8f8bf16_rowwise_out(xq, ws_[i][0], xs, ws_[i][1], y)
            ms = _time_graph(f, 30)
            r = hbm_roof(N * K + M * K + 2.0 * M * N + 4.0 * (M + N), ms)
            r.update({"M": M, "N": N, "K": K})
            few.append(r)
    out["fp8_few_tokens"] = few
    # ---- quantize_fp8_row per BASELINE shape (inputs rotate through more than the L2 holds)
    quant = []
    for M, K in ((8192, 4096), (8192, 14336), (8192, 8192), (8192, 28672), (16384, 5120), (16384, 8192)):
        nv = max(2, int(400e6 // (M * K * 2)) + 1)
        xs_ = [_randn((M, K), g) for _ in range(nv)]
        it = [0]

        def f():
            ops.quantize_fp8_row(xs_[it[0] % nv])
            it[0] += 1
        ms = _time_graph(f, 4 * nv)
        r = hbm_roof(3.0 * M * K + 4.0 * M, ms)
        r.update({"M": M, "K": K})
        quant.append(r)
        del xs_
    out["quantize_fp8_row"] = quant
    torch.cuda.empty_cache()
    # ---- configs[3]: grouped MoE, both projections
    from microbench import zipf_counts
    counts = zipf_counts(16, 16384)
    msz = counts.to(torch.int64).to(device)
    moe = {"counts": counts.tolist()}
    for name, N, K in (("gate_up", 16384, 5120), ("down", 5120, 8192)):
        xq, xs = ops.quantize_fp8_row(_randn((16384, K), g))
        wq, ws = ops.quantize_fp8_row(_randn((16, N, K), g, 0.02))
        ms = _time_plain(lambda: ops.f8f8bf16_rowwise_grouped_stacked(xq, wq, xs, ws.view(-1), msz), 20)
        moe[name] = tensor_roof(2.0 * 16384 * N * K, ms, fp8_peak, NOMINAL_FP8_TFLOPS)
        del xq, wq
    out["fp8_grouped_moe_e16"] = moe
    torch.cuda.empty_cache()
    # ---- configs[4]: NVFP4 8192^3 and M = 1 / 32 at (28672, 8192)
    fp4_peak = 4.0 * peaks["bf16_burst"]

    def nvfp4_case(M, N, K, nvar):
        x = _randn((M, K), g)
        gx = (448.0 * 6.0) / x.abs().amax().float()
        xq, sx = ops.quantize_nvfp4(x, gx)
        ws_ = []
        for _ in range(nvar):
            w = _randn((N, K), g)
            gw = (448.0 * 6.0) / w.abs().amax().float()
            wq, sw = ops.quantize_nvfp4(w, gw)
            ws_.append((wq, sw, (1.0 / (gx * gw)).reshape(1)))
        y = torch.empty((M, N), dtype=torch.bfloat16, device=device)
        it = [0]

        def f():
            i = it[0] % nvar
            it[0] += 1
            ops.f4f4bf16(xq, ws_[i][0], sx, ws_[i][1], output=y, global_scale=ws_[i][2])
        return f

    ms = _time_plain(nvfp4_case(8192, 8192, 8192, 2), 30)
    out["nvfp4_8192_cubed"] = tensor_roof(2.0 * 8192 ** 3, ms, fp4_peak, NOMINAL_FP4_TFLOPS)
    out["nvfp4_8192_cubed"]["peak_source"] = "4 x bf16_tflops (burst): the fp4 tensor rate is four times the bf16 rate"
    dec = []
    for M in (1, 32):
        N, K = 28672, 8192
        ms = _time_graph(nvfp4_case(M, N, K, 3), 30)
        r = hbm_roof(N * K / 2 + M * K / 2 + (128 + N) * K / 16 + 2.0 * M * N, ms)
        r.update({"M": M, "N": N, "K": K})
        dec.append(r)
    out["nvfp4_few_tokens"] = dec
    x = _randn((8192, 8192), g)
    gx = (448.0 * 6.0) / x.abs().amax().float()
    xs_ = [x, _randn((8192, 8192), g), _randn((8192, 8192), g)]
    it = [0]

    def fq():
        ops.quantize_nvfp4(xs_[it[0] % 3], gx)
        it[0] += 1
    ms = _time_graph(fq, 12)
    out["quantize_nvfp4_8192x8192"] = hbm_roof(8192 * 8192 * 2.5625, ms)
    # ---- MXFP4 (e8m0 scales per 32 elements, the reference's default mode of the FP4 operators): 8192^3 and its quantizer
    def fqm():
        ops.quantize_mx4(xs_[it[0] % 3], 32)
        it[0] += 1
    ms = _time_graph(fqm, 12)
    out["quantize_mx4_8192x8192"] = hbm_roof(8192 * 8192 * (2.0 + 0.5 + 1.0 / 32.0), ms)
    xq, sx = ops.quantize_mx4(xs_[0], 32)
    wqs = [ops.quantize_mx4(xs_[1 + i], 32) for i in range(2)]
    y = torch.empty((8192, 8192), dtype=torch.bfloat16, device=device)

    def fm():
        i = it[0] % 2
        it[0] += 1
        ops.f4f4bf16(xq, wqs[i][0], sx, wqs[i][1], output=y)
    ms = _time_plain(fm, 30)
    out["mxfp4_8192_cubed"] = tensor_roof(2.0 * 8192 ** 3, ms, fp4_peak, NOMINAL_FP4_TFLOPS)
    del xs_, wqs, xq, sx, y
    torch.cuda.empty_cache()
    # ---- grouped FP4 MoE (configs[3] shapes, E = 16, Zipf counts): stacked quantizers and grouped GEMMs, NVFP4 and MXFP4
    x = _randn((16384, 5120), g)
    w = _randn((16 * 16384, 5120), g, 0.02)
    w_ms = torch.full((16,), 16384, dtype=torch.int64, device=device)
    grouped = {}
    x_gs, _ = ops.calculate_group_max(x, msz)
    w_gs, _ = ops.calculate_group_max(w, w_ms)
    q_ms = _time_graph(lambda: ops.nvfp4_quantize_stacked(msz, x, x_gs), 12)
    xq, sx = ops.nvfp4_quantize_stacked(msz, x, x_gs)
    wq, sw = ops.nvfp4_quantize_stacked(w_ms, w, w_gs)
    alpha = torch.reciprocal(x_gs * w_gs)
    sw3 = sw[: 16 * 16384].view(16, 16384, -1)
    ms = _time_plain(lambda: ops.f4f4bf16_grouped_stacked(xq, wq.view(16, 16384, 2560), sx, sw3, msz, alpha, None,
                                                          use_mx=False), 20)
    grouped["nvfp4"] = {"quantize_stacked": hbm_roof(16384 * 5120 * 2.5625, q_ms),
                        "gemm_gate_up": tensor_roof(2.0 * 16384 * 16384 * 5120, ms, fp4_peak, NOMINAL_FP4_TFLOPS)}
    q_ms = _time_graph(lambda: ops.quantize_mx4_stacked(msz, x), 12)
    xq, sx = ops.quantize_mx4_stacked(msz, x)
    wq, sw = ops.quantize_mx4_stacked(w_ms, w)
    pc = 5120 // 32
    sw3 = sw[: 16 * 16384 * pc].view(16, -1)
    ms = _time_plain(lambda: ops.f4f4bf16_grouped_stacked(xq, wq.view(16, 16384, 2560), sx, sw3, msz), 20)
    grouped["mxfp4"] = {"quantize_stacked": hbm_roof(16384 * 5120 * (2.5 + 1.0 / 32.0), q_ms),
                        "gemm_gate_up": tensor_roof(2.0 * 16384 * 16384 * 5120, ms, fp4_peak, NOMINAL_FP4_TFLOPS)}
    out["fp4_grouped_moe_e16"] = grouped
    return out


def sustained_run(tp, seconds, device_index):
    """The headline step looped for at least `seconds`, with the SM clock sampled meanwhile: the power-capped
    figure beside the burst figure of the timed region."""
    sampler = ClockSampler(device_index)
    sampler.start()
    e0, e1 = _ev(), _ev()
    n = 0
    t0 = time.perf_counter()
    e0.record()
    while True:
        for _ in range(25):
            tp.step()
        n += 25
        torch.cuda.synchronize()
        if time.perf_counter() - t0 >= seconds:
            break
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / n
    return {"seconds": e0.elapsed_time(e1) / 1e3, "steps": n, "ms_per_step": ms, "tflops": ffn_flops() / ms / 1e9,
            "sm_mhz_median": clocks["sm_mhz"], "power_w_max": clocks.get("power_w_max"), "reasons": clocks["reasons"],
            "ms_times_mhz": (ms * clocks["sm_mhz"]) if clocks["sm_mhz"] else None,
            "frac_of_nominal_4500": ffn_flops() / ms / 1e9 / NOMINAL_FP8_TFLOPS}


def reference_gpu_quick(ops):
    """This library against the reference's own sm_100 kernels (baseline/_ref/libmslk_ref_gpu.so: the reference's
    sources at stock CUTLASS) on the headline shapes; None when that library is absent."""
    lib = os.path.join(ROOT, "baseline", "_ref", "libmslk_ref_gpu.so")
    if not os.path.exists(lib):
        return {"unavailable": "baseline/_ref/libmslk_ref_gpu.so is missing (python baseline/build_ref_gpu.py)"}
    try:
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import race_ref_gpu as race
        torch.ops.load_library(lib)
        ref = torch.ops.mslk_ref
        rows = [race.race_dense(ops, ref, 8192, 8192, 8192, 20, 3),
                race.race_dense(ops, ref, 8192, GATE_UP[0] // 8, GATE_UP[1], 20, 3, w_std=0.01),
                race.race_dense(ops, ref, 8192, 28672, 4096, 20, 3),
                race.race_grouped(ops, ref, 16, 16384, 16384, 5120, 10, 2),
                race.race_nvfp4(ops, ref, 8192, 8192, 8192, 20, 3),
                race.race_nvfp4(ops, ref, 32, 28672, 8192, 50, 3)]
        return {"what": "reference sources at stock CUTLASS 4.x (the reference pins a fork whose checkout is empty), "
                        "same tensors, same CUDA-event timing; ours_over_ref_speed > 1 means this library is faster",
                "cases": rows}
    except Exception as e:  # the comparator must never take the benchmark down
        return {"unavailable": f"{type(e).__name__}: {e}"[:300]}


# ----------------------------------------------------------------------------- CPU reference arm

def make_cpu_sample(tokens, seed=0):
    import oracle
    g = torch.Generator().manual_seed(seed)
    sample = []
    for n, k in (GATE_UP, DOWN):
        x = torch.randn((tokens, k), generator=g).to(torch.bfloat16)
        w = (torch.randn((n, k), generator=g) * 0.01).to(torch.bfloat16)
        wq, ws = oracle.quantize_fp8_row_cpu_path_torch(w)
        sample.append({"x": x, "wq": wq, "ws": ws})
    return sample


def cpu_reference_step(sample):
    """The reference's CPU path for one step on `sample` rows: torch per-row quantize
    (mslk/quantize/triton/fp8_quantize.py:356-378) then dequantize + fp32 matmul with the
    row/column scales (test/gemm/triton/grouped_gemm_test.py:124-129), for both projections."""
    import oracle
    for L in sample:
        xq, xs = oracle.quantize_fp8_row_cpu_path_torch(L["x"])
        oracle.gemm_f8_rowwise_torch(xq, L["wq"], xs, L["ws"])


def cpu_threads():
    """torchrun exports OMP_NUM_THREADS=1; the CPU arm uses every core this process may run on."""
    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    return cores


def base_line(args, world):
    P = world
    return {
        "metric": "FP8 rowwise GEMM TFLOP/s (f8f8bf16_rowwise, Llama-3-70B FFN projections at M=8192, tensor-parallel)",
        "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate)",
        "data": "synthetic (seeded randn; activations N(0,1), weights N(0,0.01))",
        "config": {"workload": "llama3-70b FFN at M=8192 tokens: quantize_fp8_row + f8f8bf16_rowwise gate+up "
                               "(N=57344,K=8192) N-sharded with all-gather of the bf16 output, down (N=8192,K=28672) "
                               "K-sharded with reduce-scatter; whole job = 11.5 TFLOP per step",
                   "tokens": FFN_TOKENS, "parallelism": f"tp{P}" if P > 1 else "single GPU (unsharded)",
                   "l2": "per-step working set (0.7 GB of fp8 weights + 0.37 GB activations + 1.07 GB outputs at N=1) exceeds the 126 MB L2"},
    }


def run_reference(args, rank, world):
    if rank != 0:
        return
    cores = cpu_threads()
    sample = make_cpu_sample(CPU_SAMPLE_TOKENS)
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_reference_step(sample)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_reference_step(sample)
    sec = (time.perf_counter() - t0) / args.steps
    val = ffn_flops(CPU_SAMPLE_TOKENS) / sec / 1e12
    line = base_line(args, world)
    desc = (f"{CPU_SAMPLE_TOKENS} of the {FFN_TOKENS} tokens through both projections per step (torch CPU: per-row quantize "
            f"+ dequantize/fp32 matmul of the unsharded weights), {torch.get_num_threads()} torch threads on rank 0 only")
    line.update({"impl": "reference", "value": val, "ms_per_step": sec * 1e3, "gpu_launches": 0,
                 "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": desc},
                 "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
    print(json.dumps(line), flush=True)


def time_cpu_baseline(tokens, repeats):
    sample = make_cpu_sample(tokens)
    cpu_reference_step(sample)  # warm-up
    t = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        cpu_reference_step(sample)
        t.append(time.perf_counter() - t0)
    t.sort()
    sec = t[len(t) // 2]
    return ffn_flops(tokens) / sec / 1e12, sec


# ----------------------------------------------------------------------------- end to end

def e2e_run(tp, dd, steps):
    """The step through the public operators with HOST buffers: every step copies the bf16 activation of gate+up and
    this rank's fp8 slice of the down activation from pinned host memory, and copies the results back (this rank's
    rows of the gathered gate+up output and its rows of the down output) to pinned host memory.  Three streams (copies
    in, kernels, copies out) ordered by events; steps overlap as in a serving loop, every step's bytes cross PCIe."""
    import torch.distributed as dist
    device, P, r = tp.device, tp.world, tp.rank
    rows = tp.rows
    # the activation is replicated: with P ranks each uploads its 1/P of the rows and an all-gather over NVLink
    # completes the copy on every GPU (P x fewer bytes through the host's PCIe complex)
    hx1 = torch.empty((rows, tp.x1.shape[1]), dtype=torch.bfloat16).pin_memory()
    hx1.copy_(tp.x1[r * rows:(r + 1) * rows])
    x1_slice = torch.empty((rows, tp.x1.shape[1]), dtype=torch.bfloat16, device=device) if P > 1 else None
    hx2 = torch.empty(tp.xq2_k.shape, dtype=torch.uint8).pin_memory()
    hx2.copy_(tp.xq2_k.view(torch.uint8))
    hy1 = [torch.empty((rows, GATE_UP[0]), dtype=torch.bfloat16).pin_memory() for _ in range(2)]   # results alternate, so
    hy2 = [torch.empty((rows, DOWN[0]), dtype=torch.bfloat16).pin_memory() for _ in range(2)]      # a reader has a step's time
    s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
    s_main = torch.cuda.current_stream(device)
    ev_in, ev_used, ev_done1, ev_done2 = (torch.cuda.Event() for _ in range(4))
    ev_used.record(s_main)
    # The results leave through two alternating pairs of device staging buffers: a device-to-device copy on the compute
    # stream frees the operators' output buffers for the next step at once, and the copies to the host (the slowest part
    # of the step: PCIe) run back to back on their own stream under the next steps' kernels.
    stage1 = [torch.empty((rows, GATE_UP[0]), dtype=torch.bfloat16, device=device) for _ in range(2)]
    stage2 = [torch.empty((rows, DOWN[0]), dtype=torch.bfloat16, device=device) for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    for e in ev_out:
        e.record(s_main)
    x2_u8 = tp.xq2_k.view(torch.uint8)
    count = [0]

    def step():
        b = count[0] & 1
        count[0] += 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_used)             # the previous step has consumed the device copies
            if P > 1:
                x1_slice.copy_(hx1, non_blocking=True)
                dist.all_gather_into_tensor(tp.x1, x1_slice)
            else:
                tp.x1.copy_(hx1, non_blocking=True)
            x2_u8.copy_(hx2, non_blocking=True)
            ev_in.record(s_in)
        s_main.wait_event(ev_in)
        if P > 1:
            tp.h1.barrier()                      # every rank is past its copies out of the buffers the peers store into
        xq, xs = tp.quantize()
        tp.gate_up_fused(xq, xs)
        s_main.wait_event(ev_out[b])             # the results of two steps ago have left this pair of staging buffers
        stage1[b].copy_(tp.y1[r * rows:(r + 1) * rows])
        ev_done1.record(s_main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_done1)
            hy1[b].copy_(stage1[b], non_blocking=True)
        if tp.fused_down:
            tp.down_fused()
        else:
            tp.down_nccl()
        ev_used.record(s_main)
        stage2[b].copy_(tp.y2)
        ev_done2.record(s_main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_done2)
            hy2[b].copy_(stage2[b], non_blocking=True)
            ev_out[b].record(s_out)

    def join():
        s_main.wait_stream(s_in)
        s_main.wait_stream(s_out)

    step()
    join()
    dd.barrier()
    e_steps = max(1, min(steps, 10))
    s0, s1 = _ev(), _ev()
    s0.record()
    for _ in range(e_steps):
        step()
    join()
    s1.record()
    dd.barrier()
    ms = dd.max(s0.elapsed_time(s1) / e_steps)
    # the last step's results on the host are the device's (the inputs are the same every step, so both pairs hold them)
    torch.cuda.synchronize(device)
    last = (count[0] - 1) & 1
    arrived = bool(torch.equal(hy2[last], tp.y2.cpu())) and \
        bool(torch.equal(hy1[last][:64], tp.y1[r * rows:r * rows + 64].cpu())) and \
        bool(torch.equal(hy1[last][-64:], tp.y1[(r + 1) * rows - 64:(r + 1) * rows].cpu()))
    return {"value": ffn_flops() / ms / 1e9, "unit": "TFLOP/s", "ms_per_step": ms, "results_on_host_match_device": arrived,
            "h2d_bytes_per_step": hx1.numel() * 2 + hx2.numel(), "d2h_bytes_per_step": (hy1[0].numel() + hy2[0].numel()) * 2,
            "note": "bytes are per rank; every rank copies its 1/P of the rows of the replicated activation in (an NCCL "
                    "all-gather completes it on every GPU), its K slice of the down operand in, and its own rows of both "
                    "results out"}


# ----------------------------------------------------------------------------- main arm

def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: mslk_b200 has no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    from mslk_b200 import ops, parallel as par
    from mslk_b200._lib import device_status
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    dd = Dist(world, device)
    peaks = load_peaks()
    tp = FfnTensorParallel(ops, par, rank, world, device)

    # ---- set-up: which reduce-scatter is faster on this node (both are part of the library; same choice on every rank)
    choice = None
    if world > 1:
        t_fused = dd.timed(tp.down_fused, 5, 3)
        t_nccl = dd.timed(tp.down_nccl, 5, 3)
        tp.fused_down = t_fused <= t_nccl
        choice = {"down_reduce_scatter": "fused epilogue + slot sum" if tp.fused_down else "NCCL reduce_scatter_tensor",
                  "fused_ms": t_fused, "nccl_ms": t_nccl, "gate_up_all_gather": "fused epilogue (peer stores)"}

    sampler = ClockSampler(local_rank)
    sampler.start()          # before the warm-up: nvidia-smi needs a moment to deliver its first sample
    for _ in range(max(args.warmup, 3)):
        tp.step()
    dd.barrier()

    # ---- timed region: K steps, CUDA events on the launching stream
    ev = [[_ev() for _ in range(3)] for _ in range(args.steps)]
    start, stop = _ev(), _ev()
    dd.barrier()
    start.record()
    for s in range(args.steps):
        tp.step(ev[s])
    stop.record()
    dd.barrier()
    clocks = sampler.stop()
    ms_max = dd.max(start.elapsed_time(stop))
    if device_status() != 0:
        raise RuntimeError("a kernel reported a pipeline timeout during the timed region")
    per_step_ms = ms_max / args.steps
    g1_ms = sum(ev[s][0].elapsed_time(ev[s][1]) for s in range(args.steps)) / args.steps
    g2_ms = sum(ev[s][1].elapsed_time(ev[s][2]) for s in range(args.steps)) / args.steps

    tp_parts = tp_breakdown(tp, dd, max(3, min(args.steps, 10)), 3)
    nccl_step_ms = dd.timed(tp.step_nccl, max(3, min(args.steps, 10)), 3) if world > 1 else None
    gemm_step_ms = dd.timed(tp.step_gemm_only, max(3, min(args.steps, 10)), 3)
    e2e = None if args.no_e2e else e2e_run(tp, dd, args.steps)
    moe = None if args.no_extras else moe_expert_sharded(ops, par, dd, rank, world, device, 5, 2)

    line = base_line(args, world)
    value = ffn_flops() / per_step_ms / 1e9
    if rank == 0:
        # the dominant kernel's own time: at N = 1 the event intervals around the two GEMM launches inside the timed
        # region; with collectives in the step those intervals carry the peer traffic, so the GEMMs issued alone
        if world == 1:
            gemm_only = g1_ms + g2_ms
            how = "CUDA events around the two GEMM launches inside the timed region"
        else:
            gemm_only = tp_parts["gate_up"]["gemm_only_ms"] + tp_parts["down"]["gemm_only_ms"]
            how = ("CUDA events around the two GEMM launches of a step issued alone (no collective, outputs stay local), per "
                   "GPU; in the step itself the launches also carry the peer stores")
        achieved = ffn_flops() / world / gemm_only / 1e9       # per-GPU rate of the two GEMM launches
        fp8_peak = 2.0 * peaks["bf16_burst"]
        traffic = load_traffic()
        n1l, k2l = GATE_UP[0] // world, DOWN[1] // world      # operands + output once, per rank
        alg_bytes = [FFN_TOKENS * GATE_UP[1] + n1l * GATE_UP[1] + 2 * FFN_TOKENS * n1l,
                     FFN_TOKENS * k2l + DOWN[0] * k2l + 2 * FFN_TOKENS * DOWN[0]]
        # bytes the two launches bring into the SMs' shared memory: every 256 x 256 pair tile takes 2 x 32 KB per K block of 128
        def _sm_bytes(m, n, k):
            return ((m + 255) // 256) * ((n + 255) // 256) * ((k + 127) // 128) * 2 * 32768
        sm_bytes = _sm_bytes(FFN_TOKENS, n1l, GATE_UP[1]) + _sm_bytes(FFN_TOKENS, DOWN[0], k2l)
        line.update({
            "value": value, "ms_per_step": per_step_ms, "gpu_launches": tp.launches_per_step() * args.steps,
            "roofline": {"bound": "tensor", "kernel": "gemm_f8_rowwise_pair_kernel", "achieved": achieved,
                         "peak": fp8_peak, "unit": "TFLOP/s", "frac": achieved / fp8_peak,
                         "traffic": (traffic.get("mean_dram_bytes_per_launch") if world == 1 else None),
                         "algorithmic_bytes_per_launch": sum(alg_bytes) / 2.0,
                         "measured": how,
                         "peak_source": f"2 x bf16_tflops (burst) of {peaks['source']} peaks (the fp8 tensor rate is twice the bf16 rate; "
                                        "the peaks file holds no fp8 figure)",
                         "frac_of_nominal_4500": achieved / NOMINAL_FP8_TFLOPS,
                         "flops_per_step_per_gpu": ffn_flops() / world, "ms_in_kernel": gemm_only,
                         "operand_delivery": {
                             "achieved_tbs": sm_bytes / gemm_only / 1e9, "ceiling_tbs": SM_INGEST_TBS,
                             "frac": sm_bytes / gemm_only / 1e9 / SM_INGEST_TBS, "bytes_per_step_per_gpu": sm_bytes,
                             "note": "operand bytes landing in the SMs' shared memory (2 x 32 KB per pair tile and K block) over "
                                     "the same kernel time; the ceiling is the L2 -> SM rate ncu counted on this kernel and on "
                                     "both FP4 pair kernels at 8192^3 (l1tex__m_xbar2l1tex_read_bytes per second, whatever the "
                                     "SM clock): with 256 x 256 pair tiles it caps FP8 at 3.33 PFLOP/s"}},
            "in_step_intervals_ms": {"gate_up_gemm_with_collective": g1_ms, "down_gemm_with_collective": g2_ms,
                                     "quantize_and_gaps": per_step_ms - g1_ms - g2_ms,
                                     "note": "rank 0's event intervals inside the timed region"},
            "step_over_gemm_kernels": gemm_only / per_step_ms,
            "tp": {**tp_parts, "product_path": choice,
                   "step_with_nccl_collectives_ms": nccl_step_ms,
                   "step_with_nccl_collectives_tflops": (ffn_flops() / nccl_step_ms / 1e9) if nccl_step_ms else None,
                   "step_gemms_only_ms": gemm_step_ms, "step_gemms_only_tflops": ffn_flops() / gemm_step_ms / 1e9},
            "clocks": clocks,
        })
        if e2e is not None:
            line["e2e"] = e2e
        if moe is not None:
            line["moe_expert_sharded"] = moe
    if world == 1 and not args.no_extras:
        line["sustained"] = sustained_run(tp, args.sustain_seconds, local_rank)
        del tp
        torch.cuda.empty_cache()
        line["llama3_8b_step"] = llama3_8b_step(ops, device, max(5, min(args.steps, 20)), 3)
        line["configs"] = other_configs(ops, device, peaks)
        line["reference_gpu"] = reference_gpu_quick(ops)
        if device_status() != 0:
            raise RuntimeError("a kernel reported a pipeline timeout in the extra sections")
    if world == 1 and not args.no_cpu_baseline:
        cores = cpu_threads()
        val, sec = time_cpu_baseline(CPU_SAMPLE_TOKENS, repeats=3)
        line["cpu_baseline"] = {
            "value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"{CPU_SAMPLE_TOKENS} of the {FFN_TOKENS} tokens through both projections (torch CPU per-row quantize + "
                      f"dequantize/fp32 matmul), median of 3, {sec:.2f} s per pass, {torch.get_num_threads()} torch threads"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--sustain-seconds", type=float, default=2.5)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="headline, tp and e2e sections only")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
