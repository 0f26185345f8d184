#!/usr/bin/env python
"""Benchmark of the FP8-rowwise hot path (per-row quantize -> rowwise-scaled FP8 GEMM).

One "step" is one pass of the hot path over one batch: the four linear projections of a
Llama-3-8B layer (QKV 6144x4096, O 4096x4096, gate+up 28672x4096, down 4096x14336) on a
batch of M=8192 tokens -- for each projection the bf16 activation is quantized per row to
e4m3 and multiplied with the offline-quantized weight.  The metric is TFLOP/s over the GEMM
flops (2*M*N*K summed over the four projections) divided by the time of the whole step
(quantize kernels included).  With N GPUs every rank runs the same step on its own batch
(data-parallel replicas, no collective; weak scaling).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

prints ONE JSON line (rank 0).  `--impl reference` times the reference's CPU path
(torch per-row quantize + dequantize/fp32-matmul, as its tests do) on the host cores, on a
bounded sample of the same workload.  Extra sections of the line: `roofline` (dominant
kernel = the tcgen05 GEMM), `roofline_quantize`, `cpu_baseline`, `e2e`, `clocks`, `shapes`.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M_TOKENS = 8192
PROJECTIONS = [("qkv", 6144, 4096), ("o", 4096, 4096), ("gate_up", 28672, 4096), ("down", 4096, 14336)]
CPU_SAMPLE_TOKENS = 512
NOMINAL_FP8_TFLOPS = 4500.0
NOMINAL_HBM_GBS = 8000.0


def step_flops(m=M_TOKENS):
    return sum(2.0 * m * n * k for _, n, k in PROJECTIONS)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_burst": float(p["bf16_tflops"]),
                "bf16_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


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
            time.sleep(0.15)
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
        for line in out.strip().splitlines():
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


def make_inputs(device, seed):
    """Seeded synthetic data with the shapes and distributions of the Llama-3-8B sweep:
    activations bf16 ~N(0,1), weights bf16 ~N(0,0.02) quantized per row offline."""
    from mslk_b200 import ops
    g = torch.Generator(device=device).manual_seed(seed)
    layers = []
    for name, n, k in PROJECTIONS:
        x = torch.randn((M_TOKENS, k), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
        w = (torch.randn((n, k), generator=g, device=device, dtype=torch.float32) * 0.02).to(torch.bfloat16)
        wq, ws = ops.quantize_fp8_row(w)
        del w
        layers.append({"name": name, "n": n, "k": k, "x": x, "wq": wq, "ws": ws})
    return layers


def run_step(ops, layers, outs, ev=None, side=None, prev_done=None):
    """One pass of the hot path.  With `ev`, CUDA events bracket every kernel launch.

    With `side` (a second CUDA stream) the HBM-bound quantize kernels run there and the tensor-bound
    GEMMs on the current stream, each GEMM waiting for its own input only: a quantize CTA fits on an SM
    beside the persistent GEMM CTA, so the quantization of projection i+1 overlaps the GEMM of
    projection i.  `prev_done` (events of the previous step's GEMMs) keeps the side stream at most one
    step ahead.  Returns the GEMM-done events of this step."""
    main = torch.cuda.current_stream()
    done = []
    for i, L in enumerate(layers):
        if side is None:
            if ev is not None:
                ev[i][0].record()
            xq, xs = ops.quantize_fp8_row(L["x"])
            if ev is not None:
                ev[i][1].record()
        else:
            with torch.cuda.stream(side):
                if prev_done is not None:
                    side.wait_event(prev_done[i])
                if ev is not None:
                    ev[i][0].record(side)
                xq, xs = ops.quantize_fp8_row(L["x"])
                if ev is not None:
                    ev[i][1].record(side)
                ready = torch.cuda.Event()
                ready.record(side)
            xq.record_stream(main)
            xs.record_stream(main)
            main.wait_event(ready)
        if ev is not None:
            ev[i][2].record()
        ops.f8f8bf16_rowwise_out(xq, L["wq"], xs, L["ws"], outs[i])
        if ev is not None:
            ev[i][3].record()
        if side is not None:
            d = torch.cuda.Event()
            d.record()
            done.append(d)
    return done


def cpu_reference_step(sample):
    """The reference's CPU path for one step on `sample` rows: torch per-row quantize
    (mslk/quantize/triton/fp8_quantize.py:356-378) then dequantize + fp32 matmul with the
    row/column scales (test/gemm/triton/grouped_gemm_test.py:124-129)."""
    import oracle
    for L in sample:
        xq, xs = oracle.quantize_fp8_row_cpu_path_torch(L["x"])
        oracle.gemm_f8_rowwise_torch(xq, L["wq"], xs, L["ws"])


def make_cpu_sample(tokens, seed=0):
    import oracle
    g = torch.Generator().manual_seed(seed)
    sample = []
    for name, n, k in PROJECTIONS:
        x = torch.randn((tokens, k), generator=g).to(torch.bfloat16)
        w = (torch.randn((n, k), generator=g) * 0.02).to(torch.bfloat16)
        wq, ws = oracle.quantize_fp8_row_cpu_path_torch(w)
        sample.append({"x": x, "wq": wq, "ws": ws})
    return sample


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
    return step_flops(tokens) / sec / 1e12, sec


def base_line(args, world):
    return {
        "metric": "FP8 rowwise GEMM TFLOP/s (per-row quantize + f8f8bf16_rowwise, Llama-3-8B layer projections)",
        "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate)",
        "data": "synthetic (seeded randn; activations N(0,1), weights N(0,0.02))",
        "config": {"workload": "llama3-8b layer projections, M=8192 tokens per GPU: quantize_fp8_row + "
                               "f8f8bf16_rowwise for (N,K) in (6144,4096),(4096,4096),(28672,4096),(4096,14336)",
                   "tokens_per_gpu": M_TOKENS, "parallelism": f"replicas x{world} (no collective)",
                   "streams": ("2: quantize kernels on a side stream overlap the previous projection's GEMM"
                               if getattr(args, "streams", 1) == 2 else "1"),
                   "l2": "per-step working set (0.44 GB activations + 0.22 GB weights + 0.7 GB outputs) exceeds the 126 MB L2"},
    }


def run_reference(args, rank, world):
    if rank != 0:
        return
    cores = len(os.sched_getaffinity(0))
    sample = make_cpu_sample(CPU_SAMPLE_TOKENS)
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_reference_step(sample)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_reference_step(sample)
    sec = (time.perf_counter() - t0) / args.steps
    val = step_flops(CPU_SAMPLE_TOKENS) / sec / 1e12
    line = base_line(args, world)
    desc = (f"{CPU_SAMPLE_TOKENS} of the {M_TOKENS} tokens through all four projections per step "
            f"(torch CPU: per-row quantize + dequantize/fp32 matmul), {torch.get_num_threads()} torch threads")
    line.update({"impl": "reference", "value": val, "ms_per_step": sec * 1e3, "gpu_launches": 0,
                 "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": desc},
                 "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
    print(json.dumps(line), flush=True)


def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: mslk_b200 has no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    from mslk_b200 import ops
    from mslk_b200._lib import device_status
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    layers = make_inputs(device, seed=rank)
    outs = [torch.empty((M_TOKENS, L["n"]), dtype=torch.bfloat16, device=device) for L in layers]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    sampler.start()          # before the warm-up: nvidia-smi needs a moment to deliver its first sample
    side = torch.cuda.Stream(device=device) if args.streams == 2 else None
    prev = None
    for _ in range(max(args.warmup, 3)):
        prev = run_step(ops, layers, outs, None, side, prev)
    barrier()

    # ---- timed region: K steps, CUDA events on the launching stream, events around every launch
    ev = [[[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in layers] for _ in range(args.steps)]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    prev = None
    if side is not None:
        side.wait_event(start)
    for s in range(args.steps):
        prev = run_step(ops, layers, outs, ev[s], side, prev)
    stop.record()      # the last GEMM waited for every quantize kernel, so this closes both streams
    barrier()
    clocks = sampler.stop()
    ms = start.elapsed_time(stop)
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())
    if device_status() != 0:
        raise RuntimeError("a kernel reported a pipeline timeout during the timed region")

    # The quantize kernels last 17-55 us, so an event pair around a single launch is dominated by the gap
    # between dependent launches.  Their own rate is measured by one event pair around 10 rounds over the
    # four activations (218 MB per round, more than the L2 holds) issued back to back.
    # The 40 launches are replayed from a CUDA graph, so the gaps between them are the device's, not the host's.
    q0, q1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for L in layers:
        ops.quantize_fp8_row(L["x"])
    torch.cuda.synchronize()
    q_graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(q_graph):
        for _ in range(10):
            for L in layers:
                ops.quantize_fp8_row(L["x"])
    q_graph.replay()
    torch.cuda.synchronize()
    q0.record()
    q_graph.replay()
    q1.record()
    torch.cuda.synchronize()
    q_loop_ms = q0.elapsed_time(q1) / 10.0
    del q_graph

    q_ms = [sum(ev[s][i][0].elapsed_time(ev[s][i][1]) for s in range(args.steps)) / args.steps for i in range(len(layers))]
    g_ms = [sum(ev[s][i][2].elapsed_time(ev[s][i][3]) for s in range(args.steps)) / args.steps for i in range(len(layers))]

    # ---- end to end through the public API with host buffers (pinned), copies inside the timed region
    e2e = None
    if not args.no_e2e:
        hx = [torch.empty(L["x"].shape, dtype=torch.bfloat16).pin_memory() for L in layers]
        hy = [torch.empty(o.shape, dtype=torch.bfloat16).pin_memory() for o in outs]
        for h, L in zip(hx, layers):
            h.copy_(L["x"])
        dx = [torch.empty_like(L["x"]) for L in layers]

        # Three streams: host->device copies, kernels, device->host copies.  Events order them per
        # projection (and protect the reused device buffers across steps), so the copies of one
        # projection run while another one is being computed -- what a host application that
        # streams activations through the operators would do.
        s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
        s_main = torch.cuda.current_stream(device)
        ev_in = [torch.cuda.Event() for _ in layers]      # input i is on the device
        ev_used = [torch.cuda.Event() for _ in layers]    # quantize i has read dx[i]
        ev_done = [torch.cuda.Event() for _ in layers]    # GEMM i has written outs[i]
        ev_out = [torch.cuda.Event() for _ in layers]     # outs[i] has been copied to the host
        for e in ev_used + ev_out:
            e.record(s_main)

        def e2e_step():
            for i, L in enumerate(layers):
                with torch.cuda.stream(s_in):
                    s_in.wait_event(ev_used[i])
                    dx[i].copy_(hx[i], non_blocking=True)
                    ev_in[i].record(s_in)
                s_main.wait_event(ev_in[i])
                xq, xs = ops.quantize_fp8_row(dx[i])
                ev_used[i].record(s_main)
                s_main.wait_event(ev_out[i])
                ops.f8f8bf16_rowwise_out(xq, L["wq"], xs, L["ws"], outs[i])
                ev_done[i].record(s_main)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_done[i])
                    hy[i].copy_(outs[i], non_blocking=True)
                    ev_out[i].record(s_out)

        def join():
            s_main.wait_stream(s_in)
            s_main.wait_stream(s_out)

        e2e_step()
        join()
        barrier()
        e_steps = max(1, min(args.steps, 5))
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(e_steps):
            e2e_step()
        join()
        s1.record()
        barrier()
        et = torch.tensor([s0.elapsed_time(s1) / e_steps], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(et, op=dist.ReduceOp.MAX)
        e2e = {"value": world * step_flops() / (float(et.item()) * 1e-3) / 1e12, "unit": "TFLOP/s",
               "ms_per_step": float(et.item()),
               "h2d_bytes_per_step": sum(h.numel() * 2 for h in hx), "d2h_bytes_per_step": sum(h.numel() * 2 for h in hy)}

    if rank == 0:
        peaks = load_peaks()
        per_step_ms = ms_max / args.steps
        value = world * step_flops() / (per_step_ms * 1e-3) / 1e12
        gemm_flops = step_flops()
        gemm_ms = sum(g_ms)
        achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12
        # a timed region of a few hundred ms never reaches the power cap: compare with the burst figure;
        # a region of seconds runs power-capped: compare with the sustained one
        long_run = ms_max >= 2000.0
        fp8_peak = 2.0 * (peaks["bf16_sustained"] if long_run else peaks["bf16_burst"])
        q_bytes = sum(3.0 * M_TOKENS * L["k"] + 4.0 * M_TOKENS for L in layers)
        q_gbs = q_bytes / (q_loop_ms * 1e-3) / 1e9
        q_gbs_in_step = q_bytes / (sum(q_ms) * 1e-3) / 1e9
        line = base_line(args, world)
        line.update({
            "value": value, "ms_per_step": per_step_ms, "gpu_launches": 2 * len(layers) * args.steps,
            "roofline": {"bound": "tensor", "kernel": "gemm_f8_rowwise_pair_kernel", "achieved": achieved,
                         "peak": fp8_peak, "unit": "TFLOP/s", "frac": achieved / fp8_peak,
                         # DRAM bytes per launch, mean over the step's four GEMM launches, from the ncu capture of this
                         # same command (profiles/bench_gemm_dram_traffic__llama3_8b_layer_step.md); the algorithmic
                         # mean (operands + output once) is 285e6
                         "traffic": 436.0e6, "algorithmic_bytes_per_launch": 285.0e6,
                         "peak_source": f"2 x bf16_tflops{'_sustained' if long_run else ' (burst)'} of {peaks['source']} peaks "
                                        "(the fp8 tensor rate is twice the bf16 rate)",
                         "frac_of_nominal_4500": achieved / NOMINAL_FP8_TFLOPS,
                         "flops_per_step": gemm_flops, "ms_per_step_in_kernel": gemm_ms},
            "roofline_quantize": {"bound": "hbm", "kernel": "quant_fp8_row_vec_kernel", "achieved": q_gbs,
                                  "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": q_gbs / peaks["hbm_gbs"],
                                  "traffic": None, "peak_source": f"hbm_gbs of {peaks['source']} peaks",
                                  "frac_of_nominal_8000": q_gbs / NOMINAL_HBM_GBS,
                                  "bytes_per_step": q_bytes, "ms_per_round_back_to_back": q_loop_ms,
                                  "measured": "one CUDA-event pair around a CUDA graph of 10 rounds over the four activations (40 launches)",
                                  "in_step_event_intervals": {"ms_per_step": sum(q_ms), "GB/s": q_gbs_in_step,
                                                              "note": "event pair around each single launch inside the timed "
                                                                      "region; includes the gap between dependent launches"}},
            "shapes": [{"name": L["name"], "M": M_TOKENS, "N": L["n"], "K": L["k"],
                        "gemm_ms": g_ms[i], "gemm_tflops": 2.0 * M_TOKENS * L["n"] * L["k"] / (g_ms[i] * 1e-3) / 1e12,
                        "quant_ms": q_ms[i],
                        "quant_gbs": (3.0 * M_TOKENS * L["k"] + 4.0 * M_TOKENS) / (q_ms[i] * 1e-3) / 1e9}
                       for i, L in enumerate(layers)],
            "clocks": clocks,
        })
        if e2e is not None:
            line["e2e"] = e2e
        if world == 1 and not args.no_cpu_baseline:
            val, sec = time_cpu_baseline(CPU_SAMPLE_TOKENS, repeats=3)
            line["cpu_baseline"] = {
                "value": val, "unit": "TFLOP/s", "cores": len(os.sched_getaffinity(0)), "kind": "port",
                "sample": f"{CPU_SAMPLE_TOKENS} of the {M_TOKENS} tokens through all four projections "
                          f"(torch CPU per-row quantize + dequantize/fp32 matmul), median of 3, "
                          f"{sec:.2f} s per pass, {torch.get_num_threads()} torch threads"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--streams", type=int, choices=[1, 2], default=1,
                    help="2: quantize kernels on a side stream, overlapping the previous projection's GEMM "
                         "(+2 %% throughput measured; the per-kernel GEMM intervals then include the shared time)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
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
