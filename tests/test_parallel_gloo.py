"""CPU tests of the multi-GPU sharding logic with world_size-2 gloo ranks: the tensor-parallel
wrappers around the GEMM (column-parallel + all-gather, row-parallel + reduce-scatter) and the
expert split must reproduce the single-process result.  The GEMM on the CPU ranks is the oracle's
fp32 formula; on GPUs the same wrappers call the CUDA operator."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        from helpers import randn_bf16
        from mslk_b200 import parallel as par

        M, N, K = 64, 96, 256
        x, w = randn_bf16((M, K), 1), randn_bf16((N, K), 2, 0.02)
        xq, xs = oracle.quantize_fp8_row(x)          # quantized over the FULL row on every rank
        wq, ws = oracle.quantize_fp8_row(w)
        gemm = oracle.gemm_f8_rowwise_torch
        y_full = gemm(xq, wq, xs, ws)

        # N-sharded weights + all-gather, with and without token chunking
        wq_r, ws_r = par.shard_weight_rows(wq, ws, rank, world)
        for chunks in (1, 3):
            y = par.ColumnParallelLinear(wq_r, ws_r, gemm, chunks=chunks).forward(xq, xs)
            assert y.shape == (M, N) and torch.equal(y, y_full), f"column parallel chunks={chunks}"

        # K-sharded operands + reduce-scatter over tokens
        y_part = par.RowParallelLinear(par.shard_k(wq, rank, world), ws, gemm).forward(par.shard_k(xq, rank, world), xs)
        a, b = par.shard_range(M, rank, world)
        assert y_part.shape == (M // world, N)
        torch.testing.assert_close(y_part.float(), y_full[a:b].float(), rtol=1.6e-2, atol=1e-2)

        # expert split of a stacked grouped problem: ranks own disjoint expert and row ranges
        m_sizes = [5, 0, 7, 3]
        row0, row1, (e0, e1) = par.expert_token_range(m_sizes, rank, world)
        tokens = randn_bf16((sum(m_sizes), K), 3)
        tq, ts = oracle.quantize_fp8_row(tokens)
        we = randn_bf16((4, N, K), 4, 0.02)
        weq, wes = oracle.quantize_fp8_row(we)
        y_all = oracle.gemm_f8_rowwise_grouped_stacked_torch(tq, weq, ts, wes, m_sizes)
        y_mine = oracle.gemm_f8_rowwise_grouped_stacked_torch(tq[row0:row1], weq[e0:e1], ts[row0:row1], wes[e0:e1], m_sizes[e0:e1])
        assert torch.equal(y_mine, y_all[row0:row1])
        gathered = [None] * world
        dist.all_gather_object(gathered, (row0, row1))
        assert gathered[0][1] == gathered[1][0] and gathered[-1][1] == sum(m_sizes)
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_tensor_and_expert_parallel_match_single_process(tmp_path):
    world = 2
    port = 29500 + (os.getpid() % 400)
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_shard_helpers():
    from mslk_b200 import parallel as par
    assert par.shard_range(16, 3, 8) == (6, 8)
    assert par.expert_slice(16, 1, 2) == (8, 16)
    with pytest.raises(ValueError):
        par.shard_range(10, 0, 4)
    assert par.expert_token_range([4, 0, 6, 2], 1, 2) == (4, 12, (2, 4))


def test_balanced_expert_assignment():
    from mslk_b200 import parallel as par
    counts = [279, 343, 365, 576, 320, 412, 248, 716, 1645, 0, 0, 6481, 840, 1078, 475, 2606]
    for world in (1, 2, 4, 8):
        experts, load = par.balanced_expert_assignment(counts, world)
        assert sorted(e for r in experts for e in r) == list(range(16))          # every expert exactly once
        assert load == [sum(counts[e] for e in r) for r in experts]
        assert all(r == sorted(r) for r in experts)
        # greedy longest-first is within 4/3 of the optimum, and never worse than the contiguous split
        contiguous = max(sum(counts[r * (16 // world):(r + 1) * (16 // world)]) for r in range(world))
        bound = max(max(counts), -(-sum(counts) // world))
        assert max(load) <= contiguous and max(load) <= (4 * bound + 2) // 3
    experts, load = par.balanced_expert_assignment(counts, 8)
    assert max(load) == 6481                                                      # the largest expert alone is the bound
    rows = par.expert_rows(counts, experts[0])
    assert all(b - a == counts[e] for (a, b), e in zip(rows, experts[0]))
