"""Tensor-parallel and expert-parallel sharding of the FP8-rowwise GEMM over the GPUs of one node.

The reference has no multi-GPU code on this path (its only collective user is the MoE layer,
``mslk/moe/layers.py:766-1030``); these helpers shard the single-device operator the way a
tensor-parallel FFN uses it, one process per GPU over ``torch.distributed`` (NCCL on GPUs, gloo
in the CPU tests):

* :class:`ColumnParallelLinear` -- weight rows (N) sharded; every rank multiplies the replicated
  activation with its ``[N/P, K]`` shard and the bf16 outputs are all-gathered.  With ``chunks > 1``
  the token dimension is cut into chunks so that the all-gather of chunk i runs on a side stream
  while chunk i+1 is being multiplied.
* :class:`RowParallelLinear` -- the reduction dimension (K) sharded; activations are quantized over
  the FULL row first (the scales are those of the unsharded problem), every rank multiplies its
  ``[:, K/P]`` slices and the partial products (already scaled, the epilogue is linear) are summed
  with a reduce-scatter over the token dimension.
* :func:`expert_slice` -- contiguous expert ranges per rank for the grouped (MoE) GEMM; tokens are
  bucketed per rank, no collective.
* :func:`balanced_expert_assignment` -- token-count-aware placement of the experts (greedy, largest
  first): with skewed routing the slowest rank of a contiguous split holds several popular experts, while
  the bound of any placement is max(largest expert, total / ranks) tokens on one rank.

The GEMM itself is passed in as ``gemm_fn(xq, wq, x_scale, w_scale) -> bf16 [M, N]`` so that the
sharding logic can be exercised on CPU ranks with the oracle's formula; on GPUs it is
``mslk_b200.ops.f8f8bf16_rowwise``.
"""

from __future__ import annotations

from typing import Callable, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

GemmFn = Callable[[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor], torch.Tensor]


def shard_range(n: int, rank: int, world: int) -> Tuple[int, int]:
    """Half-open range of the ``rank``-th of ``world`` equal contiguous shards of ``n`` items."""
    if n % world != 0:
        raise ValueError(f"{n} items do not divide evenly over {world} ranks")
    per = n // world
    return rank * per, (rank + 1) * per


def expert_slice(num_experts: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous expert range of a rank (16/8/4/2 experts per GPU at 1/2/4/8 GPUs for E = 16)."""
    return shard_range(num_experts, rank, world)


def expert_token_range(m_sizes: Sequence[int], rank: int, world: int) -> Tuple[int, int, Tuple[int, int]]:
    """Rows of the stacked token tensor that belong to the experts of ``rank``.
    Returns ``(row_begin, row_end, (expert_begin, expert_end))``."""
    e0, e1 = expert_slice(len(m_sizes), rank, world)
    row0 = int(sum(int(v) for v in m_sizes[:e0]))
    row1 = row0 + int(sum(int(v) for v in m_sizes[e0:e1]))
    return row0, row1, (e0, e1)


def balanced_expert_assignment(m_sizes: Sequence[int], world: int):
    """Greedy longest-processing-time placement: experts sorted by token count, each given to the rank with
    the fewest tokens so far (ties: fewest experts, then lowest rank).  Returns ``(experts_of_rank, load_of_rank)``
    with the expert ids of every rank in ascending order.  The weights of a rank are gathered ONCE with that
    index list (``wq[experts_of_rank[r]]``); per step only the tokens are bucketed by it."""
    counts = [int(v) for v in m_sizes]
    order = sorted(range(len(counts)), key=lambda e: (-counts[e], e))
    experts = [[] for _ in range(world)]
    load = [0] * world
    for e in order:
        r = min(range(world), key=lambda i: (load[i], len(experts[i]), i))
        experts[r].append(e)
        load[r] += counts[e]
    return [sorted(x) for x in experts], load


def expert_rows(m_sizes: Sequence[int], experts: Sequence[int]):
    """Half-open row ranges, in the stacked token tensor, of the given experts (for bucketing tokens by a
    non-contiguous expert placement)."""
    starts = [0]
    for v in m_sizes:
        starts.append(starts[-1] + int(v))
    return [(starts[e], starts[e + 1]) for e in experts]


class ColumnParallelLinear:
    """``y[M, N] = all_gather_N(gemm(xq, wq[rank]))`` with ``wq`` sharded over its rows."""

    def __init__(self, wq_shard: torch.Tensor, w_scale_shard: torch.Tensor, gemm_fn: GemmFn,
                 group: Optional[dist.ProcessGroup] = None, chunks: int = 1):
        self.wq, self.ws, self.gemm, self.group = wq_shard, w_scale_shard, gemm_fn, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.chunks = max(1, chunks)
        self.comm_stream = torch.cuda.Stream() if wq_shard.is_cuda and self.chunks > 1 and self.world > 1 else None

    def local(self, xq: torch.Tensor, x_scale: torch.Tensor) -> torch.Tensor:
        return self.gemm(xq, self.wq, x_scale, self.ws)

    def forward(self, xq: torch.Tensor, x_scale: torch.Tensor) -> torch.Tensor:
        M, n_local, P = xq.shape[0], self.wq.shape[0], self.world
        if P == 1:
            return self.local(xq, x_scale)
        out = torch.empty((M, P * n_local), dtype=torch.bfloat16, device=xq.device)
        bounds = [M * c // self.chunks for c in range(self.chunks + 1)]
        for c in range(self.chunks):
            r0, r1 = bounds[c], bounds[c + 1]
            if r1 == r0:
                continue
            y = self.local(xq[r0:r1], x_scale[r0:r1])
            # rank-major concatenation [P * rows, N/P] (the shape every backend accepts)
            gathered = torch.empty((P * (r1 - r0), n_local), dtype=torch.bfloat16, device=xq.device)
            if self.comm_stream is not None:
                self.comm_stream.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(self.comm_stream):
                    dist.all_gather_into_tensor(gathered, y, group=self.group)
                    # [P, rows, N/P] -> columns of the row-major [rows, N] result
                    out[r0:r1].view(r1 - r0, P, n_local).copy_(gathered.view(P, r1 - r0, n_local).permute(1, 0, 2))
                y.record_stream(self.comm_stream)
                gathered.record_stream(self.comm_stream)
            else:
                dist.all_gather_into_tensor(gathered, y, group=self.group)
                out[r0:r1].view(r1 - r0, P, n_local).copy_(gathered.view(P, r1 - r0, n_local).permute(1, 0, 2))
        if self.comm_stream is not None:
            torch.cuda.current_stream().wait_stream(self.comm_stream)
        return out


class RowParallelLinear:
    """``y[M/P, N] = reduce_scatter_M(gemm(xq[:, shard], wq[:, shard]))`` with K sharded."""

    def __init__(self, wq_kshard: torch.Tensor, w_scale: torch.Tensor, gemm_fn: GemmFn,
                 group: Optional[dist.ProcessGroup] = None):
        self.wq, self.ws, self.gemm, self.group = wq_kshard, w_scale, gemm_fn, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1

    def local(self, xq_kshard: torch.Tensor, x_scale: torch.Tensor) -> torch.Tensor:
        # x_scale / w_scale are the FULL-row scales: (sum_k over the shard) * xs * ws is this rank's
        # additive share of the unsharded result
        return self.gemm(xq_kshard, self.wq, x_scale, self.ws)

    def forward(self, xq_kshard: torch.Tensor, x_scale: torch.Tensor) -> torch.Tensor:
        partial = self.local(xq_kshard, x_scale)
        if self.world == 1:
            return partial
        M, N = partial.shape
        if M % self.world != 0:
            raise ValueError(f"{M} rows do not divide evenly over {self.world} ranks")
        out = torch.empty((M // self.world, N), dtype=partial.dtype, device=partial.device)
        dist.reduce_scatter_tensor(out, partial, op=dist.ReduceOp.SUM, group=self.group)
        return out


def shard_weight_rows(wq: torch.Tensor, w_scale: torch.Tensor, rank: int, world: int):
    """Rows ``[rank*N/P, (rank+1)*N/P)`` of an already quantized ``[N, K]`` weight and its scales."""
    a, b = shard_range(wq.shape[0], rank, world)
    return wq[a:b].contiguous(), w_scale[a:b].contiguous()


def shard_k(q: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Columns ``[rank*K/P, (rank+1)*K/P)`` of a quantized ``[rows, K]`` tensor as a contiguous copy
    (the GEMM reads contiguous operands; K/P must keep the 16-byte row rule)."""
    a, b = shard_range(q.shape[1], rank, world)
    return q[:, a:b].contiguous()
