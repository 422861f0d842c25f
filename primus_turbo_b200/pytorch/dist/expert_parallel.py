"""Expert-parallel wrapper for the grouped GEMM: experts are sharded contiguously over the ranks
(expert ``e`` lives on rank ``e // (E / world)``) and routed rows travel to their expert's owner
with one all-to-all before the local grouped GEMM and one after it.

The reference never shards ``grouped_gemm_fp8`` itself; its callers wrap it between a token
dispatch and combine (primus_turbo/pytorch/ops/moe/moe_dispatch_combine.py:20-101, backed by its
DeepEP port).  Here the exchange is a plain ``torch.distributed.all_to_all_single`` (NCCL over
NVLink on GPUs, gloo on CPU for the host-logic tests); remote rows always land in local memory
first and the GEMM kernels only ever read local memory.

Every rank holds ``x_local`` whose rows are sorted by *global* expert id, with
``counts_local[e]`` rows for expert ``e``.  ``expert_parallel_apply`` returns, for each local row
and in the same order, the output of that row's expert.  All pieces are autograd Functions, so
the backward pass performs the mirrored exchanges (grad_out dispatched, grad_x combined; weight
gradients stay with the expert's owner).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional

import torch
import torch.distributed as dist

__all__ = ["ExchangePlan", "build_exchange_plan", "expert_parallel_apply", "ep_grouped_gemm_fp8"]


@dataclass
class ExchangePlan:
    """Everything the two exchanges need, derived from the [world, E] routing count matrix."""

    send_splits: List[int]  # rows this rank sends to each destination rank
    recv_splits: List[int]  # rows this rank receives from each source rank
    gather_index: torch.Tensor  # [rows_recv] int64: expert-major row j comes from arrival row gather_index[j]
    group_lens: torch.Tensor  # [E_local] int64 rows per local expert after the exchange
    counts_matrix: torch.Tensor  # [world, E] int64 (device of the payload)


def build_exchange_plan(
    counts_local: torch.Tensor,
    group: Optional[dist.ProcessGroup] = None,
    counts_host: Optional[torch.Tensor] = None,
    host_group: Optional[dist.ProcessGroup] = None,
) -> ExchangePlan:
    """Derive the exchange from the per-expert row counts of every rank.

    ``counts_local``: int64 ``[E]`` on the payload's device.  The all-to-all needs its split sizes on
    the host.  By default they are read back from the device (one small all-gather plus one host
    synchronisation).  A caller that already holds its counts on the host passes ``counts_host``
    (CPU int64 ``[E]``) and a CPU process group (``host_group``, e.g. gloo): the counts are then
    gathered on the host and the device stream is never waited on.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    E = counts_local.numel()
    assert E % world == 0, f"{E} experts cannot be sharded evenly over {world} ranks"
    e_loc = E // world
    dev = counts_local.device
    if counts_host is not None:
        assert host_group is not None and not counts_host.is_cuda
        flat_h = torch.empty(world * E, dtype=torch.int64)
        dist.all_gather_into_tensor(flat_h, counts_host.to(torch.int64).contiguous(), group=host_group)
        host_matrix = flat_h.view(world, E)
        matrix = host_matrix.to(dev, non_blocking=True)
    else:
        flat = torch.empty(world * E, dtype=torch.int64, device=dev)
        dist.all_gather_into_tensor(flat, counts_local.to(torch.int64).contiguous(), group=group)
        matrix = flat.view(world, E)
        host_matrix = matrix.cpu()  # the one host synchronisation of the exchange
    per_dest = host_matrix.view(world, world, e_loc).sum(-1)  # [src, dst]
    send_splits = per_dest[rank].tolist()
    recv_splits = per_dest[:, rank].tolist()
    mine = matrix[:, rank * e_loc : (rank + 1) * e_loc]  # [src, e_local] rows arriving per source and expert
    # arrival order is (source, expert); the grouped GEMM wants (expert, source)
    arrive_start = (torch.cumsum(mine.reshape(-1), 0) - mine.reshape(-1)).view(world, e_loc)
    cnt_es = mine.t().reshape(-1)  # segments in (expert, source) order
    src_start_es = arrive_start.t().reshape(-1)
    dst_start_es = torch.cumsum(cnt_es, 0) - cnt_es
    total = int(sum(recv_splits))
    gather_index = torch.repeat_interleave(src_start_es - dst_start_es, cnt_es, output_size=total) + torch.arange(
        total, device=dev
    )
    return ExchangePlan(send_splits, recv_splits, gather_index, mine.sum(0).contiguous(), matrix)


class _AllToAllRows(torch.autograd.Function):
    """Row exchange; the gradient travels the same links in the opposite direction."""

    @staticmethod
    def forward(ctx, x, in_splits, out_splits, group):
        ctx.in_splits, ctx.out_splits, ctx.group = in_splits, out_splits, group
        out = x.new_empty((sum(out_splits), *x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        gx = g.new_empty((sum(ctx.in_splits), *g.shape[1:]))
        dist.all_to_all_single(gx, g.contiguous(), ctx.in_splits, ctx.out_splits, group=ctx.group)
        return gx, None, None, None


class _GatherRows(torch.autograd.Function):
    """y = x[index] for a permutation ``index``; backward scatters with the same permutation."""

    @staticmethod
    def forward(ctx, x, index):
        ctx.save_for_backward(index)
        return x.index_select(0, index)

    @staticmethod
    def backward(ctx, g):
        (index,) = ctx.saved_tensors
        gx = torch.empty_like(g)
        gx.index_copy_(0, index, g)
        return gx, None


class _ScatterRows(torch.autograd.Function):
    """y[index] = x (inverse of _GatherRows)."""

    @staticmethod
    def forward(ctx, x, index):
        ctx.save_for_backward(index)
        y = torch.empty_like(x)
        y.index_copy_(0, index, x)
        return y

    @staticmethod
    def backward(ctx, g):
        (index,) = ctx.saved_tensors
        return g.index_select(0, index), None


def expert_parallel_apply(
    x_local: torch.Tensor,
    counts_local: torch.Tensor,
    local_fn: Callable[[torch.Tensor, torch.Tensor], torch.Tensor],
    group: Optional[dist.ProcessGroup] = None,
    plan: Optional[ExchangePlan] = None,
) -> torch.Tensor:
    """Dispatch rows to their experts' owners, run ``local_fn(rows_expert_major, group_lens)`` there,
    and bring each result row back to where its input row came from."""
    if plan is None:
        plan = build_exchange_plan(counts_local, group)
    arrived = _AllToAllRows.apply(x_local, plan.send_splits, plan.recv_splits, group)
    by_expert = _GatherRows.apply(arrived, plan.gather_index)
    y = local_fn(by_expert, plan.group_lens)
    y_arrival_order = _ScatterRows.apply(y, plan.gather_index)
    return _AllToAllRows.apply(y_arrival_order, plan.recv_splits, plan.send_splits, group)


def ep_grouped_gemm_fp8(
    x_local: torch.Tensor,
    w_local: torch.Tensor,
    counts_local: torch.Tensor,
    group: Optional[dist.ProcessGroup] = None,
    trans_b: bool = True,
    config=None,
    plan: Optional[ExchangePlan] = None,
) -> torch.Tensor:
    """Expert-parallel ``grouped_gemm_fp8``: ``w_local`` holds this rank's ``E / world`` experts."""
    from primus_turbo_b200.pytorch.ops.grouped_gemm_fp8 import grouped_gemm_fp8

    def local_fn(rows, group_lens):
        return grouped_gemm_fp8(rows, w_local, group_lens, trans_b=trans_b, config=config)

    return expert_parallel_apply(x_local, counts_local, local_fn, group, plan)
