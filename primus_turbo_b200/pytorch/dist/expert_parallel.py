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

__all__ = [
    "ExchangePlan", "build_exchange_plan", "expert_parallel_apply", "ep_grouped_gemm_fp8", "BlockwiseLocalSteps",
    "SharedCountsBoard", "PeerPlan", "build_peer_plan", "expert_parallel_apply_peer", "ep_grouped_gemm_fp8_peer",
    "balanced_expert_order",
    "load_imbalance",
]


@dataclass
class ExchangePlan:
    """Everything the two exchanges need, derived from the [world, E] routing count matrix."""

    send_splits: List[int]  # rows this rank sends to each destination rank
    recv_splits: List[int]  # rows this rank receives from each source rank
    gather_index: torch.Tensor  # [rows_recv] int64: expert-major row j comes from arrival row gather_index[j]
    scatter_index: torch.Tensor  # [rows_recv] int64: the inverse permutation (arrival row i is expert-major row scatter_index[i])
    group_lens: torch.Tensor  # [E_local] int64 rows per local expert after the exchange
    counts_matrix: torch.Tensor  # [world, E] int64 (device of the payload)


class SharedCountsBoard:
    """Host-side gather of every rank's routing counts for ranks that share one machine.

    ``all_to_all_single`` needs its split sizes on the host every step.  A CPU collective (gloo
    over loopback TCP) was measured at 1.9 ms per call with two ranks and 3.7 ms with eight, which
    made an eight-GPU step host-bound; this board is a small file in shared memory, mapped by every rank, that each rank
    writes its row into and reads the others' rows from, with a per-row sequence number (tens of
    microseconds).  Rows are double-buffered by call parity: a rank can only start call ``s + 2``
    after every rank has written call ``s + 1``, which each does only after reading all of call
    ``s``, so a slot is never overwritten while someone still reads it.

    The sequence number is stored after the counts and read before them; that is enough on hosts
    with total store order (x86, which the HGX B200 boxes are).  A weakly ordered host CPU would need
    a fence between the two stores.

    Construction is collective over ``group`` (any backend; one object broadcast).  ``close()`` (or
    process exit) drops the mapping; the creating rank removes the file.
    """

    def __init__(self, num_experts: int, group: Optional[dist.ProcessGroup] = None, timeout_s: float = 120.0):
        import atexit
        import os
        import uuid

        import numpy as np

        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.E = int(num_experts)
        self.timeout_s = timeout_s
        self._calls = 0
        shape = (2, self.world, self.E + 1)
        root = "/dev/shm" if os.path.isdir("/dev/shm") else None  # a file mapped by every rank
        path = [None]
        if self.rank == 0:
            import tempfile

            fd, path[0] = tempfile.mkstemp(prefix=f"ptb_counts_{uuid.uuid4().hex[:8]}_", dir=root)
            os.ftruncate(fd, 8 * shape[0] * shape[1] * shape[2])  # zero-filled
            os.close(fd)
        src = dist.get_global_rank(group, 0) if group is not None else 0
        dist.broadcast_object_list(path, src=src, group=group)
        self._path = path[0]
        self._board = np.memmap(self._path, dtype=np.int64, mode="r+", shape=shape)
        dist.barrier(group=group)  # every rank has mapped the file before the first write
        atexit.register(self.close)

    def all_gather_counts(self, counts_host: torch.Tensor) -> torch.Tensor:
        """[E] int64 on the host from every rank -> [world, E] int64 on the host."""
        import time

        self._calls += 1
        seq, slot = self._calls, self._calls & 1
        row = self._board[slot, self.rank]
        row[: self.E] = counts_host.to(torch.int64).numpy()
        row[self.E] = seq  # written after the counts: readers take the row only once they see it
        out = torch.empty((self.world, self.E), dtype=torch.int64)
        out_np = out.numpy()
        deadline = None
        polls = 0
        for r in range(self.world):
            src = self._board[slot, r]
            while src[self.E] != seq:
                polls += 1
                if polls > 200:
                    # a rank that is late is late by far more than a poll: give the core away instead of
                    # burning the job's CPU share (eight spinning ranks starve one another on a busy host)
                    time.sleep(2e-5)
                    if deadline is None:
                        deadline = time.monotonic() + self.timeout_s
                    elif time.monotonic() > deadline:
                        raise RuntimeError(f"rank {self.rank}: no routing counts from rank {r} after {self.timeout_s} s")
            out_np[r] = src[: self.E]
        return out

    def close(self) -> None:
        import os

        board, self._board = getattr(self, "_board", None), None
        if board is None:
            return
        del board
        if self.rank == 0:
            try:
                os.unlink(self._path)  # mappings held by other ranks stay valid until they drop them
            except OSError:
                pass


class _PinnedPool:
    """Page-locked staging buffers for the plan's one host-to-device copy.  A copy from pageable
    memory makes the host wait for the stream, which would expose every launch of the step; a
    pinned source does not.  A buffer is reused only after the copy that read it has completed.  The
    pool grows to ``LIMIT`` buffers and then waits for its oldest copy instead of allocating: page-locked
    allocation and release cost a quarter of a millisecond each and synchronise with the device, and a
    host that runs many steps ahead of the GPU would otherwise pay both on every step."""

    LIMIT = 16

    def __init__(self):
        self._items = []  # (buffer, event), oldest first

    def take(self, numel: int):
        for i, (buf, ev) in enumerate(self._items):
            if buf.numel() >= numel and ev.query():
                return self._items.pop(i)[0]
        if len(self._items) >= self.LIMIT:
            for i, (buf, ev) in enumerate(self._items):
                if buf.numel() >= numel:
                    ev.synchronize()  # the host is LIMIT plans ahead of the device: let it catch up
                    return self._items.pop(i)[0]
        return torch.empty(max(numel, 1 << 16), dtype=torch.int64, pin_memory=True)

    def give_back(self, buf: torch.Tensor, ev):
        self._items.append((buf, ev))


_pinned_pool = _PinnedPool()


def _plan_from_matrix(matrix: torch.Tensor, rank: int, world: int):
    """Index arithmetic of the plan on whatever device ``matrix`` ([world, E] int64) lives on."""
    E = matrix.shape[1]
    e_loc = E // world
    dev = matrix.device
    mine = matrix[:, rank * e_loc : (rank + 1) * e_loc]  # [src, e_local] rows arriving per source and expert
    # arrival order is (source, expert); the grouped GEMM wants (expert, source)
    flat = mine.reshape(-1)
    arrive_start = (torch.cumsum(flat, 0) - flat).view(world, e_loc)
    cnt_es = mine.t().reshape(-1)  # segments in (expert, source) order
    src_start_es = arrive_start.t().reshape(-1)
    dst_start_es = torch.cumsum(cnt_es, 0) - cnt_es
    return mine, cnt_es, src_start_es - dst_start_es, dev


def build_exchange_plan(
    counts_local: torch.Tensor,
    group: Optional[dist.ProcessGroup] = None,
    counts_host: Optional[torch.Tensor] = None,
    host_group: Optional[dist.ProcessGroup] = None,
) -> ExchangePlan:
    """Derive the exchange from the per-expert row counts of every rank.

    ``counts_local``: int64 ``[E]`` on the payload's device.  The all-to-all needs its split sizes on
    the host.  By default they are read back from the device (one small all-gather plus one host
    synchronisation) and the permutations are computed on the device.  A caller that already holds
    its counts on the host passes ``counts_host`` (CPU int64 ``[E]``) and either a CPU process group
    (``host_group``, e.g. gloo) or, for ranks on one machine, a ``SharedCountsBoard`` (much lower
    latency): counts are gathered and the whole plan is computed on the host, and
    reaches the device as one copy from pinned memory, so the device stream is never waited on and
    no small kernel is launched.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    E = counts_local.numel()
    assert E % world == 0, f"{E} experts cannot be sharded evenly over {world} ranks"
    e_loc = E // world
    dev = counts_local.device
    if counts_host is not None:
        assert host_group is not None and not counts_host.is_cuda
        if isinstance(host_group, SharedCountsBoard):
            host_matrix = host_group.all_gather_counts(counts_host)
            flat_h = host_matrix.view(-1)
        else:
            flat_h = torch.empty(world * E, dtype=torch.int64)
            dist.all_gather_into_tensor(flat_h, counts_host.to(torch.int64).contiguous(), group=host_group)
            host_matrix = flat_h.view(world, E)
        mine, cnt_es, shift_es, _ = _plan_from_matrix(host_matrix, rank, world)
        total = int(mine.sum())
        gather_h = torch.repeat_interleave(shift_es, cnt_es, output_size=total) + torch.arange(total)
        scatter_h = torch.empty(total, dtype=torch.int64)
        scatter_h[gather_h] = torch.arange(total)
        lens_h = mine.sum(0)
        parts = [gather_h, scatter_h, lens_h, flat_h]
        numel = sum(p.numel() for p in parts)
        if dev.type == "cuda":
            staging = _pinned_pool.take(numel)
            torch.cat(parts, out=staging[:numel])
            packed = staging[:numel].to(dev, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(dev))
            _pinned_pool.give_back(staging, ev)
        else:
            packed = torch.cat(parts)
        gather_index, scatter_index, group_lens, mat = torch.split(packed, [p.numel() for p in parts])
        matrix = mat.view(world, E)
    else:
        flat = torch.empty(world * E, dtype=torch.int64, device=dev)
        dist.all_gather_into_tensor(flat, counts_local.to(torch.int64).contiguous(), group=group)
        matrix = flat.view(world, E)
        host_matrix = matrix.cpu()  # the one host synchronisation of the exchange
        mine, cnt_es, shift_es, _ = _plan_from_matrix(matrix, rank, world)
        total = int(host_matrix[:, rank * e_loc : (rank + 1) * e_loc].sum())
        ar = torch.arange(total, device=dev)
        gather_index = torch.repeat_interleave(shift_es, cnt_es, output_size=total) + ar
        scatter_index = torch.empty_like(gather_index)
        scatter_index[gather_index] = ar
        group_lens = mine.sum(0).contiguous()
    per_dest = host_matrix.view(world, world, e_loc).sum(-1)  # [src, dst]
    send_splits = per_dest[rank].tolist()
    recv_splits = per_dest[:, rank].tolist()
    return ExchangePlan(send_splits, recv_splits, gather_index, scatter_index, group_lens, matrix)


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


def _gather(x: torch.Tensor, index: torch.Tensor) -> torch.Tensor:
    """Row gather: the library's kernel for CUDA rows of 16-byte multiples, torch otherwise (CPU tests)."""
    if x.is_cuda and x.dim() == 2 and (x.shape[1] * x.element_size()) % 16 == 0:
        from primus_turbo_b200.pytorch.kernels.quantization_impl import gather_rows

        return gather_rows(x, index)
    return x.index_select(0, index)


class _PermuteRows(torch.autograd.Function):
    """y = x[index] for a permutation ``index`` with inverse ``inverse``.  Both directions are row
    gathers (``index_select``): a gather streams at HBM speed, a scatter through ``index_copy_``
    measured seven times slower on the same rows."""

    @staticmethod
    def forward(ctx, x, index, inverse):
        ctx.save_for_backward(index, inverse)
        return _gather(x, index)

    @staticmethod
    def backward(ctx, g):
        index, inverse = ctx.saved_tensors
        return _gather(g, inverse), None, None


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
    by_expert = _PermuteRows.apply(arrived, plan.gather_index, plan.scatter_index)
    y = local_fn(by_expert, plan.group_lens)
    y_arrival_order = _PermuteRows.apply(y, plan.scatter_index, plan.gather_index)
    return _AllToAllRows.apply(y_arrival_order, plan.recv_splits, plan.send_splits, group)


class BlockwiseLocalSteps:
    """The device steps of one blockwise ``grouped_gemm_fp8`` forward + backward, callable one by one
    (the same kernel calls ``FP8GroupedGemmBlockFunc`` makes) so that the expert-parallel wrapper can
    place them around its exchanges.  A host-logic test substitutes plain-torch steps."""

    def __init__(self, config, trans_b: bool, out_dtype: torch.dtype):
        from primus_turbo_b200.pytorch.core.low_precision import ScalingGranularity

        assert config.granularity == ScalingGranularity.BLOCKWISE and config.block_size == 128
        self.config, self.trans_b, self.out_dtype = config, trans_b, out_dtype

    def offsets(self, group_lens):
        from primus_turbo_b200.pytorch.kernels.gemm_impl import group_offs_from_lens

        return group_offs_from_lens(group_lens)

    def _dt(self, fwd: bool):
        from primus_turbo_b200.pytorch.ops.grouped_gemm_fp8 import _get_fp8_dtype

        return _get_fp8_dtype(self.config.format, fwd)

    def quant_weight(self, w):
        from primus_turbo_b200.pytorch.core.quantized_tensor import QuantizedTensor
        from primus_turbo_b200.pytorch.kernels.quantization_impl import quant_fp8_blockwise_for_weight_impl

        if isinstance(w, QuantizedTensor):  # quantised ahead of time (create_quantized_weight)
            return w.qdata, w.scale_inv
        return quant_fp8_blockwise_for_weight_impl(w, self._dt(True), 128)

    def quant_rows(self, x, lens, offs, fwd: bool):
        """-> (row copy, column copy, row scales, column scales, padded lens, padded offsets)"""
        from primus_turbo_b200.pytorch.kernels.quantization_impl import quant_fp8_blockwise_segment_m_row_col_impl

        return quant_fp8_blockwise_segment_m_row_col_impl(x.contiguous(), self._dt(fwd), 128, lens, offs)

    def _gemm(self, a, a_s, b8, b_s, lens, offs, trans_b):
        from primus_turbo_b200.pytorch.kernels.gemm_impl import grouped_gemm_fp8_impl

        return grouped_gemm_fp8_impl(
            a, b8, a_s, b_s, lens, offs, trans_a=False, trans_b=trans_b, out_dtype=self.out_dtype,
            granularity=self.config.granularity.value, num_cu=None,
        )

    def fwd(self, a_row, a_s_row, b8, b_s, lens, offs):
        return self._gemm(a_row, a_s_row, b8, b_s, lens, offs, self.trans_b)

    def dgrad(self, g_row, g_s_row, b8, b_s, lens, offs):
        return self._gemm(g_row, g_s_row, b8, b_s, lens, offs, not self.trans_b)

    def wgrad(self, a_col, a_s_col, g_col, g_s_col, vk_lens, vk_offs, num_cu=None):
        from primus_turbo_b200.pytorch.kernels.gemm_impl import grouped_gemm_fp8_variable_k_impl

        return grouped_gemm_fp8_variable_k_impl(
            a_col, g_col, a_s_col, g_s_col, vk_lens, vk_offs, trans_a=True, trans_b=False, trans_c=self.trans_b,
            out_dtype=self.out_dtype, granularity=self.config.granularity.value, num_cu=num_cu,
        )


_side_streams = {}


def _side_stream(device: torch.device) -> "torch.cuda.Stream":
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(device=key)
    return _side_streams[key]


class _Fork:
    """Runs a block of device work on a side stream that starts where the current stream stands
    (``begin``) and is joined back later (``join``); on CPU tensors it does nothing."""

    def __init__(self, ref: torch.Tensor):
        self.cuda = ref.is_cuda
        if self.cuda:
            self.cur = torch.cuda.current_stream(ref.device)
            self.side = _side_stream(ref.device)

    def begin(self):
        if self.cuda:
            self.side.wait_stream(self.cur)

    def stream(self):
        import contextlib

        return torch.cuda.stream(self.side) if self.cuda else contextlib.nullcontext()

    def uses(self, *tensors):
        """tensors allocated on the current stream that the side stream reads"""
        if self.cuda:
            for t in tensors:
                t.record_stream(self.side)

    def join(self, *produced):
        """make the current stream wait for the side stream; `produced` were allocated there"""
        if self.cuda:
            self.cur.wait_stream(self.side)
            for t in produced:
                t.record_stream(self.cur)


class _EPBlockwiseOverlapped(torch.autograd.Function):
    """Dispatch -> blockwise grouped GEMM -> combine as one autograd node, so that the two steps that
    need nothing from an exchange run beside it on a second stream: the weight quantisation beside
    the forward dispatch, and wgrad beside the return of the activation gradient.  wgrad is a
    persistent kernel (one CTA per SM): it is launched on ``148 - reserve_sms`` SMs so that the
    collective's CTAs, launched first, and all of its own CTAs are resident together.

    Measured on two B200s at the benchmark shape this form is *slower* than the serial chain
    (12.9 ms against 11.8 ms per step): the weight quantisation, wgrad and the all-to-all are all
    bound by HBM bandwidth, so running them side by side stretches each by what the other takes.
    It stays selectable (``overlap=True``) for shapes whose local GEMMs are tensor-bound."""

    @staticmethod
    def forward(ctx, x_local, w_local, plan, group, steps, reserve_sms):
        fork = _Fork(x_local)
        fork.begin()
        arrived = x_local.new_empty((sum(plan.recv_splits), *x_local.shape[1:]))
        work = dist.all_to_all_single(
            arrived, x_local.contiguous(), plan.recv_splits, plan.send_splits, group=group, async_op=True
        )
        with fork.stream():
            b8, b_s = steps.quant_weight(w_local)
        work.wait()
        rows = arrived.index_select(0, plan.gather_index)
        lens = plan.group_lens
        offs = steps.offsets(lens)
        a_row, a_col, a_s_row, a_s_col, _, _ = steps.quant_rows(rows, lens, offs, True)
        fork.join(b8, b_s)
        y = steps.fwd(a_row, a_s_row, b8, b_s, lens, offs)
        y_arrival = y.index_select(0, plan.scatter_index)
        out = y.new_empty((sum(plan.send_splits), *y.shape[1:]))
        dist.all_to_all_single(out, y_arrival, plan.send_splits, plan.recv_splits, group=group)
        ctx.save_for_backward(a_col, a_s_col, b8, b_s, lens, offs, plan.gather_index, plan.scatter_index)
        ctx.plan, ctx.group, ctx.steps, ctx.reserve_sms = plan, group, steps, reserve_sms
        return out

    @staticmethod
    def backward(ctx, g):
        a_col, a_s_col, b8, b_s, lens, offs, gather_index, scatter_index = ctx.saved_tensors
        plan, group, steps = ctx.plan, ctx.group, ctx.steps
        g_arrival = g.new_empty((sum(plan.recv_splits), *g.shape[1:]))
        dist.all_to_all_single(g_arrival, g.contiguous(), plan.recv_splits, plan.send_splits, group=group)
        gy = g_arrival.index_select(0, gather_index)
        g_row, g_col, g_s_row, g_s_col, vk_lens, vk_offs = steps.quant_rows(gy, lens, offs, False)
        ga = steps.dgrad(g_row, g_s_row, b8, b_s, lens, offs)
        ga_arrival = ga.index_select(0, scatter_index)
        gx = ga.new_empty((sum(plan.send_splits), *ga.shape[1:]))
        fork = _Fork(g)
        fork.begin()
        work = dist.all_to_all_single(gx, ga_arrival, plan.send_splits, plan.recv_splits, group=group, async_op=True)
        num_cu = None
        if fork.cuda and ctx.reserve_sms > 0:
            num_cu = max(1, torch.cuda.get_device_properties(g.device).multi_processor_count - ctx.reserve_sms)
        with fork.stream():
            fork.uses(a_col, a_s_col, g_col, g_s_col, vk_lens, vk_offs)
            gw = steps.wgrad(a_col, a_s_col, g_col, g_s_col, vk_lens, vk_offs, num_cu)
        work.wait()
        fork.join(gw)
        return gx, gw, None, None, None, None


def ep_grouped_gemm_fp8(
    x_local: torch.Tensor,
    w_local: torch.Tensor,
    counts_local: torch.Tensor,
    group: Optional[dist.ProcessGroup] = None,
    trans_b: bool = True,
    config=None,
    plan: Optional[ExchangePlan] = None,
    overlap: bool = False,
    reserve_sms: int = 16,
    steps=None,
) -> torch.Tensor:
    """Expert-parallel ``grouped_gemm_fp8``: ``w_local`` holds this rank's ``E / world`` experts.

    ``overlap=True`` (blockwise granularity only) uses the single-node form that runs the weight
    quantisation beside the dispatch and wgrad beside the return of the activation gradient; the
    results are bit-identical to ``overlap=False``.  ``steps`` replaces the device steps (tests).
    """
    from primus_turbo_b200.pytorch.ops.grouped_gemm_fp8 import grouped_gemm_fp8

    if overlap:
        if plan is None:
            plan = build_exchange_plan(counts_local, group)
        if steps is None:
            from primus_turbo_b200.pytorch.core.low_precision import Float8QuantConfig

            cfg = config if config is not None else Float8QuantConfig()
            steps = BlockwiseLocalSteps(cfg, trans_b, torch.promote_types(x_local.dtype, w_local.dtype))
        return _EPBlockwiseOverlapped.apply(x_local, w_local, plan, group, steps, reserve_sms)

    def local_fn(rows, group_lens):
        return grouped_gemm_fp8(rows, w_local, group_lens, trans_b=trans_b, config=config)

    return expert_parallel_apply(x_local, counts_local, local_fn, group, plan)


# ---------------------------------------------------------------------------------------------------
# Peer-memory exchange (one node): rows are written straight to their expert-major position
# ---------------------------------------------------------------------------------------------------
@dataclass
class PeerPlan:
    """Per-step plan of the peer-memory exchange (``peer_exchange.py``): the host-side tables plus their
    device copies (uploaded as one copy from pinned memory)."""

    tables: "object"  # peer_exchange.SegmentTables (host)
    seg_dev: tuple  # (dispatch [E,4], combine [E,4]) int64 on the device
    group_lens: torch.Tensor  # [E_local] int64 on the device
    counts_matrix: torch.Tensor  # [world, E] int64 on the host


def build_peer_plan(counts_host: torch.Tensor, host_group, device, group: Optional[dist.ProcessGroup] = None) -> PeerPlan:
    """Gather every rank's host-side routing counts (``SharedCountsBoard`` or a CPU process group) and
    derive both exchanges' row segments; nothing here waits on the device."""
    from primus_turbo_b200.pytorch.dist.peer_exchange import segment_tables

    world, rank = dist.get_world_size(group), dist.get_rank(group)
    E = counts_host.numel()
    if isinstance(host_group, SharedCountsBoard):
        matrix = host_group.all_gather_counts(counts_host)
    else:
        flat = torch.empty(world * E, dtype=torch.int64)
        dist.all_gather_into_tensor(flat, counts_host.to(torch.int64).contiguous(), group=host_group)
        matrix = flat.view(world, E)
    tables = segment_tables(matrix, rank)
    parts = [tables.dispatch.reshape(-1), tables.combine.reshape(-1), tables.group_lens]
    numel = sum(p.numel() for p in parts)
    dev = torch.device(device)
    if dev.type == "cuda":
        staging = _pinned_pool.take(numel)
        torch.cat(parts, out=staging[:numel])
        packed = staging[:numel].to(dev, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(dev))
        _pinned_pool.give_back(staging, ev)
    else:
        packed = torch.cat(parts)
    d, c, lens = torch.split(packed, [p.numel() for p in parts])
    return PeerPlan(tables, (d.view(-1, 4), c.view(-1, 4)), lens, matrix)


def expert_parallel_apply_peer(x_local: torch.Tensor, local_fn: Callable[[torch.Tensor, torch.Tensor], torch.Tensor],
                               exchange, plan: PeerPlan) -> torch.Tensor:
    """``expert_parallel_apply`` over peer-mapped buffers: dispatch and combine are one copy kernel each,
    rows arrive in expert-major order (no permutation pass), results are bit-identical to the
    all-to-all form."""
    from primus_turbo_b200.pytorch.dist.peer_exchange import peer_combine, peer_dispatch

    rows = peer_dispatch(x_local, exchange, plan.tables, plan.seg_dev)
    y = local_fn(rows, plan.group_lens)
    return peer_combine(y, exchange, plan.tables, plan.seg_dev)


class _EPPeerOverlapped(torch.autograd.Function):
    """Dispatch -> blockwise grouped GEMM -> combine over the peer-memory exchange as ONE autograd node, so
    that the two local steps that need nothing from an exchange run beside it on a second stream: the
    weight quantisation beside the forward dispatch (copy kernel + ordering collective), and wgrad beside
    the return of the activation gradient.  The copy kernel is launched with few CTAs (``exchange.num_ctas``,
    it is NVLink-bound) and the persistent wgrad kernel on the SMs that remain (``reserve_sms``), so both are
    resident together.  Results are bit-identical to the serial form."""

    @staticmethod
    def forward(ctx, x_local, w_local, plan, exchange, steps, reserve_sms):
        t = plan.tables
        fork = _Fork(x_local)
        fork.begin()
        with fork.stream():
            b8, b_s = steps.quant_weight(w_local)
        rows = exchange.push(x_local.contiguous(), plan.seg_dev[0], "dispatch", t.rows_out)
        exchange.order()
        lens = plan.group_lens
        offs = steps.offsets(lens)
        a_row, a_col, a_s_row, a_s_col, _, _ = steps.quant_rows(rows, lens, offs, True)
        fork.join(b8, b_s)
        y = steps.fwd(a_row, a_s_row, b8, b_s, lens, offs)
        out = exchange.push(y, plan.seg_dev[1], "combine", t.rows_in)
        exchange.order()
        ctx.save_for_backward(a_col, a_s_col, b8, b_s, lens, offs)
        ctx.plan, ctx.exchange, ctx.steps, ctx.reserve_sms = plan, exchange, steps, reserve_sms
        return out.clone()

    @staticmethod
    def backward(ctx, g):
        a_col, a_s_col, b8, b_s, lens, offs = ctx.saved_tensors
        plan, exchange, steps = ctx.plan, ctx.exchange, ctx.steps
        t = plan.tables
        gy = exchange.push(g.contiguous(), plan.seg_dev[0], "dispatch", t.rows_out, phase="bwd")
        exchange.order()
        g_row, g_col, g_s_row, g_s_col, vk_lens, vk_offs = steps.quant_rows(gy, lens, offs, False)
        ga = steps.dgrad(g_row, g_s_row, b8, b_s, lens, offs)
        fork = _Fork(g)
        fork.begin()
        num_cu = None
        if fork.cuda and ctx.reserve_sms > 0:
            num_cu = max(1, torch.cuda.get_device_properties(g.device).multi_processor_count - ctx.reserve_sms)
        gx = exchange.push(ga, plan.seg_dev[1], "combine", t.rows_in, phase="bwd")  # few CTAs: launched first
        with fork.stream():
            fork.uses(a_col, a_s_col, g_col, g_s_col, vk_lens, vk_offs)
            gw = steps.wgrad(a_col, a_s_col, g_col, g_s_col, vk_lens, vk_offs, num_cu)
        exchange.order()
        gx = gx.clone()
        fork.join(gw)
        return gx, gw, None, None, None, None


def ep_grouped_gemm_fp8_peer(x_local: torch.Tensor, w_local: torch.Tensor, exchange, plan: "PeerPlan", trans_b: bool = True,
                             config=None, overlap: bool = False, reserve_sms: int = 16, steps=None) -> torch.Tensor:
    """Expert-parallel blockwise ``grouped_gemm_fp8`` over the peer-memory exchange.  ``overlap=True`` runs the
    weight quantisation beside the dispatch and wgrad beside the return of the activation gradient (give the
    exchange a small ``num_ctas``, e.g. ``reserve_sms``, so that both kernels of a pair fit on the GPU)."""
    from primus_turbo_b200.pytorch.ops.grouped_gemm_fp8 import grouped_gemm_fp8

    if not overlap:
        return expert_parallel_apply_peer(
            x_local, lambda rows, lens: grouped_gemm_fp8(rows, w_local, lens, trans_b=trans_b, config=config), exchange, plan)
    if steps is None:
        from primus_turbo_b200.pytorch.core.low_precision import Float8QuantConfig

        cfg = config if config is not None else Float8QuantConfig()
        steps = BlockwiseLocalSteps(cfg, trans_b, torch.promote_types(x_local.dtype, w_local.dtype))
    return _EPPeerOverlapped.apply(x_local, w_local, plan, exchange, steps, reserve_sms)


def balanced_expert_order(expected_load: torch.Tensor, world: int) -> torch.Tensor:
    """Placement of ``E`` experts on ``world`` ranks, ``E / world`` each, that evens out the rows per rank:
    experts in decreasing order of expected load go to the least-loaded rank that still has room
    (longest-processing-time-first).  Returns ``order`` ([E] int64): position ``p`` of the placement holds
    global expert ``order[p]``, rank ``r`` owns positions ``[r*E/world, (r+1)*E/world)``.  The exchange
    itself always shards positions contiguously: a caller that wants this placement sorts its rows (and
    orders its counts and weights) by position instead of by global expert id."""
    load = expected_load.to(torch.float64).flatten()
    E = load.numel()
    assert E % world == 0
    e_loc = E // world
    totals, members = [0.0] * world, [[] for _ in range(world)]
    for e in torch.argsort(load, descending=True, stable=True).tolist():
        r = min((r for r in range(world) if len(members[r]) < e_loc), key=lambda r: (totals[r], r))
        members[r].append(e)
        totals[r] += float(load[e])
    return torch.tensor([e for m in members for e in sorted(m)], dtype=torch.int64)


def load_imbalance(load: torch.Tensor, world: int) -> float:
    """max over ranks / mean over ranks of the rows a contiguous sharding of ``load`` gives each rank."""
    per_rank = load.to(torch.float64).view(world, -1).sum(1)
    return float(per_rank.max() * world / per_rank.sum()) if float(per_rank.sum()) > 0 else 1.0
