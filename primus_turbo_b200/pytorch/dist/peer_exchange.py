"""Single-node row exchange over peer-mapped buffers: the expert-parallel dispatch and combine as ONE
copy kernel per direction that writes every row straight to its final, expert-major position in the
destination GPU's memory (plain stores over NVLink / NVSwitch), instead of an all-to-all into a
staging buffer followed by a permutation pass on the receiver.

The reference wraps ``grouped_gemm_fp8`` between a token dispatch and combine backed by its DeepEP
port (primus_turbo/pytorch/ops/moe/moe_dispatch_combine.py:20-101); this module is the same pair of
steps for ranks that share one machine.

How it works
* Every rank allocates its receive regions with torch and publishes them to the other ranks of the
  node as CUDA IPC handles (``torch.multiprocessing.reductions.reduce_tensor`` -> one object
  all-gather over a CPU group); each rank opens the others' handles once and keeps raw pointers.
* The routing counts of all ranks ([world, E]) give, on the host and for both directions, one row
  segment per (rank, expert): first source row, first destination row, row count, destination rank
  (``segment_tables``).  ``ptb_copy_segments`` (csrc/ptb_exchange.cu) performs all copies of a rank
  in one launch.
* The copy kernel waits on nothing.  Ranks are ordered by a one-element NCCL all-reduce after each
  exchange: a rank reads a region only after that collective, and a region is overwritten at the
  earliest one collective after its reader consumed it (each region is written once per step).
* No kernel here loads from peer memory through TMA, and nothing uses cluster multicast.

The CPU tests drive the same plan and bookkeeping with shared-memory tensors and a copy loop of their
own (``copy_fn``); the product path has no CPU implementation.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

__all__ = ["SegmentTables", "segment_tables", "PeerExchange", "peer_dispatch", "peer_combine"]


@dataclass
class SegmentTables:
    """Row segments of one rank for both directions, int64 ``[nseg, 4]`` each: first source row, first
    destination row, rows, destination rank."""

    dispatch: torch.Tensor  # my rows (sorted by expert) -> the owners' expert-major buffers
    combine: torch.Tensor  # my expert-major rows -> the source ranks' original positions
    group_lens: torch.Tensor  # [E_local] rows per local expert after the dispatch
    rows_in: int  # rows this rank holds before the dispatch (= after the combine)
    rows_out: int  # rows this rank holds after the dispatch


def segment_tables(counts_matrix: torch.Tensor, rank: int) -> SegmentTables:
    """Index arithmetic of both exchanges from the host copy of the ``[world, E]`` count matrix
    (``counts_matrix[s, e]`` = rows rank ``s`` routes to expert ``e``; experts sharded contiguously,
    expert ``e`` on rank ``e // (E / world)``; every rank's rows are sorted by expert)."""
    import numpy as np

    # numpy, not torch: a dozen tiny array operations per step, and torch's dispatch costs ten times numpy's
    C = counts_matrix.to(torch.int64).numpy()
    world, E = C.shape
    assert E % world == 0
    e_loc = E // world
    total = C.sum(0)  # rows per expert over all sources
    blk = total.reshape(world, e_loc)
    start_in_owner = (blk.cumsum(1) - blk).reshape(E)  # first row of expert e in its owner's buffer
    before_src = C.cumsum(0) - C  # [s, e]: rows of expert e that come from sources below s
    own_off = C.cumsum(1) - C  # [s, e]: first row of expert e in rank s's own (sorted) rows
    experts = np.arange(E)
    dispatch = np.stack([own_off[rank], start_in_owner + before_src[rank], C[rank], experts // e_loc], axis=1)
    lo, hi = rank * e_loc, (rank + 1) * e_loc
    # (local expert, source) pairs in expert-major order
    src_row = (start_in_owner[lo:hi, None] + before_src[:, lo:hi].T).reshape(-1)
    dst_row = own_off[:, lo:hi].T.reshape(-1)
    rows = C[:, lo:hi].T.reshape(-1)
    dst_rank = np.tile(np.arange(world), e_loc)
    combine = np.stack([src_row, dst_row, rows, dst_rank], axis=1)
    mine_total = np.ascontiguousarray(total[lo:hi])
    return SegmentTables(torch.from_numpy(np.ascontiguousarray(dispatch)), torch.from_numpy(np.ascontiguousarray(combine)),
                         torch.from_numpy(mine_total), int(C[rank].sum()), int(mine_total.sum()))


def _device_copy(src: torch.Tensor, dst_ptrs: List[int], segs: torch.Tensor, row_bytes: int, num_ctas: int) -> None:
    from primus_turbo_b200 import _lib

    arr = (ctypes.c_void_p * len(dst_ptrs))(*dst_ptrs)
    with torch.cuda.device(src.device):
        _lib.call("ptb_copy_segments", src.data_ptr(), arr, len(dst_ptrs), segs.data_ptr(), segs.shape[0], row_bytes,
                  num_ctas, torch.cuda.current_stream(src.device).cuda_stream)


def _device_copy_signal(src: torch.Tensor, arr, segs: torch.Tensor, row_bytes: int, num_ctas: int, slots, done_counter: int,
                        seq: int) -> None:
    """``arr`` / ``slots``: ctypes arrays of the destinations' region bases and of this rank's flag slot in each."""
    from primus_turbo_b200 import _lib

    n = len(arr)
    nseg = segs.shape[0] if src.shape[0] else 0
    with torch.cuda.device(src.device):
        _lib.call("ptb_copy_segments_signal", src.data_ptr() if nseg else None, arr, n, segs.data_ptr() if nseg else None,
                  nseg, row_bytes, num_ctas, slots, done_counter, seq, torch.cuda.current_stream(src.device).cuda_stream)


def _export_cuda_ipc(t: torch.Tensor):
    from torch.multiprocessing.reductions import reduce_tensor

    return reduce_tensor(t)


def _import_cuda_ipc(handle):
    """Open another rank's region for kernels of THIS rank's device.

    ``cudaIpcOpenMemHandle`` maps the memory into the address space of the device that is current when
    it is called.  torch's rebuild function makes the OWNER's device index current (its use case is a
    consumer that keeps working on the producer's device); a mapping made that way is not addressable
    from this rank's device -- the first store through it is an illegal address, peer access enabled or
    not.  So the handle is opened with this rank's device in the owner's place: the driver then maps
    the peer GPU's memory for this device and enables peer access as needed (the lazy-peer-access
    flag torch passes), which is the pattern NCCL and every IPC-based collective use.  The returned
    tensor claims this rank's device; it is only ever used as a raw destination pointer."""
    fn, args = handle
    args = list(args)
    assert fn.__name__ == "rebuild_cuda_tensor" and len(args) >= 8, "unexpected CUDA IPC handle format"
    args[6] = torch.cuda.current_device()  # storage_device: the device that is current during the open
    return fn(*args)


class PeerExchange:
    """Receive regions of every rank of one node, mapped into this process, plus the ordering collective.

    ``capacity_rows``: most rows a rank may receive in one dispatch (a plan that needs more raises).
    Regions are created on first use, keyed by (direction, row width in bytes, forward / backward pass); creation is collective
    (every rank must reach it in the same order, which the symmetric call sequence of a training step
    guarantees).  ``host_group`` carries the handle exchange (a CPU group); ``group`` the ordering
    collective.  ``copy_fn`` / ``alloc_fn`` replace the device pieces in CPU tests.

    Ordering after an exchange (``ordering``): ``"flags"`` (default on CUDA with the built-in copy) -- the
    copy kernel itself stores the exchange's sequence number into this rank's slot of every destination's
    flag array once its rows have landed, and ``order()`` enqueues a one-warp kernel that waits (with a
    time limit) for all sources' slots; ``"collective"`` -- a one-element all-reduce on ``group``.
    Both are a barrier among the ranks in stream order; neither blocks the host.
    """

    MAX_KEYS = 32  # regions (direction x row width x pass) one exchange object can hold

    def __init__(self, group: Optional[dist.ProcessGroup], host_group: Optional[dist.ProcessGroup], device,
                 capacity_rows: int, local_rows: int, copy_fn: Optional[Callable] = None,
                 alloc_fn: Optional[Callable] = None, num_ctas: int = 0, export_fn: Optional[Callable] = None,
                 import_fn: Optional[Callable] = None, ordering: Optional[str] = None):
        self.group, self.host_group = group, host_group
        self.device = torch.device(device)
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.capacity_rows, self.local_rows = int(capacity_rows), int(local_rows)
        self.num_ctas = num_ctas
        self._copy = copy_fn or _device_copy
        self._alloc = alloc_fn or (lambda nbytes: torch.empty(nbytes, dtype=torch.uint8, device=self.device))
        # how a region is published to / opened by the other ranks: for CUDA memory, torch's IPC handle
        # (plain picklable values: device index, cudaIpcMemHandle bytes, sizes)
        self._export = export_fn or _export_cuda_ipc
        self._import = import_fn or _import_cuda_ipc
        self._regions: Dict[Tuple[str, int, str], Tuple[torch.Tensor, List, List[int]]] = {}
        self._flag = torch.zeros(1, dtype=torch.int32, device=self.device)
        if self.device.type == "cuda" and import_fn is None:
            self._check_peer_paths()
        if ordering is None:
            ordering = "flags" if (self.device.type == "cuda" and copy_fn is None and import_fn is None) else "collective"
        assert ordering in ("flags", "collective")
        self.ordering = ordering
        self._key_index: Dict[Tuple[str, int, str], int] = {}
        self._seq: Dict[int, int] = {}
        self._last: Optional[Tuple[int, int]] = None  # (key index, sequence number) of the latest push
        self._signal_args: Dict[int, Tuple] = {}
        if ordering == "flags":
            # [MAX_KEYS, world] arrival slots (row k: one slot per source rank) and one CTA counter per key,
            # zeroed; the slots are published to the other ranks like a region
            self._flags = torch.zeros(self.MAX_KEYS * self.world + self.MAX_KEYS, dtype=torch.int32, device=self.device)
            torch.cuda.synchronize(self.device)  # the zeros are in memory before any peer may write a slot
            handles: List = [None] * self.world
            dist.all_gather_object(handles, self._export(self._flags), group=self.host_group)
            self._flag_views = [self._flags if r == self.rank else self._import(h) for r, h in enumerate(handles)]
            self._flag_ptrs = [t.data_ptr() for t in self._flag_views]

    def _check_peer_paths(self) -> None:
        """Before any region exists: every rank tells the others which device it runs on and enables peer
        access to each of them; a missing peer path raises here, on the host, on every rank."""
        from primus_turbo_b200 import _lib

        mine = self.device.index if self.device.index is not None else torch.cuda.current_device()
        devices: List = [None] * self.world
        dist.all_gather_object(devices, int(mine), group=self.host_group)
        problem = None
        with torch.cuda.device(mine):
            for d in sorted(set(devices)):
                if d != mine:
                    try:
                        _lib.call("ptb_enable_peer_access", d)
                    except _lib.PtbError as exc:
                        problem = str(exc)
        verdicts: List = [None] * self.world
        dist.all_gather_object(verdicts, problem, group=self.host_group)
        bad = [f"rank {r}: {v}" for r, v in enumerate(verdicts) if v]
        if bad:
            raise RuntimeError("peer-memory exchange unavailable: " + "; ".join(bad))

    # ---- regions ---------------------------------------------------------------------------------
    def _region(self, direction: str, row_bytes: int, phase: str = "fwd"):
        key = (direction, row_bytes, phase)
        if key not in self._regions:
            rows = self.capacity_rows if direction == "dispatch" else self.local_rows
            local = self._alloc(max(rows, 1) * row_bytes)
            handles: List = [None] * self.world
            dist.all_gather_object(handles, self._export(local), group=self.host_group)
            views, ptrs = [], []
            for r, h in enumerate(handles):
                t = local if r == self.rank else self._import(h)
                views.append(t)  # keeps the mapping alive
                ptrs.append(t.data_ptr())
            self._regions[key] = (local, views, ptrs)
            self._key_index[key] = len(self._key_index)
            if len(self._key_index) > self.MAX_KEYS:
                raise RuntimeError(f"more than {self.MAX_KEYS} distinct exchange regions")
        return self._regions[key]

    # ---- the two exchanges ------------------------------------------------------------------------
    def order(self) -> None:
        """Stream-ordered rendezvous of all ranks after the latest ``push`` (the host is not blocked)."""
        if self.ordering == "flags":
            from primus_turbo_b200 import _lib

            k, seq = self._last
            with torch.cuda.device(self.device):
                _lib.call("ptb_wait_flags", self._flag_ptrs[self.rank] + 4 * k * self.world, self.world, seq & 0xFFFFFFFF,
                          torch.cuda.current_stream(self.device).cuda_stream)
            return
        if self.device.type == "cuda":
            from primus_turbo_b200 import _lib

            with _lib.timed_region("ep_order_all_reduce"):
                dist.all_reduce(self._flag, group=self.group)
        else:
            dist.all_reduce(self._flag, group=self.group)

    def close(self) -> None:
        """Collective teardown (call before the process group is destroyed): every rank first drops its
        mappings of the other ranks' regions, all ranks meet, and only then does a rank release its own
        regions -- so no rank ever frees memory that a peer still has mapped, and no rank unmaps memory
        whose owner has already gone."""
        import gc

        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        for key, (local, views, ptrs) in list(self._regions.items()):
            self._regions[key] = (local, [], [])
        if self.ordering == "flags":
            self._flag_views, self._flag_ptrs = [self._flags], []
            self._signal_args.clear()
        gc.collect()
        if self.device.type == "cuda":
            torch.cuda.ipc_collect()
        dist.barrier(group=self.host_group)
        self._regions.clear()
        gc.collect()
        dist.barrier(group=self.host_group)

    def push(self, src: torch.Tensor, segs: torch.Tensor, direction: str, rows_received: int,
             phase: str = "fwd") -> torch.Tensor:
        """Copy ``src``'s row segments into every rank's region for ``direction`` and return this rank's
        region viewed as ``[rows_received, width]`` (valid once ``order()`` has been enqueued, until
        the next ``push`` of the same direction, width and phase).  Forward and backward passes use
        separate regions (``phase``), so rows dispatched in a forward pass stay intact through the
        matching backward pass -- a local function may keep them for its gradient -- and are replaced
        by the next forward pass: one step in flight at a time."""
        assert src.dim() == 2 and src.is_contiguous()
        row_bytes = src.shape[1] * src.element_size()
        limit = self.capacity_rows if direction == "dispatch" else self.local_rows
        if rows_received > limit:
            raise RuntimeError(f"{direction}: {rows_received} rows arrive at rank {self.rank} but the region holds {limit}")
        local, _, ptrs = self._region(direction, row_bytes, phase)
        if self.ordering == "flags":
            # the copy runs even with nothing to send: its signal is this rank's part of the rendezvous
            k = self._key_index[(direction, row_bytes, phase)]
            seq = self._seq.get(k, 0) + 1
            self._seq[k] = seq
            self._last = (k, seq)
            cached = self._signal_args.get(k)
            if cached is None:  # the pointer arrays of a region never change: build them once
                n = len(ptrs)
                cached = ((ctypes.c_void_p * n)(*ptrs),
                          (ctypes.c_void_p * n)(*[p + 4 * (k * self.world + self.rank) for p in self._flag_ptrs]),
                          self._flag_ptrs[self.rank] + 4 * (self.MAX_KEYS * self.world + k))
                self._signal_args[k] = cached
            _device_copy_signal(src, cached[0], segs, row_bytes, self.num_ctas, cached[1], cached[2], seq & 0xFFFFFFFF)
        elif segs.shape[0] and src.shape[0]:
            self._copy(src, ptrs, segs, row_bytes, self.num_ctas)
        # `.data`: a tensor over the same bytes with its own version counter -- the region is rewritten by
        # later exchanges (by kernels of other ranks), which autograd must not mistake for an in-place edit
        return local.data[: rows_received * row_bytes].view(src.dtype).view(rows_received, src.shape[1])


def _copy_out(region_view: torch.Tensor) -> torch.Tensor:
    if region_view.is_cuda:
        from primus_turbo_b200 import _lib

        with _lib.timed_region("ep_copy_out_of_region"):
            return region_view.clone()
    return region_view.clone()


class _PeerMove(torch.autograd.Function):
    """One exchange; its gradient is the opposite exchange over the same segments.  Results that leave
    this module for the caller (the combined output, the gradient of the dispatched input) are copied
    out of the region; results consumed at once by the local grouped GEMM are views of it."""

    @staticmethod
    def forward(ctx, x, ex: PeerExchange, fwd_segs, bwd_segs, direction, rows_fwd, rows_bwd):
        ctx.ex, ctx.bwd_segs, ctx.rows_bwd = ex, bwd_segs, rows_bwd
        ctx.bwd_direction = "combine" if direction == "dispatch" else "dispatch"
        out = ex.push(x.contiguous(), fwd_segs, direction, rows_fwd)
        ex.order()
        return _copy_out(out) if direction == "combine" else out

    @staticmethod
    def backward(ctx, g):
        ex = ctx.ex
        out = ex.push(g.contiguous(), ctx.bwd_segs, ctx.bwd_direction, ctx.rows_bwd, phase="bwd")
        ex.order()
        return (_copy_out(out) if ctx.bwd_direction == "combine" else out), None, None, None, None, None, None


def peer_dispatch(x_local: torch.Tensor, ex: PeerExchange, tables: SegmentTables, seg_dev: Tuple[torch.Tensor, torch.Tensor]):
    """Rows sorted by global expert -> this rank's experts' rows in expert-major order (a view of the
    receive region: consume it before the next dispatch of the same width)."""
    return _PeerMove.apply(x_local, ex, seg_dev[0], seg_dev[1], "dispatch", tables.rows_out, tables.rows_in)


def peer_combine(y: torch.Tensor, ex: PeerExchange, tables: SegmentTables, seg_dev: Tuple[torch.Tensor, torch.Tensor]):
    """Expert-major result rows -> back to the rank and position their input rows came from."""
    return _PeerMove.apply(y, ex, seg_dev[1], seg_dev[0], "combine", tables.rows_in, tables.rows_out)
