"""MoE token permutation: ``token_permute`` groups the rows of every token by the experts it is routed
to (expert-major, tokens in order inside an expert), ``token_unpermute`` brings expert outputs back to
token order and merges a token's copies, optionally weighted by its routing probabilities.

Same call surface and results as primus_turbo/pytorch/ops/moe/permutation.py:281-436 in the reference
(whose non-fused form is a chain of torch ops -- masked_select, index_select, scatter_add -- and whose
fused form runs Triton kernels over a row-id map); here there is one implementation, on this library's
CUDA kernels: a three-pass stable counting sort of the routing map (``ptb_moe_row_id_map``), the
row gather (``ptb_gather_rows``) and a deterministic per-token merge (``ptb_unpermute_rows``) that
accumulates in fp32 in expert order, i.e. the value a sequential fp32 scatter-add gives.  ``fused`` is
accepted and changes nothing but the third return value's name in the reference's documentation: both
forms return the token id of every permuted row (``sorted_indices``).

The routing map is the source of truth for ``token_unpermute``: pass the same ``routing_map`` that
``token_permute`` saw (the reference requires it only when merging with probabilities).

``drop_and_pad`` (token-drop routing padded to a fixed capacity per expert) has no kernel in the reference
either: its only form is the chain of torch ops of :332-349 / :408-436 there, restated here in the same
terms -- per expert, the first ``capacity`` tokens of a stable descending sort of its 0/1 column.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from primus_turbo_b200 import _lib
from primus_turbo_b200._lib import dtype_code, ptr, require_cuda, stream_of

__all__ = ["token_permute", "token_unpermute"]


def capacity_indices(routing_map: torch.Tensor, capacity: int) -> torch.Tensor:
    """``[num_experts * capacity]`` token ids, expert-major: an expert's routed tokens in token order and, when
    fewer than ``capacity`` are routed to it, its unrouted tokens in token order after them (a stable
    descending sort of the expert's 0/1 column cut at ``capacity``)."""
    by_expert = (routing_map != 0).to(torch.int8).T.contiguous()
    return by_expert.argsort(dim=-1, descending=True, stable=True)[:, :capacity].contiguous().view(-1)


def capacity_probs(probs: torch.Tensor, sorted_indices: torch.Tensor, num_experts: int, capacity: int) -> torch.Tensor:
    """``probs[token of slot, expert of slot]`` for every slot of ``capacity_indices``' layout."""
    num_tokens = probs.size(0)
    expert = torch.arange(num_experts, device=probs.device).unsqueeze(-1)
    flat = (expert * num_tokens + sorted_indices.view(num_experts, capacity)).view(-1)
    return probs.T.contiguous().view(-1).index_select(0, flat)


def _as_bytes(routing_map: torch.Tensor) -> torch.Tensor:
    m = routing_map.contiguous()
    if m.dtype == torch.bool:
        return m.view(torch.uint8)
    return m if m.dtype == torch.uint8 else (m != 0).view(torch.uint8)


def make_row_id_map(routing_map: torch.Tensor, capacity: int, want_sorted: bool = True):
    """-> (row_id_map [T, E] int32, tokens_per_expert [E] int64, sorted_indices [capacity] int64 or None)"""
    require_cuda(routing_map)
    m = _as_bytes(routing_map)
    T, E = m.shape
    dev = m.device
    row_id_map = torch.empty((T, E), dtype=torch.int32, device=dev)
    tpe = torch.empty(E, dtype=torch.int64, device=dev)
    # -1 marks rows past the routed total (only present when the caller asks for more rows than are routed)
    sorted_indices = torch.full((capacity,), -1, dtype=torch.int64, device=dev) if want_sorted else None
    blocks = (T + 255) // 256
    ws = torch.empty(((blocks * E * 4 + 15) // 16) * 16 + (E + 1) * 8, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.call("ptb_moe_row_id_map", ptr(m), T, E, capacity, ptr(row_id_map), ptr(tpe), ptr(sorted_indices), ptr(ws),
                  stream_of(m))
    return row_id_map, tpe, sorted_indices


def _unpermute(rows: torch.Tensor, row_id_map: torch.Tensor, probs: Optional[torch.Tensor], T: int) -> torch.Tensor:
    E = row_id_map.shape[1]
    rows = rows.contiguous()
    out = torch.empty((T, rows.shape[1]), dtype=rows.dtype, device=rows.device)
    with torch.cuda.device(rows.device):
        _lib.call("ptb_unpermute_rows", ptr(rows), dtype_code(rows.dtype), ptr(row_id_map), ptr(probs), T, E, rows.shape[1],
                  ptr(out), stream_of(rows))
    return out


class _Permute(torch.autograd.Function):
    @staticmethod
    def forward(ctx, inp, sorted_indices, row_id_map, probs, expert_of_row):
        from primus_turbo_b200.pytorch.kernels.quantization_impl import gather_rows

        ctx.save_for_backward(row_id_map, sorted_indices, expert_of_row)
        ctx.T, ctx.probs_shape = inp.shape[0], None if probs is None else probs.shape
        out = gather_rows(inp, sorted_indices)
        permuted_probs = None
        if probs is not None:
            ctx.probs_dtype = probs.dtype
            permuted_probs = probs[sorted_indices.clamp(min=0), expert_of_row] * (sorted_indices >= 0).to(probs.dtype)
        return out, permuted_probs

    @staticmethod
    def backward(ctx, g_rows, g_probs):
        row_id_map, sorted_indices, expert_of_row = ctx.saved_tensors
        g_inp = _unpermute(g_rows, row_id_map, None, ctx.T) if ctx.needs_input_grad[0] else None
        gp = None
        if ctx.probs_shape is not None and g_probs is not None and ctx.needs_input_grad[3]:
            gp = torch.zeros(ctx.probs_shape, dtype=g_probs.dtype, device=g_probs.device)
            valid = (sorted_indices >= 0).to(g_probs.dtype)
            gp.index_put_((sorted_indices.clamp(min=0), expert_of_row), g_probs * valid, accumulate=True)
        return g_inp, None, None, gp, None


class _Unpermute(torch.autograd.Function):
    @staticmethod
    def forward(ctx, rows, row_id_map, probs_f32, T):
        ctx.save_for_backward(rows, row_id_map, probs_f32)
        ctx.T = T
        return _unpermute(rows, row_id_map, probs_f32, T)

    @staticmethod
    def backward(ctx, g):
        rows, row_id_map, probs = ctx.saved_tensors
        g = g.contiguous()
        T, E = row_id_map.shape
        # rows past the routed total (a caller-chosen num_out_tokens larger than it) get zero gradient
        g_rows = torch.zeros_like(rows)
        gp = torch.empty((T, E), dtype=torch.float32, device=g.device) if probs is not None else None
        with torch.cuda.device(g.device):
            _lib.call("ptb_unpermute_rows_bwd", ptr(g), dtype_code(g.dtype), ptr(rows), ptr(row_id_map), ptr(probs), T, E,
                      g.shape[1], ptr(g_rows), ptr(gp), stream_of(g))
        return g_rows, None, gp, None


def token_permute(
    inp: torch.Tensor,
    num_out_tokens: int,
    probs: Optional[torch.Tensor] = None,
    routing_map: Optional[torch.Tensor] = None,
    topk_indices: Optional[torch.Tensor] = None,
    drop_and_pad: bool = False,
    fused: bool = False,
    return_tokens_per_expert: bool = False,
) -> Tuple[torch.Tensor, Optional[torch.Tensor], torch.Tensor, Optional[torch.Tensor]]:
    """Group token rows by expert.  ``inp`` [num_tokens, hidden]; ``routing_map`` [num_tokens, num_experts]
    (non-zero: routed); ``probs`` [num_tokens, num_experts] optional; ``num_out_tokens``: rows of the result
    (``-1`` / ``None``: all routed rows, which costs one host read of the total).
    Returns ``(permuted_input, permuted_probs, sorted_indices, tokens_per_expert)``."""
    if topk_indices is not None:
        raise NotImplementedError("not support topk_indices")
    if routing_map is None:
        raise ValueError("must be set topk_indices or routing_map")
    require_cuda(inp, routing_map)
    assert inp.dim() == 2 and inp.size(0) == routing_map.size(0), "Permute not possible"
    T, E = routing_map.shape
    if drop_and_pad and not fused and num_out_tokens is not None:  # (the reference's fused form ignores the flag)
        # every expert takes exactly num_out_tokens / num_experts rows
        capacity = int(num_out_tokens) // E
        assert not routing_map.requires_grad
        sorted_indices = capacity_indices(routing_map, capacity)
        permuted_probs = capacity_probs(probs, sorted_indices, E, capacity) if probs is not None else None
        return inp.index_select(0, sorted_indices), permuted_probs, sorted_indices, (routing_map != 0).sum(0)
    if num_out_tokens is None or num_out_tokens < 0:
        capacity = int(_as_bytes(routing_map).sum().item())
    else:
        capacity = int(num_out_tokens)
    row_id_map, tpe, sorted_indices = make_row_id_map(routing_map, capacity)
    with torch.no_grad():
        # expert of every permuted row (rows at or beyond the routed total repeat the last expert; they are
        # only read when num_out_tokens exceeds the routed total, and then sorted_indices is unset there too)
        bounds = torch.cumsum(tpe, 0)
        expert_of_row = torch.searchsorted(bounds, torch.arange(capacity, device=inp.device), right=True).clamp_(max=E - 1)
    out, permuted_probs = _Permute.apply(inp, sorted_indices, row_id_map, probs, expert_of_row)
    return out, permuted_probs, sorted_indices, (tpe if (return_tokens_per_expert or not fused) else None)


def token_unpermute(
    inp: torch.Tensor,
    sorted_indices: torch.Tensor,
    merging_probs: Optional[torch.Tensor] = None,
    restore_shape: Optional[torch.Size] = None,
    routing_map: Optional[torch.Tensor] = None,
    fused: bool = False,
    drop_and_pad: bool = False,
) -> torch.Tensor:
    """Bring expert-major rows back to token order, summing a token's copies (times ``merging_probs[t, e]``
    when given).  ``restore_shape`` = (num_tokens, hidden)."""
    if drop_and_pad and not fused:
        # the slots of a capacity-padded layout are defined by ``sorted_indices`` alone (a padded slot holds a
        # token that is not routed to the expert), so the rows go back by scatter-add, as in the reference
        assert restore_shape is not None, "restore_shape must be provided"
        require_cuda(inp, sorted_indices)
        input_dtype = inp.dtype
        if merging_probs is not None:
            assert routing_map is not None, "Mask must be provided to permute the probs."
            E = routing_map.size(1)
            slot_probs = capacity_probs(merging_probs, sorted_indices, E, sorted_indices.size(0) // E)
            inp = inp * slot_probs.unsqueeze(-1)
        out = torch.zeros(tuple(restore_shape), dtype=inp.dtype, device=inp.device)
        out.scatter_add_(0, sorted_indices.unsqueeze(1).expand(-1, inp.size(1)), inp)
        return out.to(input_dtype)
    assert routing_map is not None, "routing_map must be provided (it defines where every row goes back to)"
    require_cuda(inp, routing_map)
    T = int(restore_shape[0]) if restore_shape is not None else routing_map.shape[0]
    row_id_map, _, _ = make_row_id_map(routing_map, inp.shape[0], want_sorted=False)
    probs = None
    if merging_probs is not None:
        probs = merging_probs.to(torch.float32).contiguous()
    return _Unpermute.apply(inp, row_id_map, probs, T)
