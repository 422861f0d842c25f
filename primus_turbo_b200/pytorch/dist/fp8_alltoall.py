"""``FP8AllToAll``: an all-to-all(-v) over dim 0 whose payload travels as FP8 bytes
(primus_turbo/pytorch/dist/fp8_alltoall.py:25-194 in the reference).

Each direction (forward, backward) optionally quantises its tensor tensorwise, sends the one-byte payload
and dequantises on arrival; the backward pass sends the gradient over the transposed split sizes.  As in
the reference, every rank quantises with its own scale and the group then agrees on one ``scale_inv`` by a
MIN all-reduce, which the receivers dequantise with: the op is exact when the ranks' amax agree and
otherwise scales a rank's rows by (smallest amax / its own amax).  That behaviour is kept because callers
of the reference see it; it is stated here so that nobody mistakes it for a property of this library's
kernels.  Only ``ScalingGranularity.TENSORWISE`` with ``ScalingStrategy.DYNAMIC`` is supported, formats
E4M3 and HYBRID (E5M2 gradients), as in the reference.
"""

from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from primus_turbo_b200.pytorch.core.low_precision import (
    Float8QuantConfig,
    Format,
    ScalingGranularity,
    ScalingStrategy,
    float8_e4m3,
    float8_e5m2,
)
from primus_turbo_b200.pytorch.ops.quantization import dequantize_fp8, quantize_fp8

__all__ = ["FP8AllToAll"]


def _wire_dtype(config: Float8QuantConfig, forward: bool) -> torch.dtype:
    if config.format == Format.E4M3:
        return float8_e4m3
    if config.format == Format.HYBRID:
        return float8_e4m3 if forward else float8_e5m2
    raise ValueError("FP8AlltoAll only support E4M3 and HYBRID format.")


def _exchange(x: torch.Tensor, out_splits: Optional[List[int]], in_splits: Optional[List[int]], group,
              quant: bool, wire: torch.dtype, config: Float8QuantConfig) -> torch.Tensor:
    """One direction: [quantise ->] all_to_all_single over dim 0 [-> dequantise]."""
    orig_dtype = x.dtype
    x = x.contiguous()
    scale_inv = None
    if quant:
        x, scale_inv = quantize_fp8(x, wire, config.granularity)
        dist.all_reduce(scale_inv, op=dist.ReduceOp.MIN, group=group)
        x = x.view(torch.uint8)  # collectives move plain bytes
    rows = x.shape[0] if out_splits is None else sum(out_splits)
    out = torch.empty((rows, *x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_to_all_single(out, x, output_split_sizes=out_splits, input_split_sizes=in_splits, group=group)
    if out.numel() == 0:
        return torch.empty(out.shape, dtype=orig_dtype, device=out.device)
    if quant:
        out = dequantize_fp8(out.view(wire), orig_dtype, config.granularity, scale_inv=scale_inv)
    return out


class FP8AllToAll(torch.autograd.Function):
    """``FP8AllToAll.apply(group, input_, output_split_sizes, input_split_sizes, fwd_quant, bwd_quant, config)``.

    ``output_split_sizes`` / ``input_split_sizes``: per-rank row counts of dim 0 (``None``: equal split).
    ``fwd_quant`` / ``bwd_quant``: send the forward tensor / the gradient as FP8.
    """

    @staticmethod
    def forward(ctx, group, input_, output_split_sizes, input_split_sizes, fwd_quant, bwd_quant, config):
        assert group is not None, "group should not be None."
        assert config.strategy == ScalingStrategy.DYNAMIC
        assert config.granularity == ScalingGranularity.TENSORWISE
        wire = _wire_dtype(config, True)
        ctx.group, ctx.config, ctx.bwd_quant = group, config, bwd_quant
        ctx.output_split_sizes, ctx.input_split_sizes = output_split_sizes, input_split_sizes
        if dist.get_world_size(group=group) == 1:
            return input_
        return _exchange(input_, output_split_sizes, input_split_sizes, group, fwd_quant, wire, config)

    @staticmethod
    def backward(ctx, grad_output):
        wire = _wire_dtype(ctx.config, False)
        if dist.get_world_size(group=ctx.group) == 1:
            return None, grad_output, None, None, None, None, None
        dgrad = _exchange(grad_output, ctx.input_split_sizes, ctx.output_split_sizes, ctx.group, ctx.bwd_quant, wire,
                          ctx.config)
        return None, dgrad, None, None, None, None, None
