"""``grouped_gemm_fp8``: MoE grouped GEMM with FP8 quantisation and autograd
(primus_turbo/pytorch/ops/grouped_gemm_fp8.py:75-211 blockwise, :214-393 rowwise, :396-568
tensorwise, :808-904 public entry).

``a`` is the packed activation ``[sum(group_lens), K]``; ``b`` is ``[G, N, K]`` (``trans_b``) or
``[G, K, N]``.  Forward and dgrad run the row-segmented grouped kernel; wgrad runs the variable-K
kernel whose contraction axis is the group's row range.  Nothing here synchronises with the host:
group boundaries are read on the device.
"""

from __future__ import annotations

from typing import Optional, Union

import torch

from primus_turbo_b200.pytorch.core.low_precision import (
    Float8QuantConfig,
    Format,
    ScalingGranularity,
    ScalingRecipe,
    float8_e4m3,
    float8_e5m2,
)
from primus_turbo_b200.pytorch.core.quantized_tensor import (
    QuantizedTensor,
    QuantizedTensorPair,
    check_quantized_tensor,
)
from primus_turbo_b200.pytorch.kernels.custom_ops import (
    grouped_gemm_fp8_impl,
    grouped_gemm_fp8_variable_k_impl,
)
from primus_turbo_b200.pytorch.kernels.custom_ops import quant_fp8_blockwise_for_weight as quant_fp8_blockwise_for_weight_impl
from primus_turbo_b200.pytorch.kernels.custom_ops import (
    quant_fp8_blockwise_segment_m_row_col as quant_fp8_blockwise_segment_m_row_col_impl,
)
from primus_turbo_b200.pytorch.kernels.gemm_impl import (
    group_offs_from_lens,
    grouped_gemm_mxfp8_impl,
    grouped_gemm_mxfp8_variable_k_impl,
)
from primus_turbo_b200.pytorch.kernels.quantization_impl import (
    grouped_quantize_mxfp8_impl,
    packed_row_index,
    quantize_mxfp8_impl,
)

__all__ = ["grouped_gemm_fp8"]

_WEIGHT_RECIPE = ScalingRecipe(use_2d_block=True)  # how BLOCKWISE weights are quantised (128x128 blocks)


def _get_fp8_dtype(format: Format, is_fwd_stage: bool):
    if format == Format.E4M3:
        return float8_e4m3
    if format == Format.E5M2:
        return float8_e5m2
    if format == Format.HYBRID:
        return float8_e4m3 if is_fwd_stage else float8_e5m2
    raise ValueError(f"Unsupported FP8 format: {format}")


def _contig(t: torch.Tensor) -> torch.Tensor:
    return t if t.is_contiguous() else t.contiguous()


class FP8GroupedGemmBlockFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, group_lens, group_offs, trans_b, out_dtype, config, num_cu):
        assert config.granularity == ScalingGranularity.BLOCKWISE
        assert config.block_size in [128], "Only block_size 128 is supported currently."
        assert a.ndim == 2, "Input tensor must be 2-dimensional."
        assert b.ndim == 3, "Weight tensor must be 3-dimensional."
        assert group_lens.size(0) == b.size(0), "group_lens size must match b size(0)."
        assert out_dtype in [torch.float16, torch.bfloat16]
        dt = _get_fp8_dtype(config.format, True)
        assert not isinstance(a, QuantizedTensor), (
            "BLOCKWISE activations are quantised inside grouped_gemm_fp8 (their column copy depends on the groups)"
        )
        # one read of a -> 1x128 row copy (forward) + segment-padded 128x1 column copy (wgrad)
        a_row, a_col, a_s_row, a_s_col, _, _ = quant_fp8_blockwise_segment_m_row_col_impl(
            _contig(a), dt, config.block_size, group_lens, group_offs
        )
        if isinstance(b, QuantizedTensor):
            # A weight quantised ahead of time (create_quantized_weight): 128x128 blocks, used as stored by
            # forward and dgrad alike, so the 3-bytes-per-element re-quantisation of every forward goes away.
            # The reference accepts pre-quantised weights for its tensorwise / rowwise grouped paths only
            # (ops/grouped_gemm_fp8.py:886-889 there); this is the same hook extended to BLOCKWISE.
            assert not b._is_grouped_tensor, "B QuantizedTensor input must not be a grouped tensor"
            check_quantized_tensor(b, config, scaling_recipe=_WEIGHT_RECIPE)
            assert b.real_dtype == dt, f"pre-quantised weight is {b.real_dtype}, the config asks for {dt}"
            b8, b_s = b.qdata, b.scale_inv
        else:
            b8, b_s = quant_fp8_blockwise_for_weight_impl(b, dt, config.block_size)
        out = grouped_gemm_fp8_impl(
            a_row, b8, a_s_row, b_s, group_lens, group_offs, trans_a=False, trans_b=trans_b, out_dtype=out_dtype,
            granularity=config.granularity.value, num_cu=num_cu,
        )
        ctx.save_for_backward(a_col, a_s_col, b8, b_s, group_lens, group_offs)
        ctx.trans_b, ctx.config, ctx.out_dtype, ctx.num_cu = trans_b, config, out_dtype, num_cu
        return out

    @staticmethod
    def backward(ctx, grad_out):
        grad_out = _contig(grad_out)
        a_col, a_s_col, b8, b_s, group_lens, group_offs = ctx.saved_tensors
        cfg = ctx.config
        g_row, g_col, g_s_row, g_s_col, vk_lens, vk_offs = quant_fp8_blockwise_segment_m_row_col_impl(
            grad_out, _get_fp8_dtype(cfg.format, False), cfg.block_size, group_lens, group_offs
        )
        grad_a = grouped_gemm_fp8_impl(
            g_row, b8, g_s_row, b_s, group_lens, group_offs, trans_a=False, trans_b=not ctx.trans_b,
            out_dtype=ctx.out_dtype, granularity=cfg.granularity.value, num_cu=ctx.num_cu,
        )
        grad_b = grouped_gemm_fp8_variable_k_impl(
            a_col, g_col, a_s_col, g_s_col, vk_lens, vk_offs, trans_a=True, trans_b=False, trans_c=ctx.trans_b,
            out_dtype=ctx.out_dtype, granularity=cfg.granularity.value, num_cu=ctx.num_cu,
        )
        return grad_a, grad_b, None, None, None, None, None, None


class FP8GroupedGemmRowFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, a_t, b_t, group_lens, group_offs, trans_b, out_dtype, config, num_cu):
        assert config.granularity == ScalingGranularity.ROWWISE
        g = config.granularity
        dt = _get_fp8_dtype(config.format, True)
        if isinstance(a, QuantizedTensor):
            assert a._is_grouped_tensor, "A QuantizedTensor input must be a grouped tensor"
            check_quantized_tensor(a, config, axis=-1)
            qa, group_offs = a, a.group_offs
        else:
            qa = QuantizedTensor.quantize(a, dt, g, axis=-1, block_size=config.block_size, group_lens=group_lens)
        b_row_axis, b_col_axis = (-1, -2) if trans_b else (-2, -1)
        if isinstance(b, QuantizedTensor):
            assert not b._is_grouped_tensor, "B QuantizedTensor input must not be a grouped tensor"
            check_quantized_tensor(b, config, axis=b_row_axis)
            qb = b
        else:
            qb = QuantizedTensor.quantize(b, dt, g, axis=b_row_axis, block_size=config.block_size)
        out = grouped_gemm_fp8_impl(
            qa.qdata, qb.qdata, qa.scale_inv, qb.scale_inv, group_lens, group_offs, trans_a=False, trans_b=trans_b,
            out_dtype=out_dtype, granularity=g.value, num_cu=num_cu,
        )
        # backward companions: re-quantise the dequantised forward operands along the other axis
        qa_t = a_t if a_t is not None else QuantizedTensor.quantize(
            qa.dequantize(), qa.real_dtype, g, axis=-2, block_size=config.block_size, group_lens=group_lens
        )
        qb_t = b_t if b_t is not None else QuantizedTensor.quantize(
            qb.dequantize(), qb.real_dtype, g, axis=b_col_axis, block_size=config.block_size
        )
        ctx.save_for_backward(qa_t.qdata, qb_t.qdata, qa_t.scale_inv, qb_t.scale_inv, group_lens, group_offs)
        ctx.trans_b, ctx.config, ctx.out_dtype, ctx.num_cu = trans_b, config, out_dtype, num_cu
        return out

    @staticmethod
    def backward(ctx, grad_out):
        grad_out = _contig(grad_out)
        a_col, b_col, a_s_col, b_s_col, group_lens, group_offs = ctx.saved_tensors
        cfg = ctx.config
        g = cfg.granularity
        gdt = _get_fp8_dtype(cfg.format, False)
        qg = QuantizedTensor.quantize(grad_out, gdt, g, axis=-1, block_size=cfg.block_size, group_lens=group_lens)
        grad_a = grouped_gemm_fp8_impl(
            qg.qdata, b_col, qg.scale_inv, b_s_col, group_lens, group_offs, trans_a=False, trans_b=not ctx.trans_b,
            out_dtype=ctx.out_dtype, granularity=g.value, num_cu=ctx.num_cu,
        )
        qg_t = QuantizedTensor.quantize(grad_out, gdt, g, axis=-2, block_size=cfg.block_size, group_lens=group_lens)
        grad_b = grouped_gemm_fp8_variable_k_impl(
            a_col, qg_t.qdata, a_s_col, qg_t.scale_inv, group_lens, group_offs, trans_a=True, trans_b=False,
            trans_c=ctx.trans_b, out_dtype=ctx.out_dtype, granularity=g.value, num_cu=ctx.num_cu,
        )
        return grad_a, grad_b, None, None, None, None, None, None, None, None


class FP8GroupedGemmTensorFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, a_t, b_t, group_lens, group_offs, trans_b, out_dtype, config, num_cu):
        assert config.granularity == ScalingGranularity.TENSORWISE
        g = config.granularity
        dt = _get_fp8_dtype(config.format, True)
        if isinstance(a, QuantizedTensor):
            assert a._is_grouped_tensor, "A QuantizedTensor input must be a grouped tensor"
            check_quantized_tensor(a, config)
            qa, group_offs = a, a.group_offs
        else:
            qa = QuantizedTensor.quantize(a, dt, g, axis=-1, block_size=config.block_size, group_lens=group_lens)
        if isinstance(b, QuantizedTensor):
            assert not b._is_grouped_tensor, "B QuantizedTensor input must not be a grouped tensor"
            check_quantized_tensor(b, config)
            qb = b
        else:
            qb = QuantizedTensor.quantize(b, dt, g, axis=-1, block_size=config.block_size)
        out = grouped_gemm_fp8_impl(
            qa.qdata, qb.qdata, qa.scale_inv, qb.scale_inv, group_lens, group_offs, trans_a=False, trans_b=trans_b,
            out_dtype=out_dtype, granularity=g.value, num_cu=num_cu,
        )
        # the tensor cores read b transposed in place, so backward reuses the forward payload
        ctx.save_for_backward(qa.qdata, qb.qdata, qa.scale_inv, qb.scale_inv, group_lens, group_offs)
        ctx.trans_b, ctx.config, ctx.out_dtype, ctx.num_cu = trans_b, config, out_dtype, num_cu
        return out

    @staticmethod
    def backward(ctx, grad_out):
        grad_out = _contig(grad_out)
        a8, b8, a_s, b_s, group_lens, group_offs = ctx.saved_tensors
        cfg = ctx.config
        g = cfg.granularity
        qg = QuantizedTensor.quantize(
            grad_out, _get_fp8_dtype(cfg.format, False), g, axis=-1, block_size=cfg.block_size, group_lens=group_lens
        )
        grad_a = grouped_gemm_fp8_impl(
            qg.qdata, b8, qg.scale_inv, b_s, group_lens, group_offs, trans_a=False, trans_b=not ctx.trans_b,
            out_dtype=ctx.out_dtype, granularity=g.value, num_cu=ctx.num_cu,
        )
        grad_b = grouped_gemm_fp8_variable_k_impl(
            a8, qg.qdata, a_s, qg.scale_inv, group_lens, group_offs, trans_a=True, trans_b=False,
            trans_c=ctx.trans_b, out_dtype=ctx.out_dtype, granularity=g.value, num_cu=ctx.num_cu,
        )
        return grad_a, grad_b, None, None, None, None, None, None, None, None


@torch._dynamo.disable(recursive=True, reason="builds QuantizedTensor wrappers inside autograd.Function.forward")
class FP8GroupedGemmMXFunc(torch.autograd.Function):
    """MX_BLOCKWISE grouped GEMM (primus_turbo/pytorch/ops/grouped_gemm_fp8.py:571-795): a and grad_out are
    quantised per group in both directions in one pass, b per expert in both directions (32x32 tiles);
    forward and dgrad read the row copies, wgrad the transposed column copies over each group's 128-padded
    row range.  The reference's forward reads a row copy padded to 32 rows per group and writes a packed
    output; 1x32 blocks along K do not depend on the padding, so this build keeps the row copy unpadded
    and the numbers are the same."""

    @staticmethod
    def forward(ctx, a, b, a_t, b_t, group_lens, group_offs, trans_b, out_dtype, config, num_cu):
        assert config.granularity == ScalingGranularity.MX_BLOCKWISE
        assert a.ndim == 2 and b.ndim == 3
        assert trans_b, "MXFP8 grouped GEMM only supports trans_b=True (NT layout)."
        dt = _get_fp8_dtype(config.format, True)
        a_offs, pack = group_offs, None
        if isinstance(a, QuantizedTensor):
            # A grouped activation quantised ahead of time carries the reference's layout: the row copy with every
            # group padded to 32 rows.  The GEMM runs over that layout (the padding rows cost a little and their
            # results are dropped) and the rows that exist are gathered into the packed output, which is what the
            # reference does with its padded / packed offset pair (:693-720).  The column copy comes from ``a_t``
            # or from re-quantising the dequantised row copy along the other axis (:634-648).
            recipe = ScalingRecipe()
            assert a._is_grouped_tensor, "A QuantizedTensor input must be a grouped tensor"
            check_quantized_tensor(a, config, axis=-1, scaling_recipe=recipe)
            if a_t is None:
                a_t = QuantizedTensor.quantize(
                    a.dequantize(), a.real_dtype, config.granularity, axis=-2, block_size=config.block_size,
                    scaling_recipe=recipe, group_lens=group_lens,
                )
            else:
                assert isinstance(a_t, QuantizedTensor) and a_t._is_grouped_tensor
                check_quantized_tensor(a_t, config, axis=-2, scaling_recipe=recipe)
            a_row, a_row_s, a_col, a_col_s = a.qdata, a.scale_inv, a_t.qdata, a_t.scale_inv
            a_offs = a.group_offs
            pack = packed_row_index(group_offs, a_offs, a.shape[0])
        else:
            a_row, a_row_s, a_col, a_col_s, _, _, _, _ = grouped_quantize_mxfp8_impl(
                _contig(a), dt, config.block_size, group_lens, group_offs, False, False, row_align=1
            )
        if isinstance(b, QuantizedTensor):
            # a weight quantised ahead of time (32x32 tiles, axis -1); its column copy comes from ``b_t`` or from
            # re-quantising the dequantised row copy along the other axis, as in the reference (:668-692)
            recipe = ScalingRecipe(use_2d_block=True)
            assert not b._is_grouped_tensor, "B QuantizedTensor input must not be a grouped tensor"
            check_quantized_tensor(b, config, axis=-1, scaling_recipe=recipe)
            if b_t is None:
                b_t = QuantizedTensor.quantize(
                    b.dequantize(), b.real_dtype, config.granularity, axis=-2, block_size=config.block_size,
                    scaling_recipe=recipe,
                )
            else:
                assert isinstance(b_t, QuantizedTensor)
                check_quantized_tensor(b_t, config, axis=-2, scaling_recipe=recipe)
            b_row, b_row_s, b_col, b_col_s = b.qdata, b.scale_inv, b_t.qdata, b_t.scale_inv
        else:
            b_row, b_row_s, b_col, b_col_s = quantize_mxfp8_impl(_contig(b), dt, None, config.block_size, True, True, True)
        sms = num_cu or 0
        out = grouped_gemm_mxfp8_impl(a_row, a_row_s, b_row, b_row_s, a_offs, out_dtype, sms)
        if pack is not None:
            out = out.index_select(0, pack)
        ctx.save_for_backward(a_col, a_col_s, b_col, b_col_s, group_lens, group_offs)
        ctx.config, ctx.out_dtype, ctx.sms = config, out_dtype, sms
        return out

    @staticmethod
    def backward(ctx, grad_out):
        a_col, a_col_s, b_col, b_col_s, group_lens, group_offs = ctx.saved_tensors
        cfg = ctx.config
        g_row, g_row_s, g_col, g_col_s, _, _, _, col_offs = grouped_quantize_mxfp8_impl(
            _contig(grad_out), _get_fp8_dtype(cfg.format, False), cfg.block_size, group_lens, group_offs, False, False,
            row_align=1,
        )
        # dgrad: grad_a = grad_out . b   = [M, N_pad] x (b_col [G, K, N_pad])^T
        grad_a = grouped_gemm_mxfp8_impl(g_row, g_row_s, b_col, b_col_s, group_offs, ctx.out_dtype, ctx.sms)
        # wgrad: grad_b[g] = grad_out_g^T . a_g = g_col [N, rows] x (a_col [K, rows])^T over the group's padded rows
        grad_b = grouped_gemm_mxfp8_variable_k_impl(g_col, g_col_s, a_col, a_col_s, col_offs, ctx.out_dtype, ctx.sms)
        return grad_a, grad_b, None, None, None, None, None, None, None, None


def grouped_gemm_fp8(
    a: Union[torch.Tensor, QuantizedTensor, QuantizedTensorPair],
    b: Union[torch.Tensor, QuantizedTensor, QuantizedTensorPair],
    group_lens: torch.Tensor,
    group_offs: Optional[torch.Tensor] = None,
    trans_b: bool = True,
    out_dtype: Optional[torch.dtype] = None,
    config: Optional[Float8QuantConfig] = None,
    num_cu: Optional[int] = None,
) -> torch.Tensor:
    """Grouped GEMM ``out[rows of group g] = a[rows of group g] @ op(b[g])`` in FP8.

    group_lens: CUDA int64 ``[G]``; group_offs (optional): its exclusive prefix sum ``[G+1]``.
    ``num_cu`` caps the number of SMs the persistent kernel occupies.  Rows of the output at or
    beyond ``sum(group_lens)`` are zero.
    """
    if config is None:
        config = Float8QuantConfig()
    if group_offs is None:
        group_offs = group_offs_from_lens(group_lens)
    a_data, a_data_t = (a.data, a.data_t) if isinstance(a, QuantizedTensorPair) else (a, None)
    b_data, b_data_t = (b.data, b.data_t) if isinstance(b, QuantizedTensorPair) else (b, None)
    if out_dtype is None:
        out_dtype = torch.promote_types(a_data.dtype, b_data.dtype)
    if config.granularity == ScalingGranularity.TENSORWISE:
        return FP8GroupedGemmTensorFunc.apply(
            a_data, b_data, a_data_t, b_data_t, group_lens, group_offs, trans_b, out_dtype, config, num_cu
        )
    if config.granularity == ScalingGranularity.ROWWISE:
        return FP8GroupedGemmRowFunc.apply(
            a_data, b_data, a_data_t, b_data_t, group_lens, group_offs, trans_b, out_dtype, config, num_cu
        )
    if config.granularity == ScalingGranularity.BLOCKWISE:
        # raw activations; the weight may be raw or pre-quantised (the pair's forward member: forward
        # and dgrad read the same 128x128-block payload)
        return FP8GroupedGemmBlockFunc.apply(a_data, b_data, group_lens, group_offs, trans_b, out_dtype, config, num_cu)
    if config.granularity == ScalingGranularity.MX_BLOCKWISE:
        return FP8GroupedGemmMXFunc.apply(a_data, b_data, a_data_t, b_data_t, group_lens, group_offs, trans_b, out_dtype, config, num_cu)
    raise ValueError(f"Unsupported FP8 ScalingGranularity: {config.granularity}")
