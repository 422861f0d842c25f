"""Public FP8 quantize / dequantize ops (signatures of primus_turbo/pytorch/ops/quantization.py:52-269)."""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from primus_turbo_b200.pytorch.core.low_precision import ScalingGranularity, ScalingRecipe
from primus_turbo_b200.pytorch.core.low_precision import MXFP8_BLOCK_SIZE
from primus_turbo_b200.pytorch.kernels import custom_ops as _ops
from primus_turbo_b200.pytorch.kernels.quantization_impl import (
    dequantize_mxfp8_impl,
    grouped_dequantize_mxfp8_impl,
    grouped_quantize_mxfp8_impl,
    quantize_mxfp8_impl,
)

__all__ = [
    "quantize_fp8",
    "quantize_fp8_with_trans",
    "dequantize_fp8",
    "grouped_quantize_fp8",
    "grouped_quantize_fp8_with_trans",
    "grouped_dequantize_fp8",
]


def quantize_fp8(
    x: torch.Tensor,
    out_dtype: torch.dtype,
    granularity: ScalingGranularity,
    *,
    block_size: Optional[int] = None,
    axis: Optional[int] = None,
    scaling_recipe: Optional[ScalingRecipe] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(x_fp8, scale_inv)``.

    TENSORWISE: one scale.  ROWWISE: ``axis`` required, scale_inv keeps x's shape with 1 on axis.
    BLOCKWISE: ``block_size`` (128) required; ``scaling_recipe.use_2d_block`` selects one scale per
    128x128 tile (weights), otherwise ``axis`` picks 1x128 (axis 1/-1) or 128x1 (axis 0/-2) blocks.
    """
    if granularity == ScalingGranularity.TENSORWISE:
        return _ops.quantize_fp8_tensorwise(x, out_dtype)
    if granularity == ScalingGranularity.ROWWISE:
        if axis is None:
            raise ValueError("axis must be specified for rowwise FP8 quantization")
        assert x.is_contiguous(), "The x tensor must be contiguous."
        return _ops.quantize_fp8_rowwise(x, out_dtype, axis if axis >= 0 else axis + x.dim())
    if granularity == ScalingGranularity.BLOCKWISE:
        assert block_size is not None, "block_size must be specified for BLOCKWISE quantization"
        if scaling_recipe is not None and scaling_recipe.use_2d_block:
            return _ops.quant_fp8_blockwise_for_weight(x, out_dtype, block_size)
        assert axis is not None, "axis must be specified for 1D BLOCKWISE quantization"
        return _ops.quant_fp8_blockwise(x, out_dtype, axis, block_size)
    if granularity == ScalingGranularity.MX_BLOCKWISE:
        # x 2-D (axis 0: along columns, transposed copy; axis 1: along rows) or 3-D (axis 1 / 2); block 32
        assert block_size == MXFP8_BLOCK_SIZE, f"The block size must be {MXFP8_BLOCK_SIZE} for MXFP8 quantization"
        _reject_shuffle(scaling_recipe)
        return quantize_mxfp8_impl(
            x, out_dtype, axis, block_size, False, bool(scaling_recipe is not None and scaling_recipe.use_2d_block)
        )
    raise NotImplementedError(f"Unknown granularity {granularity}")


def _reject_shuffle(recipe: Optional[ScalingRecipe]) -> None:
    """The reference's pre-shuffled scale / data layouts feed its own GEMM back ends; this build's GEMM
    reads the plain layouts, so the options are refused instead of silently ignored."""
    if recipe is not None and (getattr(recipe, "shuffle_scale", False) or getattr(recipe, "shuffle_out", False)):
        raise NotImplementedError("shuffled MXFP8 layouts are not part of this build")


def quantize_fp8_with_trans(
    x: torch.Tensor,
    out_dtype: torch.dtype,
    granularity: ScalingGranularity,
    *,
    block_size: Optional[int] = None,
    scaling_recipe: Optional[ScalingRecipe] = None,
    scaling_recipe_for_trans: Optional[ScalingRecipe] = None,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """One read of x -> (row copy, row scales [M, N/128], column copy [M,N], column scales [M/128, N])."""
    if granularity == ScalingGranularity.BLOCKWISE:
        assert block_size is not None, "block_size must be specified for BLOCKWISE quantization"
        return _ops.quant_fp8_blockwise_dual(x, out_dtype, block_size)
    if granularity == ScalingGranularity.MX_BLOCKWISE:
        # -> (row copy [.., M, N_pad], scales [.., M, N_pad/32], transposed column copy [.., N, M_pad], scales [.., N, M_pad/32])
        assert block_size == MXFP8_BLOCK_SIZE, f"The block size must be {MXFP8_BLOCK_SIZE} for MXFP8 quantization"
        _reject_shuffle(scaling_recipe)
        _reject_shuffle(scaling_recipe_for_trans)
        return quantize_mxfp8_impl(
            x, out_dtype, None, block_size, True,
            bool(scaling_recipe is not None and scaling_recipe.use_2d_block),
            bool(scaling_recipe_for_trans is not None and scaling_recipe_for_trans.use_2d_block),
        )
    raise NotImplementedError(f"Unknown granularity {granularity}")


def grouped_quantize_fp8(
    x: torch.Tensor,
    out_dtype: torch.dtype,
    granularity: ScalingGranularity,
    group_lens: torch.Tensor,
    group_offs: torch.Tensor,
    *,
    block_size: Optional[int] = None,
    axis: Optional[int] = None,
    scaling_recipe: Optional[ScalingRecipe] = None,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """MXFP8 only (ops/quantization.py:143-176 in the reference): one direction of x [M, N] per group ->
    (data, scale_inv, group_lens_padded, group_offs_padded); axis 1: the row copy, groups padded to 32 rows;
    axis 0: the transposed column copy, groups padded to 128.  One kernel makes both directions here; the
    other one is dropped."""
    if granularity == ScalingGranularity.MX_BLOCKWISE:
        assert block_size == MXFP8_BLOCK_SIZE, f"The block size must be {MXFP8_BLOCK_SIZE} for MXFP8 quantization"
        assert axis in (0, 1), "The axis must be 0 or 1."
        _reject_shuffle(scaling_recipe)
        use_2d = bool(scaling_recipe is not None and scaling_recipe.use_2d_block)
        outs = grouped_quantize_mxfp8_impl(x, out_dtype, block_size, group_lens, group_offs, use_2d, use_2d)
        return (outs[0], outs[1], outs[4], outs[5]) if axis == 1 else (outs[2], outs[3], outs[6], outs[7])
    raise NotImplementedError(f"Unknown granularity {granularity}")


def grouped_dequantize_fp8(
    x: torch.Tensor,
    out_dtype: torch.dtype,
    granularity: ScalingGranularity,
    group_offs: torch.Tensor,
    group_offs_padded: torch.Tensor,
    *,
    block_size: Optional[int] = None,
    axis: Optional[int] = None,
    scale_inv: torch.Tensor,
    scaling_recipe: Optional[ScalingRecipe] = None,
    total_M: Optional[int] = None,
) -> torch.Tensor:
    """MXFP8 only (ops/quantization.py:272-296 in the reference): a grouped payload back to its packed rows."""
    if granularity == ScalingGranularity.MX_BLOCKWISE:
        assert block_size == MXFP8_BLOCK_SIZE, f"The block size must be {MXFP8_BLOCK_SIZE} for MXFP8 quantization"
        return grouped_dequantize_mxfp8_impl(
            x, out_dtype, axis, block_size, scale_inv, group_offs, group_offs_padded, total_M
        )
    raise NotImplementedError(f"Unknown granularity {granularity}")


def grouped_quantize_fp8_with_trans(
    x: torch.Tensor,
    out_dtype: torch.dtype,
    granularity: ScalingGranularity,
    group_lens: torch.Tensor,
    group_offs: torch.Tensor,
    *,
    block_size: Optional[int] = None,
    scaling_recipe: Optional[ScalingRecipe] = None,
    scaling_recipe_for_trans: Optional[ScalingRecipe] = None,
):
    """MXFP8 only (as in the reference, ops/quantization.py:181-222): both directions of x [M, N] per group;
    -> (x_rowwise, scale_rowwise, x_colwise_t, scale_colwise, group_lens_padded_rowwise,
    group_offs_padded_rowwise, group_lens_padded_colwise, group_offs_padded_colwise).  The row copy pads every
    group to 32 rows, the transposed column copy to 128."""
    if granularity == ScalingGranularity.MX_BLOCKWISE:
        assert block_size == MXFP8_BLOCK_SIZE, f"The block size must be {MXFP8_BLOCK_SIZE} for MXFP8 quantization"
        _reject_shuffle(scaling_recipe)
        _reject_shuffle(scaling_recipe_for_trans)
        return grouped_quantize_mxfp8_impl(
            x, out_dtype, block_size, group_lens, group_offs,
            bool(scaling_recipe is not None and scaling_recipe.use_2d_block),
            bool(scaling_recipe_for_trans is not None and scaling_recipe_for_trans.use_2d_block),
        )
    raise NotImplementedError(f"Unknown granularity {granularity}")


def dequantize_fp8(
    x: torch.Tensor,
    out_dtype: torch.dtype,
    granularity: ScalingGranularity,
    *,
    block_size: Optional[int] = None,
    axis: Optional[int] = None,
    scale_inv: torch.Tensor,
    scaling_recipe: Optional[ScalingRecipe] = None,
) -> torch.Tensor:
    if granularity == ScalingGranularity.TENSORWISE:
        return _ops.dequantize_fp8(x, scale_inv, out_dtype, 1, 0, 0)
    if granularity == ScalingGranularity.ROWWISE:
        if axis is None:
            raise ValueError("axis must be specified for rowwise FP8 de-quantization")
        return _ops.dequantize_fp8(x, scale_inv, out_dtype, 2, axis if axis >= 0 else axis + x.dim(), 0)
    if granularity == ScalingGranularity.BLOCKWISE:
        assert block_size is not None, "block_size must be specified for BLOCKWISE de-quantization"
        if scaling_recipe is not None and scaling_recipe.use_2d_block:
            return _ops.dequantize_fp8(x, scale_inv, out_dtype, 4, 0, block_size)
        assert axis is not None, "axis must be specified for 1D BLOCKWISE de-quantization"
        return _ops.dequantize_fp8(x, scale_inv, out_dtype, 3, axis, block_size)
    if granularity == ScalingGranularity.MX_BLOCKWISE:
        assert block_size == MXFP8_BLOCK_SIZE, f"The block size must be {MXFP8_BLOCK_SIZE} for MXFP8 quantization"
        return dequantize_mxfp8_impl(x, out_dtype, axis, block_size, scale_inv)
    raise NotImplementedError(f"Unknown granularity {granularity}")
