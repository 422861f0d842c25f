"""``gemm_fp8``: FP8 dense GEMM with autograd (primus_turbo/pytorch/ops/gemm_fp8.py:58-743).

The three autograd Functions keep the reference's quantisation schedule exactly, because it
defines the numbers a caller sees:
  * TENSORWISE (:58-228): a, b and grad_out each quantised once with one scale; dgrad / wgrad reuse
    the forward payloads.  The reference materialises transposed copies on its newer GPUs; here the
    tensor cores read transposed operands in place, which gives the same values with no copy.
  * ROWWISE (:231-379): backward operands are re-quantised from the *dequantised* forward operands
    along the other axis; grad_out is quantised twice from the original.
  * BLOCKWISE (:382-506): a -> 1x128 row copy + 128x1 column copy in one pass, b -> 128x128 tiles
    reused in backward, grad_out -> row + column copies.
  * MX_BLOCKWISE (:509-647): every operand is quantised in both directions in one pass (1x32 blocks for
    a and grad_out, 32x32 for b), the column copies are stored transposed, so forward, dgrad and wgrad
    are all "NT" products of K-major operands whose E8M0 scales the tensor cores apply themselves.
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
from primus_turbo_b200.pytorch.kernels.custom_ops import gemm_fp8_impl
from primus_turbo_b200.pytorch.kernels.gemm_impl import gemm_mxfp8_impl
from primus_turbo_b200.pytorch.ops.quantization import quantize_fp8, quantize_fp8_with_trans

__all__ = ["gemm_fp8"]


def _get_fp8_dtype(format: Format, is_fwd_stage: bool):
    if format == Format.E4M3:
        return float8_e4m3
    if format == Format.E5M2:
        return float8_e5m2
    if format == Format.HYBRID:
        return float8_e4m3 if is_fwd_stage else float8_e5m2
    raise ValueError(f"Unsupported FP8 format: {format}")


def _q(x, dtype, config, axis):
    return QuantizedTensor.quantize(x, dtype, config.granularity, axis=axis, block_size=config.block_size)


class FP8GemmTensorFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, a_t, b_t, trans_a, trans_b, out_dtype, config):
        g = config.granularity.value
        if isinstance(a, QuantizedTensor):
            check_quantized_tensor(a, config)
            qa = a
        else:
            qa = _q(a, _get_fp8_dtype(config.format, True), config, -1)
        if isinstance(b, QuantizedTensor):
            check_quantized_tensor(b, config)
            qb = b
        else:
            qb = _q(b, _get_fp8_dtype(config.format, True), config, -1)
        out = gemm_fp8_impl(qa.qdata, qa.scale_inv, trans_a, qb.qdata, qb.scale_inv, trans_b, out_dtype, False, g)
        ctx.save_for_backward(qa.qdata, qa.scale_inv, qb.qdata, qb.scale_inv)
        ctx.trans_a, ctx.trans_b, ctx.out_dtype, ctx.config = trans_a, trans_b, out_dtype, config
        return out

    @staticmethod
    def backward(ctx, grad_out):
        grad_out = grad_out.contiguous()
        a8, a_s, b8, b_s = ctx.saved_tensors
        g = ctx.config.granularity.value
        qg = QuantizedTensor.quantize(
            grad_out, _get_fp8_dtype(ctx.config.format, False), ctx.config.granularity, axis=-1
        )
        a_grad = gemm_fp8_impl(
            qg.qdata, qg.scale_inv, False, b8, b_s, not ctx.trans_b, ctx.out_dtype, ctx.trans_a, g
        )
        b_grad = gemm_fp8_impl(
            a8, a_s, not ctx.trans_a, qg.qdata, qg.scale_inv, False, ctx.out_dtype, ctx.trans_b, g
        )
        return a_grad, b_grad, None, None, None, None, None, None


class FP8GemmRowFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, a_t, b_t, trans_a, trans_b, out_dtype, config):
        assert trans_a == False, "trans_a has to be False"
        g = config.granularity.value
        fwd_dtype = _get_fp8_dtype(config.format, True)
        if isinstance(a, QuantizedTensor):
            check_quantized_tensor(a, config, axis=-1)
            qa = a
        else:
            qa = _q(a, fwd_dtype, config, -1)
        if a_t is None:
            qa_t = _q(qa.dequantize(), qa.real_dtype, config, -2)
        else:
            assert isinstance(a_t, QuantizedTensor)
            qa_t = a_t
        b_axis = -1 if trans_b else -2
        if isinstance(b, QuantizedTensor):
            check_quantized_tensor(b, config, axis=b_axis)
            qb = b
        else:
            qb = _q(b, fwd_dtype, config, b_axis)
        if b_t is None:
            qb_t = _q(qb.dequantize(), qb.real_dtype, config, -2 if trans_b else -1)
        else:
            assert isinstance(b_t, QuantizedTensor)
            qb_t = b_t
        out = gemm_fp8_impl(qa.qdata, qa.scale_inv, trans_a, qb.qdata, qb.scale_inv, trans_b, out_dtype, False, g)
        ctx.save_for_backward(qa_t.qdata, qa_t.scale_inv, qb_t.qdata, qb_t.scale_inv)
        ctx.trans_a, ctx.trans_b, ctx.out_dtype, ctx.config = trans_a, trans_b, out_dtype, config
        return out

    @staticmethod
    def backward(ctx, grad_out):
        grad_out = grad_out.contiguous()
        a8_t, a_t_s, b8_t, b_t_s = ctx.saved_tensors
        cfg = ctx.config
        g = cfg.granularity.value
        gdt = _get_fp8_dtype(cfg.format, False)
        qg = _q(grad_out, gdt, cfg, -1)
        a_grad = gemm_fp8_impl(
            qg.qdata, qg.scale_inv, False, b8_t, b_t_s, not ctx.trans_b, ctx.out_dtype, ctx.trans_a, g
        )
        qg_t = _q(grad_out, gdt, cfg, -2)
        b_grad = gemm_fp8_impl(
            a8_t, a_t_s, not ctx.trans_a, qg_t.qdata, qg_t.scale_inv, False, ctx.out_dtype, ctx.trans_b, g
        )
        return a_grad, b_grad, None, None, None, None, None, None


class FP8GemmBlockFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, a_t, b_t, trans_a, trans_b, out_dtype, config):
        assert trans_a == False, "trans_a has to be False"
        g = config.granularity.value
        dt = _get_fp8_dtype(config.format, True)
        if isinstance(a, QuantizedTensor):
            check_quantized_tensor(a, config, axis=-1)
            a_row, a_row_s = a.qdata, a.scale_inv
            if a_t is None:
                a_t = _q(a.dequantize(), dt, config, -2)
            a_col, a_col_s = a_t.qdata, a_t.scale_inv
        else:
            a_row, a_row_s, a_col, a_col_s = quantize_fp8_with_trans(
                a.contiguous(), dt, config.granularity, block_size=config.block_size
            )
        recipe = ScalingRecipe(use_2d_block=True)
        if isinstance(b, QuantizedTensor):
            check_quantized_tensor(b, config, scaling_recipe=recipe)
            b8, b_s = b.qdata, b.scale_inv
        else:
            b8, b_s = quantize_fp8(b, dt, config.granularity, block_size=config.block_size, scaling_recipe=recipe)
        out = gemm_fp8_impl(a_row, a_row_s, trans_a, b8, b_s, trans_b, out_dtype, False, g)
        ctx.save_for_backward(a_col, a_col_s, b8, b_s)
        ctx.trans_a, ctx.trans_b, ctx.out_dtype, ctx.config = trans_a, trans_b, out_dtype, config
        return out

    @staticmethod
    def backward(ctx, grad_out):
        a_col, a_col_s, b8, b_s = ctx.saved_tensors
        cfg = ctx.config
        g = cfg.granularity.value
        grad_out = grad_out.contiguous()
        g_row, g_row_s, g_col, g_col_s = quantize_fp8_with_trans(
            grad_out, _get_fp8_dtype(cfg.format, False), cfg.granularity, block_size=cfg.block_size
        )
        grad_a = gemm_fp8_impl(g_row, g_row_s, False, b8, b_s, not ctx.trans_b, ctx.out_dtype, False, g)
        grad_b = gemm_fp8_impl(a_col, a_col_s, not ctx.trans_a, g_col, g_col_s, False, ctx.out_dtype, ctx.trans_b, g)
        return grad_a, grad_b, None, None, None, None, None, None


class FP8GemmMXFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, a_t, b_t, trans_a, trans_b, out_dtype, config):
        assert trans_a == False and trans_b == True, "trans_a has to be False and trans_b has to be True"
        dt = _get_fp8_dtype(config.format, True)

        def both_directions(x, x_t, recipe):
            """(row copy, its scales, transposed column copy, its scales) of one operand.  A pre-quantised
            operand brings its row copy; its column copy comes from ``x_t`` or, as in the reference (:537-548),
            from re-quantising the dequantised row copy along the other axis."""
            if not isinstance(x, QuantizedTensor):
                return quantize_fp8_with_trans(
                    x.contiguous(), dt, config.granularity, block_size=config.block_size, scaling_recipe=recipe,
                    scaling_recipe_for_trans=recipe,
                )
            check_quantized_tensor(x, config, axis=-1, scaling_recipe=recipe)
            if x_t is None:
                x_t = QuantizedTensor.quantize(
                    x.dequantize(), x.real_dtype, config.granularity, axis=-2, block_size=config.block_size,
                    scaling_recipe=recipe,
                )
            else:
                assert isinstance(x_t, QuantizedTensor)
                check_quantized_tensor(x_t, config, axis=-2, scaling_recipe=recipe)
            return x.qdata, x.scale_inv, x_t.qdata, x_t.scale_inv

        a_row, a_row_s, a_col, a_col_s = both_directions(a, a_t, ScalingRecipe())
        b_row, b_row_s, b_col, b_col_s = both_directions(b, b_t, ScalingRecipe(use_2d_block=True))
        out = gemm_mxfp8_impl(a_row, a_row_s, b_row, b_row_s, out_dtype)  # [M, K_pad] x [N, K_pad]^T
        ctx.save_for_backward(a_col, a_col_s, b_col, b_col_s)
        ctx.out_dtype, ctx.config = out_dtype, config
        return out

    @staticmethod
    def backward(ctx, grad_out):
        a_col, a_col_s, b_col, b_col_s = ctx.saved_tensors
        cfg = ctx.config
        grad_out = grad_out.reshape(grad_out.shape[0], -1).contiguous()
        g_row, g_row_s, g_col, g_col_s = quantize_fp8_with_trans(
            grad_out, _get_fp8_dtype(cfg.format, False), cfg.granularity, block_size=cfg.block_size
        )
        grad_a = gemm_mxfp8_impl(g_row, g_row_s, b_col, b_col_s, ctx.out_dtype)  # [M, N_pad] x [K, N_pad]^T
        grad_b = gemm_mxfp8_impl(g_col, g_col_s, a_col, a_col_s, ctx.out_dtype)  # [N, M_pad] x [K, M_pad]^T
        return grad_a, grad_b, None, None, None, None, None, None


@torch._dynamo.disable(recursive=True, reason="builds QuantizedTensor wrappers inside autograd.Function.forward")
def gemm_fp8(
    a: Union[torch.Tensor, QuantizedTensor, QuantizedTensorPair],
    b: Union[torch.Tensor, QuantizedTensor, QuantizedTensorPair],
    trans_a: bool = False,
    trans_b: bool = False,
    out_dtype: Optional[torch.dtype] = None,
    config: Optional[Float8QuantConfig] = None,
) -> torch.Tensor:
    """``op(a) @ op(b)`` with FP8 quantisation of both operands (and of the gradients in backward).

    a: (M, K) or (K, M) if trans_a; b: (K, N) or (N, K) if trans_b; 2-D only.  Default config is
    TENSORWISE / E4M3.  Output dtype defaults to ``promote_types(a.dtype, b.dtype)``.
    """
    if config is None:
        config = Float8QuantConfig()
    a_data, a_data_t = (a.data, a.data_t) if isinstance(a, QuantizedTensorPair) else (a, None)
    b_data, b_data_t = (b.data, b.data_t) if isinstance(b, QuantizedTensorPair) else (b, None)
    assert a_data.ndim == 2, "Only 2D tensors are supported"
    assert b_data.ndim == 2, "Only 2D tensors are supported"
    if out_dtype is None:
        out_dtype = torch.promote_types(a_data.dtype, b_data.dtype)
    args = (a_data, b_data, a_data_t, b_data_t, trans_a, trans_b, out_dtype, config)
    if config.granularity == ScalingGranularity.TENSORWISE:
        return FP8GemmTensorFunction.apply(*args)
    if config.granularity == ScalingGranularity.ROWWISE:
        return FP8GemmRowFunction.apply(*args)
    if config.granularity == ScalingGranularity.BLOCKWISE:
        return FP8GemmBlockFunction.apply(*args)
    if config.granularity == ScalingGranularity.MX_BLOCKWISE:
        return FP8GemmMXFunction.apply(*args)
    raise ValueError(f"Unsupported FP8 ScalingGranularity: {config.granularity}")
