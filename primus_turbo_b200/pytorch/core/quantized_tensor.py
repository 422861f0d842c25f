"""``QuantizedTensor``: a wrapper tensor carrying an FP8 payload and its inverse scales.

API-compatible with primus_turbo/pytorch/core/quantized_tensor.py:113-145 (check_quantized_tensor),
:148-835 (QuantizedTensor) and :884-894 (QuantizedTensorPair) for the FP8 tensorwise / rowwise /
blockwise granularities and for (non-grouped) MXFP8 payloads: an MX tensor holds its FP8 bytes padded to a
multiple of 128 along the quantised direction (axis -1: ``[.., M, K_pad]``; axis -2: the TRANSPOSED copy
``[.., K, M_pad]``) and one E8M0 byte per 32 elements; its wrapper shape stays the logical one.  A grouped MX
activation holds the per-group padded layout of its direction (32 rows per group for the row copy, 128 for the
transposed column copy) together with the padded and the original group lengths / offsets.  FP4 payloads are
not part of this build.
"""

from __future__ import annotations

from typing import Any, NamedTuple, Optional, Tuple, Union

import torch

from primus_turbo_b200.pytorch.core.low_precision import (
    MXFP8_BLOCK_SIZE,
    MXFP8_PADDING_ALIGN_SIZE,
    Float8QuantConfig,
    ScalingGranularity,
    ScalingRecipe,
    float8_e4m3,
    float8_e5m2,
)

_FP8 = (float8_e4m3, float8_e5m2)
_GRANS = (
    ScalingGranularity.TENSORWISE,
    ScalingGranularity.ROWWISE,
    ScalingGranularity.BLOCKWISE,
    ScalingGranularity.MX_BLOCKWISE,
)


def _pad_inner_dim(shape, align: int):
    """``shape`` with its last extent rounded up to a multiple of ``align`` (the MX payloads' inner padding)."""
    if len(shape) == 0 or align <= 1:
        return tuple(shape)
    return (*shape[:-1], (shape[-1] + align - 1) // align * align)


def _norm_axis(axis: Optional[int], ndim: int) -> Optional[int]:
    if axis is None:
        return None
    return axis if axis >= 0 else axis + ndim


def check_quantized_tensor(
    quantized_tensor: "QuantizedTensor",
    config: Any,
    axis: Optional[int] = None,
    scaling_recipe: Optional[ScalingRecipe] = None,
) -> None:
    """Assert that a QuantizedTensor matches ``config`` (duck-typed: granularity, block_size)."""
    assert quantized_tensor.granularity == config.granularity, (
        f"QuantizedTensor granularity {quantized_tensor.granularity} does not match config "
        f"granularity {config.granularity}"
    )
    assert quantized_tensor.block_size == config.block_size, (
        f"QuantizedTensor block_size {quantized_tensor.block_size} does not match config "
        f"block_size {config.block_size}"
    )
    if axis is not None:
        want = _norm_axis(axis, quantized_tensor.qdata.ndim)
        have = _norm_axis(quantized_tensor.quantized_axis, quantized_tensor.qdata.ndim)
        assert have == want, f"QuantizedTensor quantized_axis {have} does not match axis={want}"
    if scaling_recipe is not None:
        assert quantized_tensor.scaling_recipe == scaling_recipe, (
            f"QuantizedTensor scaling_recipe {quantized_tensor.scaling_recipe} does not match config "
            f"scaling_recipe {scaling_recipe}"
        )


class QuantizedTensor(torch.Tensor):
    """Wrapper subclass: logical shape/dtype of the high-precision tensor, FP8 bytes inside."""

    @staticmethod
    def __new__(
        cls,
        data: torch.Tensor,
        scale_inv: torch.Tensor,
        *,
        shape,
        orig_dtype: torch.dtype,
        dest_dtype: torch.dtype,
        granularity: ScalingGranularity,
        orig_group_lens: Optional[torch.Tensor] = None,
        orig_group_offs: Optional[torch.Tensor] = None,
        group_lens: Optional[torch.Tensor] = None,
        group_offs: Optional[torch.Tensor] = None,
        is_grouped_tensor: bool = False,
        block_size: Optional[int] = None,
        scaling_recipe: Optional[ScalingRecipe] = None,
        quantized_axis: Optional[int] = None,
        requires_grad: bool = False,
    ):
        assert dest_dtype in _FP8, "Unsupported quantized dtype"
        assert data.is_contiguous(), "data must be contiguous"
        assert scale_inv.is_contiguous(), "scale_inv must be contiguous"
        self = torch.Tensor._make_wrapper_subclass(
            cls, shape, dtype=orig_dtype, layout=data.layout, requires_grad=requires_grad, device=data.device
        )
        self._data, self._scale_inv = data, scale_inv
        self._orig_dtype, self._dest_dtype = orig_dtype, dest_dtype
        self._granularity, self._block_size = granularity, block_size
        self._scaling_recipe = scaling_recipe
        self._quantized_axis = quantized_axis
        self._group_lens, self._group_offs = group_lens, group_offs
        self._orig_group_lens, self._orig_group_offs = orig_group_lens, orig_group_offs
        self._is_grouped_tensor = is_grouped_tensor
        return self

    # ---- construction ---------------------------------------------------------------------------
    @classmethod
    def quantize(
        cls,
        hp_tensor: torch.Tensor,
        dest_dtype: torch.dtype,
        granularity: ScalingGranularity,
        *,
        axis: Optional[int] = None,
        group_lens: Optional[torch.Tensor] = None,
        block_size: Optional[int] = None,
        scaling_recipe: Optional[ScalingRecipe] = None,
    ) -> "QuantizedTensor":
        from primus_turbo_b200.pytorch.kernels.gemm_impl import group_offs_from_lens
        from primus_turbo_b200.pytorch.ops.quantization import quantize_fp8

        assert hp_tensor.ndim in (2, 3), f"data must be a 2D or 3D tensor, got {hp_tensor.ndim}D"
        assert dest_dtype in _FP8, "Unsupported quantized dtype"
        assert granularity in _GRANS, f"Unsupported granularity {granularity}"
        if granularity == ScalingGranularity.BLOCKWISE:
            assert block_size is not None, "block_size must be provided for BLOCKWISE"
        if granularity == ScalingGranularity.MX_BLOCKWISE:
            assert block_size == MXFP8_BLOCK_SIZE, "block_size must be MXFP8_BLOCK_SIZE for MX_BLOCKWISE"
            assert scaling_recipe is not None, "scaling_recipe must be provided for MX_BLOCKWISE"
        if granularity != ScalingGranularity.TENSORWISE:
            assert axis is not None, "axis must be provided for non-TENSORWISE granularity"
        grouped = group_lens is not None
        g_lens = g_offs = p_lens = p_offs = None
        if grouped:
            assert granularity != ScalingGranularity.BLOCKWISE, (
                "grouped BLOCKWISE activations are quantised inside grouped_gemm_fp8"
            )
            assert hp_tensor.ndim == 2 and group_lens.is_cuda
            g_lens, g_offs = group_lens, group_offs_from_lens(group_lens)
        if grouped and granularity == ScalingGranularity.MX_BLOCKWISE:
            # every group quantised on its own into the padded layout of that direction (32 rows per group for
            # the row copy, 128 for the transposed column copy); the tensor keeps both sets of lengths / offsets
            # (:325-338 in the reference)
            from primus_turbo_b200.pytorch.ops.quantization import grouped_quantize_fp8

            with torch.no_grad():
                data, scale_inv, p_lens, p_offs = grouped_quantize_fp8(
                    hp_tensor.detach().contiguous(), dest_dtype, granularity, g_lens, g_offs, block_size=block_size,
                    axis=_norm_axis(axis, 2), scaling_recipe=scaling_recipe,
                )
        else:
            # Tensorwise / rowwise scales do not depend on the grouping: the packed [sum(M_g), K] tensor is
            # quantised as a whole and only carries the group metadata along.
            p_lens, p_offs = g_lens, g_offs
            with torch.no_grad():
                data, scale_inv = quantize_fp8(
                    hp_tensor.detach().contiguous(),
                    dest_dtype,
                    granularity,
                    block_size=block_size,
                    axis=_norm_axis(axis, hp_tensor.ndim),
                    scaling_recipe=scaling_recipe,
                )
        return cls(
            data,
            scale_inv,
            shape=hp_tensor.size(),
            orig_dtype=hp_tensor.dtype,
            dest_dtype=dest_dtype,
            granularity=granularity,
            block_size=block_size,
            scaling_recipe=scaling_recipe,
            requires_grad=hp_tensor.requires_grad,
            quantized_axis=axis,
            orig_group_lens=g_lens,
            orig_group_offs=g_offs,
            group_lens=p_lens,
            group_offs=p_offs,
            is_grouped_tensor=grouped,
        )

    # ---- accessors ------------------------------------------------------------------------------
    @property
    def qdata(self) -> torch.Tensor:
        return self._data

    @property
    def scale_inv(self) -> torch.Tensor:
        return self._scale_inv

    @property
    def group_lens(self):
        return self._group_lens

    @property
    def group_offs(self):
        return self._group_offs

    @property
    def real_dtype(self) -> torch.dtype:
        return self._dest_dtype

    @property
    def granularity(self) -> ScalingGranularity:
        return self._granularity

    @property
    def block_size(self):
        return self._block_size

    @property
    def scaling_recipe(self):
        return self._scaling_recipe

    @property
    def quantized_axis(self):
        """The axis the scales run along, as a non-negative index into the payload (the reference resolves
        negative axes the same way, quantized_tensor.py:507-509 there)."""
        return _norm_axis(self._quantized_axis, self._data.ndim)

    @torch.no_grad()
    def dequantize(self) -> torch.Tensor:
        """Back to the original high-precision dtype: cast(float(q) * scale_inv)."""
        from primus_turbo_b200.pytorch.ops.quantization import dequantize_fp8, grouped_dequantize_fp8

        if self._is_grouped_tensor and self._granularity == ScalingGranularity.MX_BLOCKWISE:
            # the padded layout back to the packed rows (:533-549 in the reference)
            out = grouped_dequantize_fp8(
                self._data, self._orig_dtype, self._granularity, self._orig_group_offs, self._group_offs,
                block_size=self._block_size, axis=_norm_axis(self._quantized_axis, 2), scale_inv=self._scale_inv,
                scaling_recipe=self._scaling_recipe, total_M=self.shape[0],
            )
            return out if out.shape == self.shape else out[:, : self.size(-1)].contiguous()
        out = dequantize_fp8(
            self._data,
            self._orig_dtype,
            self._granularity,
            block_size=self._block_size,
            axis=_norm_axis(self._quantized_axis, self._data.ndim),
            scale_inv=self._scale_inv,
            scaling_recipe=self._scaling_recipe,
        )
        if self._granularity == ScalingGranularity.MX_BLOCKWISE and out.shape != self.shape:
            # drop the zero padding of the quantised direction (the reference unpads the inner extent,
            # quantized_tensor.py:605-611 there; the transposed copy's padding lies on the other extent)
            out = out[..., : self.size(-2), : self.size(-1)].contiguous()
        return out

    # ---- torch.compile / FSDP flattening ----------------------------------------------------------
    def __tensor_flatten__(self):
        names = ["_data", "_scale_inv"]
        for n in ("_orig_group_lens", "_orig_group_offs", "_group_lens", "_group_offs"):
            if getattr(self, n) is not None:
                names.append(n)
        meta = {
            "_orig_dtype": self._orig_dtype,
            "_dest_dtype": self._dest_dtype,
            "_granularity": self._granularity,
            "_block_size": self._block_size,
            "_scaling_recipe": self._scaling_recipe,
            "_is_grouped_tensor": self._is_grouped_tensor,
            "_quantized_axis": self._quantized_axis,
        }
        return names, meta

    @staticmethod
    def __tensor_unflatten__(inner, meta, outer_size, outer_stride):
        return QuantizedTensor(
            inner["_data"],
            inner["_scale_inv"],
            shape=outer_size,
            orig_dtype=meta["_orig_dtype"],
            dest_dtype=meta["_dest_dtype"],
            granularity=meta["_granularity"],
            block_size=meta["_block_size"],
            scaling_recipe=meta["_scaling_recipe"],
            orig_group_lens=inner.get("_orig_group_lens"),
            orig_group_offs=inner.get("_orig_group_offs"),
            group_lens=inner.get("_group_lens"),
            group_offs=inner.get("_group_offs"),
            is_grouped_tensor=meta["_is_grouped_tensor"],
            quantized_axis=meta.get("_quantized_axis"),
        )

    def _like(self, data, scale_inv, shape) -> "QuantizedTensor":
        return QuantizedTensor(
            data,
            scale_inv,
            shape=shape,
            orig_dtype=self._orig_dtype,
            dest_dtype=self._dest_dtype,
            granularity=self._granularity,
            block_size=self._block_size,
            scaling_recipe=self._scaling_recipe,
            orig_group_lens=self._orig_group_lens,
            orig_group_offs=self._orig_group_offs,
            group_lens=self._group_lens,
            group_offs=self._group_offs,
            is_grouped_tensor=self._is_grouped_tensor,
            quantized_axis=self._quantized_axis,
            requires_grad=self.requires_grad,
        )

    @staticmethod
    def _view_data_and_scale_inv(tensor: "QuantizedTensor", target_shape, op):
        """Apply ``op`` (``Tensor.view`` or ``Tensor.reshape``) to the payload.  The target keeps the
        number of dimensions; the inverse scales are carried along unchanged, exactly as the reference
        does for its non-MX formats (quantized_tensor.py:700-740 there), so a caller who reshapes
        across a scaled axis owns the consequences."""
        assert len(target_shape) == tensor.qdata.ndim
        out_shape = torch.Size(target_shape)
        if out_shape == tensor.shape:
            return tensor._data, tensor._scale_inv, out_shape
        if tensor._granularity == ScalingGranularity.MX_BLOCKWISE:
            # the payload's inner extent is padded to 128 and every 32 of its elements own a scale byte: both
            # follow the new leading extents (row-direction payloads only; :709-731 in the reference)
            padded = _pad_inner_dim(tuple(target_shape), MXFP8_PADDING_ALIGN_SIZE)
            scale_shape = (*padded[:-1], padded[-1] // tensor._block_size)
            return op(tensor._data, *padded), op(tensor._scale_inv, *scale_shape), out_shape
        return op(tensor._data, *target_shape), tensor._scale_inv, out_shape

    def view(self, *shape) -> "QuantizedTensor":
        """View without dequantising (autograd-aware)."""
        return _ViewFunc.apply(self, _shape_arg(shape))

    def reshape(self, *shape) -> "QuantizedTensor":
        """Reshape without dequantising (autograd-aware)."""
        return _ReshapeFunc.apply(self, _shape_arg(shape))

    @classmethod
    def _transpose(cls, t: "QuantizedTensor", dim0: int, dim1: int) -> "QuantizedTensor":
        """TENSORWISE: exact byte transpose.  Other granularities: dequantise and re-quantise the
        transposed view along axis -2 (quantized_tensor.py:741-777 in the reference)."""
        from primus_turbo_b200.pytorch.kernels.quantization_impl import transpose_2d_fp8

        nd = t.dim()
        d0, d1 = _norm_axis(dim0, nd), _norm_axis(dim1, nd)
        if d0 == d1:
            return t._like(t._data, t._scale_inv, t.shape)
        assert not t._is_grouped_tensor, "transpose is not supported for grouped QuantizedTensor"
        assert {d0, d1} == {nd - 2, nd - 1}, "only the two innermost dimensions can be transposed"
        shape = list(t.shape)
        shape[d0], shape[d1] = shape[d1], shape[d0]
        if t._granularity == ScalingGranularity.TENSORWISE:
            return t._like(transpose_2d_fp8(t._data), t._scale_inv, torch.Size(shape))
        if t._granularity == ScalingGranularity.MX_BLOCKWISE:
            # the column-direction copy of the same logical tensor, whose payload IS the transposed layout
            # (:766-775 in the reference)
            return cls.quantize(
                t.dequantize(), t._dest_dtype, t._granularity, axis=-2, block_size=t._block_size,
                scaling_recipe=t._scaling_recipe,
            )
        return cls.quantize(
            t.dequantize().transpose(d0, d1).contiguous(),
            t._dest_dtype,
            t._granularity,
            axis=-2,
            block_size=t._block_size,
            scaling_recipe=t._scaling_recipe,
        )

    @classmethod
    def __torch_dispatch__(cls, func, types, args=(), kwargs=None):
        aten = torch.ops.aten
        t = args[0] if args else None
        if isinstance(t, QuantizedTensor):
            if func in (aten.detach.default, aten.alias.default):
                return t._like(t._data.detach(), t._scale_inv.detach(), t.shape)
            if func in (aten.t.default, aten.transpose.int):
                if func is aten.t.default:
                    assert t.dim() == 2, "t() expects a 2D QuantizedTensor"
                    return cls._transpose(t, 0, 1)
                return cls._transpose(t, args[1], args[2])
            if func is aten.select.int:
                return func(t._data, *args[1:], **(kwargs or {}))
            if func in (aten.view.default, aten._unsafe_view.default, aten.reshape.default):
                # only shape-preserving views keep the scale layout valid
                target = torch.Size(args[1])
                if t._granularity == ScalingGranularity.TENSORWISE:
                    return t._like(t._data.reshape(target), t._scale_inv, target)
                if t._granularity == ScalingGranularity.MX_BLOCKWISE:
                    data, scale_inv, shape = cls._view_data_and_scale_inv(t, target, torch.Tensor.reshape)
                    return t._like(data, scale_inv, shape)
                assert tuple(target) == tuple(t.shape), "only identity views are supported for scaled layouts"
                return t._like(t._data, t._scale_inv, t.shape)
            if func is aten.clone.default:
                return t._like(t._data.clone(), t._scale_inv.clone(), t.shape)
        raise NotImplementedError(f"Unsupported dispatch: {func}")

    __torch_function__ = torch._C._disabled_torch_function_impl

    def __repr__(self):  # pragma: no cover - debugging aid
        return (
            f"QuantizedTensor(shape={tuple(self.shape)}, dtype={self._dest_dtype}, "
            f"granularity={self._granularity.name}, axis={self._quantized_axis})"
        )


def _shape_arg(shape) -> Tuple[int, ...]:
    if len(shape) == 1 and isinstance(shape[0], (tuple, list, torch.Size)):
        shape = tuple(shape[0])
    return tuple(int(d) for d in shape)


def _resolve_minus_one(shape: Tuple[int, ...], numel: int) -> Tuple[int, ...]:
    if -1 not in shape:
        return shape
    known = 1
    for d in shape:
        if d != -1:
            known *= d
    return tuple(numel // max(known, 1) if d == -1 else d for d in shape)


class _ViewFunc(torch.autograd.Function):
    """View a QuantizedTensor without dequantising; the gradient is reshaped back
    (quantized_tensor.py:838-858 in the reference)."""

    @staticmethod
    def forward(ctx, tensor: QuantizedTensor, shape: Tuple[int, ...]) -> QuantizedTensor:
        ctx.shape = tensor.shape
        shape = _resolve_minus_one(shape, tensor.numel())
        data, sinv, out_shape = QuantizedTensor._view_data_and_scale_inv(tensor, shape, torch.Tensor.view)
        return tensor._like(data, sinv, out_shape)

    @staticmethod
    def backward(ctx, grad):
        return grad.reshape(ctx.shape), None


class _ReshapeFunc(torch.autograd.Function):
    """Reshape a QuantizedTensor without dequantising (quantized_tensor.py:861-881 in the reference)."""

    @staticmethod
    def forward(ctx, tensor: QuantizedTensor, shape: Tuple[int, ...]) -> QuantizedTensor:
        ctx.shape = tensor.shape
        shape = _resolve_minus_one(shape, tensor.numel())
        data, sinv, out_shape = QuantizedTensor._view_data_and_scale_inv(tensor, shape, torch.Tensor.reshape)
        return tensor._like(data, sinv, out_shape)

    @staticmethod
    def backward(ctx, grad):
        return grad.reshape(ctx.shape), None


class QuantizedTensorPair(NamedTuple):
    """Row-wise quantised tensor plus the optional column-wise (backward) companion."""

    data: QuantizedTensor
    data_t: Optional[QuantizedTensor] = None


def create_quantized_weight(
    weight: torch.Tensor,
    dest_dtype: torch.dtype,
    quant_config: Float8QuantConfig,
    need_weight_transpose_cache: bool = False,
) -> Tuple[QuantizedTensor, Optional[QuantizedTensor]]:
    """Quantise a weight once, optionally with its backward-direction companion
    (quantized_tensor.py:897-956 in the reference)."""
    g = quant_config.granularity
    blocked = g in (ScalingGranularity.BLOCKWISE, ScalingGranularity.MX_BLOCKWISE)
    recipe = ScalingRecipe(use_2d_block=True) if blocked else ScalingRecipe()
    qw = QuantizedTensor.quantize(
        weight, dest_dtype, g, block_size=quant_config.block_size, scaling_recipe=recipe, axis=-1
    )
    qw_t = None
    if need_weight_transpose_cache:
        if g == ScalingGranularity.TENSORWISE:
            qw_t = qw.transpose(-2, -1)
        elif g == ScalingGranularity.ROWWISE:
            qw_t = QuantizedTensor.quantize(
                weight.transpose(-2, -1).contiguous(), dest_dtype, g, block_size=quant_config.block_size,
                scaling_recipe=recipe, axis=-2,
            )
        elif blocked:
            # axis -2 of the same weight: for MX the payload of that copy is the transposed layout
            qw_t = QuantizedTensor.quantize(
                weight, dest_dtype, g, block_size=quant_config.block_size, scaling_recipe=recipe, axis=-2
            )
        else:
            raise ValueError(f"Unsupported granularity: {g}")
    return qw, qw_t


__all__ = ["QuantizedTensor", "QuantizedTensorPair", "check_quantized_tensor", "create_quantized_weight"]
