"""``torch.library.custom_op`` registrations of the kernel wrappers, each with a fake (meta)
implementation, so that ``torch.compile`` / FakeTensor tracing treat them as opaque ops with known
output shapes -- the role the reference's ``register_fake`` functions play
(primus_turbo/pytorch/kernels/quantization/quantization_impl.py:121-137,275-292,353-376 and
primus_turbo/pytorch/kernels/gemm/gemm_fp8_impl.py:470-486).  The eager bodies are the ctypes
wrappers in ``quantization_impl`` / ``gemm_impl``; nothing here computes anything itself.
"""

from typing import List, Optional, Tuple

import torch

from primus_turbo_b200.pytorch.kernels import gemm_impl as _g
from primus_turbo_b200.pytorch.kernels import quantization_impl as _q

_NS = "primus_turbo_b200"


def _cdiv(a: int, b: int) -> int:
    return (a + b - 1) // b


# ---- quantize ----------------------------------------------------------------------------------------
@torch.library.custom_op(f"{_NS}::quantize_fp8_tensorwise", mutates_args=())
def quantize_fp8_tensorwise(x: torch.Tensor, out_dtype: torch.dtype) -> Tuple[torch.Tensor, torch.Tensor]:
    return _q.quantize_fp8_tensorwise_impl(x, out_dtype)


@quantize_fp8_tensorwise.register_fake
def _(x, out_dtype):
    return torch.empty(x.shape, dtype=out_dtype, device=x.device), torch.empty((), dtype=torch.float32, device=x.device)


@torch.library.custom_op(f"{_NS}::quantize_fp8_rowwise", mutates_args=())
def quantize_fp8_rowwise(x: torch.Tensor, out_dtype: torch.dtype, axis: int) -> Tuple[torch.Tensor, torch.Tensor]:
    return _q.quantize_fp8_rowwise_impl(x, out_dtype, axis)


@quantize_fp8_rowwise.register_fake
def _(x, out_dtype, axis):
    shape = list(x.shape)
    shape[axis] = 1
    return torch.empty(x.shape, dtype=out_dtype, device=x.device), torch.empty(shape, dtype=torch.float32, device=x.device)


@torch.library.custom_op(f"{_NS}::quant_fp8_blockwise", mutates_args=())
def quant_fp8_blockwise(x: torch.Tensor, dtype: torch.dtype, axis: int, block_size: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    return _q.quant_fp8_blockwise_impl(x, dtype, axis, block_size)


@quant_fp8_blockwise.register_fake
def _(x, dtype, axis, block_size=128):
    assert x.dim() == 2, "Input must be 2D"
    M, N = x.shape
    s = (M, _cdiv(N, block_size)) if axis % 2 == 1 else (_cdiv(M, block_size), N)
    return torch.empty((M, N), dtype=dtype, device=x.device), torch.empty(s, dtype=torch.float32, device=x.device)


@torch.library.custom_op(f"{_NS}::quant_fp8_blockwise_dual", mutates_args=())
def quant_fp8_blockwise_dual(
    x: torch.Tensor, dtype: torch.dtype, block_size: int = 128
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    return _q.quant_fp8_blockwise_dual_impl(x, dtype, block_size)


@quant_fp8_blockwise_dual.register_fake
def _(x, dtype, block_size=128):
    assert x.dim() == 2, "Input must be 2D"
    M, N = x.shape
    f32 = dict(dtype=torch.float32, device=x.device)
    return (
        torch.empty((M, N), dtype=dtype, device=x.device),
        torch.empty((M, _cdiv(N, block_size)), **f32),
        torch.empty((M, N), dtype=dtype, device=x.device),
        torch.empty((_cdiv(M, block_size), N), **f32),
    )


@torch.library.custom_op(f"{_NS}::quant_fp8_blockwise_for_weight", mutates_args=())
def quant_fp8_blockwise_for_weight(w: torch.Tensor, dtype: torch.dtype, block_size: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    return _q.quant_fp8_blockwise_for_weight_impl(w, dtype, block_size)


@quant_fp8_blockwise_for_weight.register_fake
def _(w, dtype, block_size=128):
    assert w.dim() in (2, 3)
    s = (*w.shape[:-2], _cdiv(w.shape[-2], block_size), _cdiv(w.shape[-1], block_size))
    return torch.empty(w.shape, dtype=dtype, device=w.device), torch.empty(s, dtype=torch.float32, device=w.device)


@torch.library.custom_op(f"{_NS}::quant_fp8_blockwise_segment_m_row_col", mutates_args=())
def quant_fp8_blockwise_segment_m_row_col(
    x: torch.Tensor, dtype: torch.dtype, block_size: int, group_lens: torch.Tensor, group_offs: torch.Tensor
) -> List[torch.Tensor]:
    return list(_q.quant_fp8_blockwise_segment_m_row_col_impl(x, dtype, block_size, group_lens, group_offs))


@quant_fp8_blockwise_segment_m_row_col.register_fake
def _(x, dtype, block_size, group_lens, group_offs):
    M, N = x.shape
    G = group_lens.shape[0]
    mp = M + G * block_size
    dev = x.device
    return [
        torch.empty((M, N), dtype=dtype, device=dev),
        torch.empty((mp, N), dtype=dtype, device=dev),
        torch.empty((_cdiv(N, block_size), M), dtype=torch.float32, device=dev),
        torch.empty((_cdiv(mp, block_size), N), dtype=torch.float32, device=dev),
        torch.empty((G,), dtype=torch.int64, device=dev),
        torch.empty((G + 1,), dtype=torch.int64, device=dev),
    ]


# ---- dequantize ---------------------------------------------------------------------------------------
@torch.library.custom_op(f"{_NS}::dequantize_fp8", mutates_args=())
def dequantize_fp8(
    x: torch.Tensor, scale_inv: torch.Tensor, out_dtype: torch.dtype, kind: int, axis: int, block_size: int
) -> torch.Tensor:
    """kind: 1 tensorwise, 2 rowwise, 3 blockwise 1-D, 4 blockwise 2-D."""
    if kind == 1:
        return _q.dequantize_fp8_tensorwise_impl(x, out_dtype, scale_inv)
    if kind == 2:
        return _q.dequantize_fp8_rowwise_impl(x, out_dtype, axis, scale_inv)
    if kind == 3:
        return _q.dequant_fp8_blockwise_impl(x, scale_inv, out_dtype, axis, block_size)
    return _q.dequant_fp8_blockwise_for_weight_impl(x, scale_inv, out_dtype, block_size)


@dequantize_fp8.register_fake
def _(x, scale_inv, out_dtype, kind, axis, block_size):
    return torch.empty(x.shape, dtype=out_dtype, device=x.device)


# ---- GEMM ----------------------------------------------------------------------------------------------
@torch.library.custom_op(f"{_NS}::gemm_fp8_impl", mutates_args=())
def gemm_fp8_impl(
    a: torch.Tensor, a_scale_inv: torch.Tensor, trans_a: bool, b: torch.Tensor, b_scale_inv: torch.Tensor,
    trans_b: bool, out_dtype: torch.dtype, trans_c: bool, granularity: int,
) -> torch.Tensor:
    return _g.gemm_fp8_impl(a, a_scale_inv, trans_a, b, b_scale_inv, trans_b, out_dtype, trans_c, granularity)


@gemm_fp8_impl.register_fake
def _(a, a_scale_inv, trans_a, b, b_scale_inv, trans_b, out_dtype, trans_c, granularity):
    m, n, _k = _g.get_gemm_logical_shape(a, b, trans_a, trans_b)
    if trans_c:
        m, n = n, m
    return torch.empty((m, n), dtype=out_dtype, device=a.device)


@torch.library.custom_op(f"{_NS}::grouped_gemm_fp8_impl", mutates_args=())
def grouped_gemm_fp8_impl(
    a: torch.Tensor, b: torch.Tensor, a_scales: torch.Tensor, b_scales: torch.Tensor, group_lens: torch.Tensor,
    group_offs: torch.Tensor, trans_a: bool, trans_b: bool, out_dtype: torch.dtype, granularity: int,
    num_cu: Optional[int] = None,
) -> torch.Tensor:
    return _g.grouped_gemm_fp8_impl(a, b, a_scales, b_scales, group_lens, group_offs, trans_a, trans_b, out_dtype,
                                    granularity, num_cu)


@grouped_gemm_fp8_impl.register_fake
def _(a, b, a_scales, b_scales, group_lens, group_offs, trans_a, trans_b, out_dtype, granularity, num_cu=None):
    n = b.shape[1] if trans_b else b.shape[2]
    return torch.empty((a.shape[0], n), dtype=out_dtype, device=a.device)


@torch.library.custom_op(f"{_NS}::grouped_gemm_fp8_variable_k_impl", mutates_args=())
def grouped_gemm_fp8_variable_k_impl(
    a: torch.Tensor, b: torch.Tensor, a_scales: torch.Tensor, b_scales: torch.Tensor, group_lens: torch.Tensor,
    group_offs: torch.Tensor, trans_a: bool, trans_b: bool, trans_c: bool, out_dtype: torch.dtype, granularity: int,
    num_cu: Optional[int] = None,
) -> torch.Tensor:
    return _g.grouped_gemm_fp8_variable_k_impl(a, b, a_scales, b_scales, group_lens, group_offs, trans_a, trans_b,
                                               trans_c, out_dtype, granularity, num_cu)


@grouped_gemm_fp8_variable_k_impl.register_fake
def _(a, b, a_scales, b_scales, group_lens, group_offs, trans_a, trans_b, trans_c, out_dtype, granularity,
      num_cu=None):
    G = group_offs.shape[0] - 1
    m, n = (b.shape[1], a.shape[1]) if trans_c else (a.shape[1], b.shape[1])
    return torch.empty((G, m, n), dtype=out_dtype, device=a.device)


# ---- eager fast path ----------------------------------------------------------------------------------------
# Outside tracing, a registered op's Python dispatcher (autograd wrapper, redispatch, dynamo frame guard) costs
# about 70 us per call -- several times the ctypes call it wraps, and with six such calls per grouped-GEMM
# step it is most of the host time of a step, which is what paces a short multi-GPU step.  The public names of
# this module therefore run the op's own body directly in plain eager mode and go through the registered op
# only while compiling or under a dispatch mode (FakeTensorMode, functionalisation, ...), where the op and its
# fake kernel are what the tracer needs.  Same function either way; `.op` is the registered op.
def _with_eager_fast_path(op):
    body = op._init_fn  # the undecorated function the op was created from

    def call(*args, **kwargs):
        if torch.compiler.is_compiling() or torch._C._len_torch_dispatch_stack() > 0:
            return op(*args, **kwargs)
        return body(*args, **kwargs)

    call.__name__ = call.__qualname__ = body.__name__
    call.__doc__ = body.__doc__
    call.op = op
    return call


for _name in ("quantize_fp8_tensorwise", "quantize_fp8_rowwise", "quant_fp8_blockwise", "quant_fp8_blockwise_dual",
              "quant_fp8_blockwise_for_weight", "quant_fp8_blockwise_segment_m_row_col", "dequantize_fp8", "gemm_fp8_impl",
              "grouped_gemm_fp8_impl", "grouped_gemm_fp8_variable_k_impl"):
    globals()[_name] = _with_eager_fast_path(globals()[_name])
del _name
