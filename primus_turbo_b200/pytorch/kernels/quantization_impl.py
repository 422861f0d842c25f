"""Thin torch layer over the quantize / dequantize entry points of the C ABI.

Each function allocates its outputs with torch on the input's device and passes raw pointers and
the current CUDA stream to the library, the way the reference's C++ bindings allocate with
``at::empty`` and enqueue on the current stream (csrc/pytorch/quantization/quantization.cpp:48,77).
Function names and return conventions follow
primus_turbo/pytorch/kernels/quantization/quantization_impl.py.
"""

from __future__ import annotations

from typing import Tuple

import torch

from primus_turbo_b200 import _lib
from primus_turbo_b200._lib import dtype_code, ptr, require_cuda, stream_of


def ceil_div(a: int, b: int) -> int:
    return (a + b - 1) // b


def _check_in(x: torch.Tensor, allow_fp32: bool = True) -> None:
    require_cuda(x)
    ok = (torch.float16, torch.bfloat16, torch.float32) if allow_fp32 else (torch.float16, torch.bfloat16)
    if x.dtype not in ok:
        raise _lib.PtbError(f"input dtype {x.dtype} is not supported")


def quantize_fp8_tensorwise_impl(x: torch.Tensor, out_dtype: torch.dtype, scale: torch.Tensor | None = None):
    """quantization.cpp:42-88: returns (x_fp8, scale_inv[]) ."""
    _check_in(x)
    xc = x.contiguous()
    q = torch.empty(xc.shape, dtype=out_dtype, device=x.device)
    scale_inv = torch.empty((), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        if scale is None:
            ws = torch.empty(_lib.PTB_TENSORWISE_WS_BYTES, dtype=torch.uint8, device=x.device)
            _lib.call(
                "ptb_quant_fp8_tensorwise", ptr(xc), dtype_code(xc.dtype), xc.numel(), ptr(q),
                dtype_code(out_dtype), ptr(scale_inv), ptr(ws), stream_of(x),
            )
        else:
            assert scale.numel() == 1, "tensorwise scale must be scalar tensor"
            sc = scale.to(device=x.device, dtype=torch.float32).contiguous()
            _lib.call(
                "ptb_quant_fp8_tensorwise_with_scale", ptr(xc), dtype_code(xc.dtype), xc.numel(), ptr(sc),
                ptr(q), dtype_code(out_dtype), ptr(scale_inv), stream_of(x),
            )
    return q, scale_inv


def _bmn(shape, axis: int) -> Tuple[int, int, int]:
    B = 1
    for d in shape[:axis]:
        B *= d
    N = 1
    for d in shape[axis + 1 :]:
        N *= d
    return B, shape[axis], N


def quantize_fp8_rowwise_impl(x: torch.Tensor, out_dtype: torch.dtype, axis: int):
    """quantization.cpp:108-206: scale_inv keeps x's shape with shape[axis] = 1."""
    _check_in(x)
    assert x.is_contiguous(), "The x tensor must be contiguous."
    nd = x.dim()
    ax = axis if axis >= 0 else nd + axis
    if not (0 <= ax < nd):
        raise _lib.PtbError(f"axis {axis} out of range for a {nd}-d tensor")
    B, M, N = _bmn(tuple(x.shape), ax)
    sshape = list(x.shape)
    sshape[ax] = 1
    q = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    scale_inv = torch.empty(sshape, dtype=torch.float32, device=x.device)
    ws = torch.empty(max(B * N, 1), dtype=torch.float32, device=x.device) if N > 1 else None
    with torch.cuda.device(x.device):
        _lib.call(
            "ptb_quant_fp8_rowwise", ptr(x), dtype_code(x.dtype), B, M, N, ptr(q), dtype_code(out_dtype),
            ptr(scale_inv), ptr(ws), stream_of(x),
        )
    return q, scale_inv


def quant_fp8_blockwise_impl(x: torch.Tensor, dtype: torch.dtype, axis: int, block_size: int = 128):
    """quantization_impl.py:74-118."""
    assert x.is_contiguous() and x.dim() == 2, "Input must be 2D and contiguous"
    assert axis in (-2, -1, 0, 1), f"axis must be 0 or 1 (or -1, -2), got {axis}"
    assert block_size == 128, "Only block_size 128 is supported"
    _check_in(x)
    axis = axis % 2
    M, N = x.shape
    q = torch.empty((M, N), dtype=dtype, device=x.device)
    sshape = (M, ceil_div(N, block_size)) if axis == 1 else (ceil_div(M, block_size), N)
    s = torch.empty(sshape, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.call(
            "ptb_quant_fp8_block1d", ptr(x), dtype_code(x.dtype), M, N, axis, ptr(q), dtype_code(dtype),
            ptr(s), stream_of(x),
        )
    return q, s


def quant_fp8_blockwise_dual_impl(x: torch.Tensor, dtype: torch.dtype, block_size: int = 128):
    """quantization_impl.py:229-274: (row copy, row scales [M, N/128], col copy, col scales [M/128, N])."""
    assert x.is_contiguous() and x.dim() == 2, "Input must be 2D and contiguous"
    assert block_size == 128, "Only block_size 128 is supported"
    _check_in(x)
    M, N = x.shape
    q_row = torch.empty((M, N), dtype=dtype, device=x.device)
    s_row = torch.empty((M, ceil_div(N, block_size)), dtype=torch.float32, device=x.device)
    q_col = torch.empty((M, N), dtype=dtype, device=x.device)
    s_col = torch.empty((ceil_div(M, block_size), N), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.call(
            "ptb_quant_fp8_block1d_dual", ptr(x), dtype_code(x.dtype), M, N, ptr(q_row), ptr(s_row),
            ptr(q_col), ptr(s_col), dtype_code(dtype), stream_of(x),
        )
    return q_row, s_row, q_col, s_col


def quant_fp8_blockwise_for_weight_impl(w: torch.Tensor, dtype: torch.dtype, block_size: int = 128):
    """quantization_impl.py:295-350: 2-D or 3-D weight, one scale per 128x128 tile."""
    assert w.dim() in (2, 3)
    assert block_size == 128, "Only block_size 128 is supported"
    _check_in(w)
    if not w.is_contiguous():
        w = w.contiguous()
    if w.dim() == 2:
        B, (M, N) = 1, w.shape
        sshape = (ceil_div(M, block_size), ceil_div(N, block_size))
    else:
        B, M, N = w.shape
        sshape = (B, ceil_div(M, block_size), ceil_div(N, block_size))
    q = torch.empty(w.shape, dtype=dtype, device=w.device)
    s = torch.empty(sshape, dtype=torch.float32, device=w.device)
    with torch.cuda.device(w.device):
        _lib.call(
            "ptb_quant_fp8_block2d", ptr(w), dtype_code(w.dtype), B, M, N, ptr(q), dtype_code(dtype), ptr(s),
            stream_of(w),
        )
    return q, s


def quant_fp8_blockwise_segment_m_row_col_impl(
    x: torch.Tensor,
    dtype: torch.dtype,
    block_size: int,
    group_lens: torch.Tensor,
    group_offs: torch.Tensor,
    gemm_other_dim: int | None = None,
):
    """quantization_impl.py:379-464.  Returns (x_fp8_row [M,N], x_fp8_col_padded [M+128G,N],
    x_scales_row [N/128, M], x_scales_col_padded [(M+128G)/128, N], var_k_group_lens [G],
    var_k_group_offs [G+1])."""
    assert x.is_contiguous() and x.dim() == 2
    assert block_size == 128, "Only block_size 128 is supported"
    _check_in(x)
    require_cuda(group_lens, group_offs)
    assert group_lens.dtype == torch.int64 and group_offs.dtype == torch.int64
    M, N = x.shape
    G = group_lens.numel()
    m_pad = M + G * block_size
    dev = x.device
    q_row = torch.empty((M, N), dtype=dtype, device=dev)
    q_col = torch.empty((m_pad, N), dtype=dtype, device=dev)
    s_row = torch.empty((ceil_div(N, block_size), M), dtype=torch.float32, device=dev)
    s_col = torch.empty((ceil_div(m_pad, block_size), N), dtype=torch.float32, device=dev)
    vk_lens = torch.empty(G, dtype=torch.int64, device=dev)
    vk_offs = torch.empty(G + 1, dtype=torch.int64, device=dev)
    # workspace: per padded 128-row block, where its source rows start and end (written by the call)
    table = torch.empty((ceil_div(m_pad, block_size), 2), dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        _lib.call(
            "ptb_quant_fp8_segment_row_col", ptr(x), dtype_code(x.dtype), M, N, G,
            ptr(group_lens.contiguous()), ptr(group_offs.contiguous()), ptr(q_row), ptr(q_col), ptr(s_row),
            ptr(s_col), ptr(vk_lens), ptr(vk_offs), ptr(table), dtype_code(dtype), stream_of(x),
        )
    return q_row, q_col, s_row, s_col, vk_lens, vk_offs


# ---- dequantize ------------------------------------------------------------------------------------
def dequantize_fp8_tensorwise_impl(x: torch.Tensor, out_dtype: torch.dtype, scale_inv: torch.Tensor):
    require_cuda(x, scale_inv)
    xc = x.contiguous()
    out = torch.empty(xc.shape, dtype=out_dtype, device=x.device)
    with torch.cuda.device(x.device):
        _lib.call(
            "ptb_dequant_fp8_tensorwise", ptr(xc), dtype_code(xc.dtype), xc.numel(),
            ptr(scale_inv.contiguous()), ptr(out), dtype_code(out_dtype), stream_of(x),
        )
    return out


def dequantize_fp8_rowwise_impl(x: torch.Tensor, out_dtype: torch.dtype, axis: int, scale_inv: torch.Tensor):
    assert x.is_contiguous(), "The x tensor must be contiguous."
    assert scale_inv.is_contiguous(), "The scale_inv tensor must be contiguous."
    require_cuda(x, scale_inv)
    nd = x.dim()
    ax = axis if axis >= 0 else nd + axis
    B, M, N = _bmn(tuple(x.shape), ax)
    out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    with torch.cuda.device(x.device):
        _lib.call(
            "ptb_dequant_fp8_rowwise", ptr(x), dtype_code(x.dtype), B, M, N, ptr(scale_inv), ptr(out),
            dtype_code(out_dtype), stream_of(x),
        )
    return out


def dequant_fp8_blockwise_impl(x_fp8, scale_inv, out_dtype, axis: int, block_size: int = 128):
    assert x_fp8.is_contiguous() and x_fp8.dim() == 2, "Input must be 2D and contiguous"
    assert axis in (-2, -1, 0, 1), f"axis must be 0 or 1 (or -1, -2), got {axis}"
    assert block_size == 128
    require_cuda(x_fp8, scale_inv)
    axis = axis % 2
    M, N = x_fp8.shape
    out = torch.empty((M, N), dtype=out_dtype, device=x_fp8.device)
    with torch.cuda.device(x_fp8.device):
        _lib.call(
            "ptb_dequant_fp8_block1d", ptr(x_fp8), dtype_code(x_fp8.dtype), M, N, axis,
            ptr(scale_inv.contiguous()), ptr(out), dtype_code(out_dtype), stream_of(x_fp8),
        )
    return out


def dequant_fp8_blockwise_for_weight_impl(w_fp8, scale_inv, out_dtype, block_size: int = 128):
    assert w_fp8.dim() in (2, 3)
    assert block_size == 128
    require_cuda(w_fp8, scale_inv)
    if not w_fp8.is_contiguous():
        w_fp8 = w_fp8.contiguous()
    if w_fp8.dim() == 2:
        B, (M, N) = 1, w_fp8.shape
    else:
        B, M, N = w_fp8.shape
    out = torch.empty(w_fp8.shape, dtype=out_dtype, device=w_fp8.device)
    with torch.cuda.device(w_fp8.device):
        _lib.call(
            "ptb_dequant_fp8_block2d", ptr(w_fp8), dtype_code(w_fp8.dtype), B, M, N,
            ptr(scale_inv.contiguous()), ptr(out), dtype_code(out_dtype), stream_of(w_fp8),
        )
    return out


def transpose_2d_fp8(x: torch.Tensor) -> torch.Tensor:
    """[..., M, N] -> [..., N, M] physical transpose of an FP8 payload (reference op transpose_2d)."""
    require_cuda(x)
    assert x.dim() >= 2 and x.element_size() == 1
    xc = x.contiguous()
    M, N = xc.shape[-2:]
    B = xc.numel() // max(M * N, 1) if M * N else 0
    out = torch.empty((*xc.shape[:-2], N, M), dtype=xc.dtype, device=xc.device)
    with torch.cuda.device(x.device):
        _lib.call(
            "ptb_transpose_2d_u8", ptr(xc), B, M, N, ptr(out), stream_of(x),
        )
    return out


def gather_rows(x: torch.Tensor, index: torch.Tensor) -> torch.Tensor:
    """``out[i] = x[index[i]]`` over the rows of a 2-D tensor whose rows are a multiple of 16 bytes (the row
    gather of the MoE token permutation, ``inp.index_select(0, sorted_indices)`` in
    primus_turbo/pytorch/ops/moe/permutation.py:281-369); an index outside ``[0, rows)`` gives a zero row."""
    require_cuda(x, index)
    assert x.dim() == 2 and index.dim() == 1 and index.dtype == torch.int64
    xc = x.contiguous()
    row_bytes = xc.shape[1] * xc.element_size()
    out = torch.empty((index.numel(), xc.shape[1]), dtype=xc.dtype, device=xc.device)
    with torch.cuda.device(x.device):
        _lib.call("ptb_gather_rows", ptr(xc), ptr(index.contiguous()), index.numel(), xc.shape[0], row_bytes, ptr(out),
                  stream_of(x))
    return out


# ---- MXFP8 (1x32 blocks, E8M0 scale bytes) -------------------------------------------------------------
MX_BLOCK = 32
MX_PAD = 128
E8M0 = torch.float8_e8m0fnu


def quantize_mxfp8_impl(
    x: torch.Tensor,
    out_dtype: torch.dtype,
    axis: int | None,
    block_size: int,
    with_trans: bool = False,
    use_2d_block: bool = False,
    use_2d_block_for_trans: bool | None = None,
):
    """x [M, N] or [G, M, N] (bf16 / fp16, contiguous).

    with_trans=False: ``axis`` picks the direction -- 2-D: 1 = blocks along a row -> (q [M, N_pad],
    scales [M, N_pad/32]); 0 = blocks along a column -> (q [N, M_pad], scales [N, M_pad/32], i.e. the
    TRANSPOSED copy); 3-D: axis 2 / 1 likewise per group.  with_trans=True returns both directions
    from one pass.  Scales have dtype float8_e8m0fnu.  Padded extents are multiples of 128.
    (primus_turbo/pytorch/kernels/quantization/quantization_impl.py:489-543,
    csrc/pytorch/quantization/quantization.cpp:736-966 in the reference.)
    """
    require_cuda(x)
    assert block_size == MX_BLOCK, f"The block size must be {MX_BLOCK} for MXFP8 quantization"
    assert x.dtype in (torch.bfloat16, torch.float16), "Input must be BFloat16 or Half"
    assert x.is_contiguous(), "Input must be contiguous"
    assert x.dim() in (2, 3), f"The input tensor must be 2D or 3D but got {x.dim()}D."
    batched = x.dim() == 3
    G = x.shape[0] if batched else 1
    M, N = x.shape[-2], x.shape[-1]
    assert N % MX_BLOCK == 0, f"N must be divisible by {MX_BLOCK}"
    if with_trans:
        assert axis is None, "The axis must be None when with_trans is True."
        want_row = want_col = True
        col_2d = use_2d_block if use_2d_block_for_trans is None else use_2d_block_for_trans
        row_2d = use_2d_block
    else:
        lo = 1 if batched else 0
        assert axis in (lo, lo + 1), f"The axis must be {lo} or {lo + 1} when with_trans is False."
        want_row, want_col = axis == lo + 1, axis == lo
        row_2d = col_2d = use_2d_block
    M_pad, N_pad = ceil_div(M, MX_PAD) * MX_PAD, ceil_div(N, MX_PAD) * MX_PAD
    lead = (G,) if batched else ()
    dev = x.device
    q_row = s_row = q_col = s_col = None
    if want_row:
        q_row = torch.empty(lead + (M, N_pad), dtype=out_dtype, device=dev)
        s_row = torch.empty(lead + (M, N_pad // MX_BLOCK), dtype=torch.uint8, device=dev)
    if want_col:
        q_col = torch.empty(lead + (N, M_pad), dtype=out_dtype, device=dev)
        s_col = torch.empty(lead + (N, M_pad // MX_BLOCK), dtype=torch.uint8, device=dev)
    if G * M * N > 0:
        with torch.cuda.device(dev):
            _lib.call(
                "ptb_quant_mxfp8", ptr(x), dtype_code(x.dtype), G, M, N, ptr(q_row), ptr(s_row), ptr(q_col), ptr(s_col),
                int(row_2d), int(col_2d), dtype_code(out_dtype), stream_of(x),
            )
    outs = []
    if want_row:
        outs += [q_row, s_row.view(E8M0)]
    if want_col:
        outs += [q_col, s_col.view(E8M0)]
    return tuple(outs)


def dequantize_mxfp8_impl(x: torch.Tensor, out_dtype: torch.dtype, axis: int, block_size: int, scale_inv: torch.Tensor):
    """2-D: axis 1 -> [M, N_pad]; axis 0 (x is the transposed copy [N, M_pad]) -> [M_pad, N].  3-D: axis 2 ->
    [G, M, N_pad]; axis 1 -> [G, M_pad, N].  (csrc/pytorch/quantization/quantization.cpp:283-358 in the reference.)"""
    require_cuda(x, scale_inv)
    assert block_size == MX_BLOCK, f"The block size must be {MX_BLOCK} for MXFP8 quantization"
    assert x.is_contiguous() and scale_inv.is_contiguous()
    assert x.dim() in (2, 3) and scale_inv.dim() == x.dim(), "scale_inv rank must match input"
    assert scale_inv.dtype in (E8M0, torch.uint8), "scale_inv must be Float8_e8m0fnu / uint8 tensor"
    lo = 1 if x.dim() == 3 else 0
    assert axis in (lo, lo + 1)
    rowwise = axis == lo + 1
    R, C = x.shape[-2], x.shape[-1]
    assert C % MX_BLOCK == 0, "The last dimension must be divisible by block_size"
    G = x.shape[0] if x.dim() == 3 else 1
    lead = (G,) if x.dim() == 3 else ()
    out = torch.empty(lead + ((R, C) if rowwise else (C, R)), dtype=out_dtype, device=x.device)
    s8 = scale_inv.view(torch.uint8)
    with torch.cuda.device(x.device):
        for g in range(G):
            xg, sg, og = (x[g], s8[g], out[g]) if x.dim() == 3 else (x, s8, out)
            if R * C > 0:
                _lib.call(
                    "ptb_dequant_mxfp8", ptr(xg), dtype_code(x.dtype), R, C, ptr(sg), 0 if rowwise else 1, ptr(og),
                    dtype_code(out_dtype), stream_of(x),
                )
    return out


def grouped_quantize_mxfp8_impl(
    x: torch.Tensor,
    out_dtype: torch.dtype,
    block_size: int,
    group_lens: torch.Tensor,
    group_offs: torch.Tensor,
    use_2d_block: bool = False,
    use_2d_block_for_trans: bool = False,
    row_align: int = 32,
):
    """x [M, N] whose rows form ``len(group_lens)`` groups -> (q_row, s_row, q_col_t, s_col, row_lens_padded,
    row_offs_padded, col_lens_padded, col_offs_padded): every group quantised on its own, padded to
    ``row_align`` rows in the row copy (32: the reference's layout; 1: no padding, what this build's grouped
    GEMM reads) and to 128 rows in the transposed column copy.  Nothing synchronises with the host; the
    outputs are allocated for the worst case.  Rows of the row copy that hold no group row are unspecified
    (the reference leaves them unwritten as well).
    (primus_turbo/pytorch/kernels/quantization/quantization_impl.py:546-599,
    csrc/pytorch/quantization/quantization.cpp:1075-1195 in the reference.)"""
    require_cuda(x, group_lens, group_offs)
    assert block_size == MX_BLOCK, f"The block size must be {MX_BLOCK} for MXFP8 quantization"
    assert x.dtype in (torch.bfloat16, torch.float16), "Input must be BFloat16 or Half"
    assert x.dim() == 2 and x.is_contiguous(), "Input must be 2D and contiguous"
    assert group_lens.dtype == torch.int64 and group_offs.dtype == torch.int64, "group_lens / group_offs must be int64"
    assert group_offs.numel() == group_lens.numel() + 1 and group_lens.numel() >= 1
    M, N = x.shape
    G = group_lens.numel()
    assert N % MX_BLOCK == 0, f"N must be divisible by {MX_BLOCK}"
    N_pad = ceil_div(N, MX_PAD) * MX_PAD
    M_row = ceil_div(M + G * row_align, row_align) * row_align if row_align > 1 else M
    M_col = ceil_div(M + G * MX_PAD, MX_PAD) * MX_PAD
    dev = x.device
    q_row = torch.empty((M_row, N_pad), dtype=out_dtype, device=dev)
    s_row = torch.empty((M_row, N_pad // MX_BLOCK), dtype=torch.uint8, device=dev)
    q_col = torch.empty((N, M_col), dtype=out_dtype, device=dev)
    s_col = torch.empty((N, M_col // MX_BLOCK), dtype=torch.uint8, device=dev)
    layout = torch.empty(4 * G + 2, dtype=torch.int64, device=dev)
    row_lens, row_offs, col_lens, col_offs = layout[:G], layout[G : 2 * G + 1], layout[2 * G + 1 : 3 * G + 1], layout[3 * G + 1 :]
    table = torch.empty(M_col // MX_PAD * 4, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        _lib.call(
            "ptb_quant_mxfp8_grouped", ptr(x), dtype_code(x.dtype), M, N, ptr(group_offs.contiguous()), G, row_align, ptr(q_row),
            ptr(s_row), ptr(q_col), ptr(s_col), ptr(row_lens), ptr(row_offs), ptr(col_lens), ptr(col_offs), ptr(table),
            int(use_2d_block), int(use_2d_block_for_trans), dtype_code(out_dtype), stream_of(x),
        )
    return q_row, s_row.view(E8M0), q_col, s_col.view(E8M0), row_lens, row_offs, col_lens, col_offs


def packed_row_index(group_offs: torch.Tensor, group_offs_padded: torch.Tensor, total_rows: int) -> torch.Tensor:
    """For each of ``total_rows`` packed rows (group g holds rows [offs[g], offs[g+1])) its row in a layout where
    group g starts at ``offs_padded[g]``: ``offs_padded[g] + (r - offs[g])``.  Computed on the device, no
    synchronisation; rows at or past ``offs[G]`` follow the last group (they stay inside the padded layout,
    whose allocation bounds every group's padding)."""
    G = group_offs.numel() - 1
    r = torch.arange(total_rows, device=group_offs.device, dtype=torch.int64)
    g = torch.searchsorted(group_offs[1:].contiguous(), r, right=True).clamp_(max=G - 1)
    return r + (group_offs_padded[:-1] - group_offs[:-1])[g]


def grouped_dequantize_mxfp8_impl(
    x: torch.Tensor,
    out_dtype: torch.dtype,
    axis: int,
    block_size: int,
    scale_inv: torch.Tensor,
    group_offs: torch.Tensor,
    group_offs_padded: torch.Tensor,
    total_M: int | None = None,
) -> torch.Tensor:
    """Back from a grouped MXFP8 payload (axis 1: the row copy, groups padded to 32 rows; axis 0: the transposed
    column copy, groups padded to 128) to the packed rows ``[total_M, N_pad]`` / ``[total_M, N]``: the padded
    layout is dequantised as a whole and the rows that exist are gathered out of it.  ``total_M`` defaults to
    ``group_offs[-1]`` (one synchronisation).
    (primus_turbo/pytorch/kernels/quantization/quantization_impl.py:727-754 in the reference.)"""
    assert x.dim() == 2 and scale_inv.dim() == 2, "The x and scale_inv must be 2D tensors."
    assert axis in (0, 1), "The axis must be 0 or 1."
    assert group_offs.dtype == torch.int64 and group_offs_padded.dtype == torch.int64
    assert group_offs.numel() == group_offs_padded.numel() >= 2
    full = dequantize_mxfp8_impl(x, out_dtype, axis, block_size, scale_inv)
    if total_M is None:
        total_M = int(group_offs[-1])
    return full.index_select(0, packed_row_index(group_offs, group_offs_padded, total_M))

