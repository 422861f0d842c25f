"""Thin torch layer over the GEMM entry points of the C ABI.

Signatures follow the reference custom ops ``primus_turbo::gemm_fp8_impl``
(primus_turbo/pytorch/kernels/gemm/gemm_fp8_impl.py:438-467), ``grouped_gemm_fp8_impl`` and
``grouped_gemm_fp8_variable_k_impl``
(primus_turbo/pytorch/kernels/grouped_gemm/grouped_gemm_fp8_impl.py:817-901), minus the backend
selector: there is one implementation.  Transposed operands are consumed in place (the tensor cores
read MN-major tiles), so no layout ever needs a physical transpose.
"""

from __future__ import annotations

import torch

from primus_turbo_b200 import _lib
from primus_turbo_b200._lib import (
    PTB_BLOCKWISE,
    PTB_ROWWISE,
    PTB_TENSORWISE,
    dtype_code,
    ptr,
    require_cuda,
    stream_of,
)


def get_gemm_logical_shape(a, b, trans_a: bool, trans_b: bool):
    m, k = (a.shape[1], a.shape[0]) if trans_a else (a.shape[0], a.shape[1])
    kb, n = (b.shape[1], b.shape[0]) if trans_b else (b.shape[0], b.shape[1])
    assert k == kb, f"contraction sizes differ: {k} vs {kb}"
    return m, n, k


def _as_rows(t: torch.Tensor) -> torch.Tensor:
    """2-D FP8 operand with unit inner stride and a row pitch that TMA accepts."""
    if t.stride(-1) != 1:
        t = t.contiguous()
    return t


def _f32(t: torch.Tensor) -> torch.Tensor:
    return t if t.dtype == torch.float32 else t.to(torch.float32)


def gemm_fp8_impl(
    a: torch.Tensor,
    a_scale_inv: torch.Tensor,
    trans_a: bool,
    b: torch.Tensor,
    b_scale_inv: torch.Tensor,
    trans_b: bool,
    out_dtype: torch.dtype,
    trans_c: bool,
    granularity: int,
    default_backend: int | None = None,  # accepted and ignored: single implementation
    num_sms: int = 0,
) -> torch.Tensor:
    require_cuda(a, b, a_scale_inv, b_scale_inv)
    assert a.dim() == 2 and b.dim() == 2, "Only 2D tensors are supported"
    if trans_c:
        if granularity == PTB_BLOCKWISE and not (trans_a and not trans_b):
            # 1x128 / 128x128 scale roles cannot swap sides; materialise the transpose instead
            return gemm_fp8_impl(
                a, a_scale_inv, trans_a, b, b_scale_inv, trans_b, out_dtype, False, granularity, num_sms=num_sms
            ).t().contiguous()
        # C^T = op(B)^T . op(A)^T : swap the operands
        return gemm_fp8_impl(
            b, b_scale_inv, not trans_b, a, a_scale_inv, not trans_a, out_dtype, False, granularity, num_sms=num_sms
        )
    a, b = _as_rows(a), _as_rows(b)
    m, n, k = get_gemm_logical_shape(a, b, trans_a, trans_b)
    out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    a_s, b_s = _f32(a_scale_inv), _f32(b_scale_inv)
    b_block_2d = 1
    if granularity == PTB_TENSORWISE:
        assert a_s.numel() == 1 and b_s.numel() == 1
        asm = ask = bsn = bsk = 0
    elif granularity == PTB_ROWWISE:
        a_s, b_s = a_s.reshape(-1).contiguous(), b_s.reshape(-1).contiguous()
        assert a_s.numel() == m and b_s.numel() == n, "rowwise scales must be vectors over the output rows / columns"
        asm, ask, bsn, bsk = 1, 0, 1, 0
    elif granularity == PTB_BLOCKWISE:
        assert a_s.dim() == 2 and b_s.dim() == 2
        if not trans_a:
            asm, ask = a_s.stride(0), a_s.stride(1)  # [M, K/128]
            if trans_b:
                bsn, bsk = b_s.stride(0), b_s.stride(1)  # [N/128, K/128]
            else:
                bsn, bsk = b_s.stride(1), b_s.stride(0)  # [K/128, N/128]
        else:
            if trans_b:
                raise ValueError(f"Unsupported layout for blockwise FP8: trans_a={trans_a}, trans_b={trans_b}")
            asm, ask = a_s.stride(1), a_s.stride(0)  # [K/128, M]
            bsn, bsk = b_s.stride(1), b_s.stride(0)  # [K/128, N]
            b_block_2d = 0
    else:
        raise ValueError(f"Unsupported granularity {granularity}")
    with torch.cuda.device(a.device):
        _lib.call(
            "ptb_gemm_fp8", ptr(a), dtype_code(a.dtype), int(trans_a), a.stride(0), ptr(b),
            dtype_code(b.dtype), int(trans_b), b.stride(0), ptr(out), dtype_code(out_dtype), out.stride(0), m,
            n, k, granularity, ptr(a_s), asm, ask, ptr(b_s), bsn, bsk, b_block_2d, num_sms, stream_of(a),
        )
    return out


def gemm_mxfp8_impl(
    a: torch.Tensor, a_scale_inv: torch.Tensor, b: torch.Tensor, b_scale_inv: torch.Tensor, out_dtype: torch.dtype,
    num_sms: int = 0,
) -> torch.Tensor:
    """a [M, K_pad] . b [N, K_pad]^T with E8M0 scale bytes [rows, K_pad/32] applied by the block-scaled
    tensor-core instruction.  The reference reaches this as gemm_fp8_impl(..., granularity=MX_BLOCKWISE)
    with trans_a=False, trans_b=True (primus_turbo/pytorch/ops/gemm_fp8.py:582-640)."""
    require_cuda(a, b, a_scale_inv, b_scale_inv)
    assert a.dim() == 2 and b.dim() == 2 and a.shape[1] == b.shape[1], "MX GEMM takes [M, K] and [N, K]"
    a, b = _as_rows(a), _as_rows(b)
    a_s, b_s = a_scale_inv.view(torch.uint8), b_scale_inv.view(torch.uint8)
    assert a_s.stride(-1) == 1 and b_s.stride(-1) == 1
    m, k = a.shape
    n = b.shape[0]
    out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    with torch.cuda.device(a.device):
        _lib.call(
            "ptb_gemm_mxfp8", ptr(a), dtype_code(a.dtype), a.stride(0), ptr(a_s), a_s.stride(0), ptr(b),
            dtype_code(b.dtype), b.stride(0), ptr(b_s), b_s.stride(0), ptr(out), dtype_code(out_dtype), out.stride(0),
            m, n, k, num_sms, stream_of(a),
        )
    return out


def grouped_gemm_mxfp8_impl(
    a: torch.Tensor, a_scale_inv: torch.Tensor, b: torch.Tensor, b_scale_inv: torch.Tensor, group_offs: torch.Tensor,
    out_dtype: torch.dtype, num_sms: int = 0,
) -> torch.Tensor:
    """out[rows of group g] = a[rows of group g] . b[g]^T: a [M, K_pad] with scale bytes [M, K_pad/32] (rows at
    their unpadded positions), b [G, N, K_pad] with [G, N, K_pad/32]; rows at or past group_offs[G] are zero."""
    require_cuda(a, b, a_scale_inv, b_scale_inv, group_offs)
    assert a.dim() == 2 and b.dim() == 3 and a.shape[1] == b.shape[2]
    a, b = _as_rows(a), b.contiguous()
    a_s, b_s = a_scale_inv.view(torch.uint8), b_scale_inv.view(torch.uint8).contiguous()
    m, k = a.shape
    g, n = b.shape[0], b.shape[1]
    out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    with torch.cuda.device(a.device):
        _lib.call(
            "ptb_grouped_gemm_mxfp8", ptr(a), dtype_code(a.dtype), a.stride(0), ptr(a_s), a_s.stride(0), ptr(b),
            dtype_code(b.dtype), ptr(b_s), ptr(out), dtype_code(out_dtype), out.stride(0), ptr(group_offs), g, m, n, k,
            num_sms, stream_of(a),
        )
    return out


def grouped_gemm_mxfp8_variable_k_impl(
    lhs: torch.Tensor, lhs_scale_inv: torch.Tensor, rhs: torch.Tensor, rhs_scale_inv: torch.Tensor,
    group_offs_padded: torch.Tensor, out_dtype: torch.dtype, num_sms: int = 0,
) -> torch.Tensor:
    """out[g] = lhs[:, cols of g] . rhs[:, cols of g]^T for the transposed column copies lhs [OUT_M, rows_padded],
    rhs [OUT_N, rows_padded] of the grouped quantiser; -> [G, OUT_M, OUT_N]."""
    require_cuda(lhs, rhs, lhs_scale_inv, rhs_scale_inv, group_offs_padded)
    assert lhs.dim() == 2 and rhs.dim() == 2 and lhs.shape[1] == rhs.shape[1]
    lhs, rhs = _as_rows(lhs), _as_rows(rhs)
    l_s, r_s = lhs_scale_inv.view(torch.uint8), rhs_scale_inv.view(torch.uint8)
    g = group_offs_padded.numel() - 1
    out = torch.empty((g, lhs.shape[0], rhs.shape[0]), dtype=out_dtype, device=lhs.device)
    with torch.cuda.device(lhs.device):
        _lib.call(
            "ptb_grouped_gemm_mxfp8_variable_k", ptr(lhs), dtype_code(lhs.dtype), lhs.stride(0), ptr(l_s), l_s.stride(0),
            ptr(rhs), dtype_code(rhs.dtype), rhs.stride(0), ptr(r_s), r_s.stride(0), ptr(out), dtype_code(out_dtype),
            ptr(group_offs_padded), g, lhs.shape[1], lhs.shape[0], rhs.shape[0], num_sms, stream_of(lhs),
        )
    return out


def group_offs_from_lens(group_lens: torch.Tensor) -> torch.Tensor:
    """Exclusive prefix sum on the device (grouped_gemm_utils.py:28-34)."""
    assert group_lens.is_cuda, "group_lens must be on CUDA"
    assert group_lens.dtype == torch.int64
    gl = group_lens.contiguous()
    offs = torch.empty(gl.numel() + 1, dtype=torch.int64, device=gl.device)
    with torch.cuda.device(gl.device):
        _lib.call(
            "ptb_group_offs", ptr(gl), gl.numel(), ptr(offs), stream_of(gl),
        )
    return offs


def grouped_gemm_fp8_impl(
    a: torch.Tensor,
    b: torch.Tensor,
    a_scales: torch.Tensor,
    b_scales: torch.Tensor,
    group_lens: torch.Tensor,
    group_offs: torch.Tensor,
    trans_a: bool,
    trans_b: bool,
    out_dtype: torch.dtype,
    granularity: int,
    num_cu: int | None = None,
    default_backend: int | None = None,
) -> torch.Tensor:
    """out[offs[g]:offs[g+1]] = a[offs[g]:offs[g+1]] . op(b[g]); rows past offs[G] are zeroed."""
    assert not trans_a, "Only trans_a=False is supported."
    require_cuda(a, b, a_scales, b_scales, group_offs)
    assert a.dim() == 2 and b.dim() == 3
    a = _as_rows(a)
    b = b.contiguous()
    G = b.shape[0]
    m_total, k = a.shape
    n = b.shape[1] if trans_b else b.shape[2]
    assert (b.shape[2] if trans_b else b.shape[1]) == k
    assert group_offs.numel() == G + 1 and group_offs.dtype == torch.int64
    out = torch.empty((m_total, n), dtype=out_dtype, device=a.device)
    a_s, b_s = _f32(a_scales), _f32(b_scales)
    if granularity == PTB_TENSORWISE:
        asm = ask = bsg = bsn = bsk = 0
    elif granularity == PTB_ROWWISE:
        a_s, b_s = a_s.reshape(-1).contiguous(), b_s.reshape(G, -1).contiguous()
        assert a_s.numel() == m_total and b_s.shape[1] == n
        asm, ask, bsg, bsn, bsk = 1, 0, n, 1, 0
    elif granularity == PTB_BLOCKWISE:
        assert a_s.dim() == 2 and b_s.dim() == 3
        asm, ask = a_s.stride(1), a_s.stride(0)  # [K/128, M_total]
        bsg = b_s.stride(0)
        bsn, bsk = (b_s.stride(1), b_s.stride(2)) if trans_b else (b_s.stride(2), b_s.stride(1))
    else:
        raise ValueError(f"Unsupported granularity {granularity}")
    with torch.cuda.device(a.device):
        _lib.call(
            "ptb_grouped_gemm_fp8", ptr(a), dtype_code(a.dtype), a.stride(0), ptr(b), dtype_code(b.dtype),
            int(trans_b), ptr(out), dtype_code(out_dtype), out.stride(0), ptr(group_offs.contiguous()), G,
            m_total, n, k, granularity, ptr(a_s), asm, ask, ptr(b_s), bsg, bsn, bsk, int(num_cu or 0),
            stream_of(a),
        )
    return out


def grouped_gemm_fp8_variable_k_impl(
    a: torch.Tensor,
    b: torch.Tensor,
    a_scales: torch.Tensor,
    b_scales: torch.Tensor,
    group_lens: torch.Tensor,
    group_offs: torch.Tensor,
    trans_a: bool,
    trans_b: bool,
    trans_c: bool,
    out_dtype: torch.dtype,
    granularity: int,
    num_cu: int | None = None,
    default_backend: int | None = None,
) -> torch.Tensor:
    """C[g] = a_g^T . b_g over rows [offs[g], offs[g+1]); trans_c swaps the operands -> b_g^T . a_g."""
    assert trans_a and not trans_b, "Only trans_a=True and trans_b=False are supported."
    require_cuda(a, b, a_scales, b_scales, group_offs)
    lhs, rhs, lhs_s, rhs_s = (b, a, b_scales, a_scales) if trans_c else (a, b, a_scales, b_scales)
    lhs, rhs = _as_rows(lhs), _as_rows(rhs)
    assert lhs.dim() == 2 and rhs.dim() == 2 and lhs.shape[0] == rhs.shape[0]
    G = group_offs.numel() - 1
    rows, out_m = lhs.shape
    out_n = rhs.shape[1]
    out = torch.empty((G, out_m, out_n), dtype=out_dtype, device=lhs.device)
    lhs_s, rhs_s = _f32(lhs_s).contiguous(), _f32(rhs_s).contiguous()
    if granularity == PTB_ROWWISE:
        assert lhs_s.numel() == out_m and rhs_s.numel() == out_n, "rowwise scales must span the output rows / columns"
    elif granularity == PTB_TENSORWISE:
        assert lhs_s.numel() == 1 and rhs_s.numel() == 1
    with torch.cuda.device(lhs.device):
        _lib.call(
            "ptb_grouped_gemm_fp8_variable_k", ptr(lhs), dtype_code(lhs.dtype), lhs.stride(0), ptr(rhs),
            dtype_code(rhs.dtype), rhs.stride(0), ptr(out), dtype_code(out_dtype),
            ptr(group_offs.contiguous()), G, rows, out_m, out_n, granularity, ptr(lhs_s), ptr(rhs_s),
            int(num_cu or 0), stream_of(lhs),
        )
    return out


__all__ = [
    "gemm_fp8_impl",
    "grouped_gemm_fp8_impl",
    "grouped_gemm_fp8_variable_k_impl",
    "group_offs_from_lens",
    "get_gemm_logical_shape",
]
