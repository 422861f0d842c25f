"""``swiglu_with_probs``: SwiGLU of a fused gate+up projection scaled by each row's routing probability,
with autograd (primus_turbo/pytorch/ops/activation.py:23-83 in the reference; kernels
primus_turbo/triton/activation/swiglu_kernel.py).

``x`` is ``[..., 2H]``: the first half goes through SiLU, the second half multiplies it; ``probs`` is fp32
with one value per row; ``row_mask`` (int64, optional) zeroes the rows it marks 0.

``swiglu_with_probs_quant_segment`` is the same activation fused into the grouped activation quantiser:
it returns what ``quant_fp8_blockwise_segment_m_row_col`` would return for the activation, without the
activation ever being written (byte-identical to running the two steps one after the other).
"""

from __future__ import annotations

from typing import Optional

import torch

from primus_turbo_b200 import _lib
from primus_turbo_b200._lib import dtype_code, ptr, require_cuda, stream_of

__all__ = ["swiglu_with_probs", "swiglu_with_probs_quant_segment"]


class _SwiGLUWithProbs(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, probs, row_mask):
        x_shape, p_shape = x.size(), probs.size()
        x2 = x.reshape(-1, x.size(-1)).contiguous()
        p1 = probs.reshape(-1).contiguous()
        assert x2.size(0) == p1.size(0), "first dimension of x and probs must be the same"
        assert p1.dtype == torch.float32, "probs must be float32"
        require_cuda(x2, p1)
        if row_mask is not None:
            assert row_mask.is_cuda, "row_mask must be a CUDA tensor"
            assert row_mask.ndim == 1 and x2.size(0) == row_mask.size(0), "row_mask must be 1D with one entry per row"
            assert row_mask.dtype == torch.int64, "The dtype of row_mask must be torch.int64."
            row_mask = row_mask.contiguous()
        rows, h2 = x2.shape
        out = torch.empty((rows, h2 // 2), dtype=x2.dtype, device=x2.device)
        with torch.cuda.device(x2.device):
            _lib.call("ptb_swiglu_probs_fwd", ptr(x2), dtype_code(x2.dtype), ptr(p1), ptr(row_mask), rows, h2 // 2, ptr(out),
                      stream_of(x2))
        ctx.save_for_backward(x2, p1, row_mask)
        ctx.x_shape, ctx.p_shape = x_shape, p_shape
        return out

    @staticmethod
    def backward(ctx, grad_output):
        assert grad_output.ndim == 2
        x2, p1, row_mask = ctx.saved_tensors
        g = grad_output.contiguous()
        rows, h2 = x2.shape
        grad_x = torch.empty_like(x2)
        grad_p = torch.empty_like(p1)
        with torch.cuda.device(x2.device):
            _lib.call("ptb_swiglu_probs_bwd", ptr(g), ptr(x2), dtype_code(x2.dtype), ptr(p1), ptr(row_mask), rows, h2 // 2,
                      ptr(grad_x), ptr(grad_p), stream_of(x2))
        return grad_x.view(ctx.x_shape), grad_p.view(ctx.p_shape), None


def swiglu_with_probs(x: torch.Tensor, probs: torch.Tensor, row_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    return _SwiGLUWithProbs.apply(x, probs, row_mask)


def swiglu_with_probs_quant_segment(x: torch.Tensor, probs: torch.Tensor, dtype: torch.dtype, group_lens: torch.Tensor,
                                    group_offs: torch.Tensor, block_size: int = 128):
    """SwiGLU-with-probs of ``x`` [M, 2N] quantised for the grouped blockwise GEMM in one pass.  Returns
    ``(q_row [M,N], q_col_padded [M+128G,N], s_row [N/128,M], s_col_padded [(M+128G)/128,N], var_k_group_lens [G],
    var_k_group_offs [G+1])``, the tuple of ``quant_fp8_blockwise_segment_m_row_col_impl`` on the activation."""
    assert block_size == 128, "Only block_size 128 is supported"
    assert x.dim() == 2 and x.is_contiguous() and x.shape[1] % 2 == 0
    assert probs.dtype == torch.float32 and probs.numel() == x.shape[0]
    require_cuda(x, probs, group_lens, group_offs)
    M, N = x.shape[0], x.shape[1] // 2
    G = group_lens.numel()
    m_pad = M + G * block_size
    dev = x.device
    cd = lambda a, b: (a + b - 1) // b  # noqa: E731
    q_row = torch.empty((M, N), dtype=dtype, device=dev)
    q_col = torch.empty((m_pad, N), dtype=dtype, device=dev)
    s_row = torch.empty((cd(N, block_size), M), dtype=torch.float32, device=dev)
    s_col = torch.empty((cd(m_pad, block_size), N), dtype=torch.float32, device=dev)
    vk_lens = torch.empty(G, dtype=torch.int64, device=dev)
    vk_offs = torch.empty(G + 1, dtype=torch.int64, device=dev)
    table = torch.empty((cd(m_pad, block_size), 2), dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        _lib.call("ptb_swiglu_quant_fp8_segment_row_col", ptr(x), dtype_code(x.dtype), ptr(probs.contiguous()), M, N, G,
                  ptr(group_offs.contiguous()), ptr(q_row), ptr(q_col), ptr(s_row), ptr(s_col), ptr(vk_lens), ptr(vk_offs),
                  ptr(table), dtype_code(dtype), stream_of(x))
    return q_row, q_col, s_row, s_col, vk_lens, vk_offs
