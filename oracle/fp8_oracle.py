"""CPU oracle for the FP8 quantize / GEMM / grouped-GEMM path.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain fp32 torch on the CPU, the arithmetic of the reference kernels.
It is the checker for the CUDA path: only the test-suite, the smoke check and the CPU-baseline
leg of the benchmark may import it.  Nothing in the shipped package may call it.

PARITY UNPINNED at the bit level: the reference holds no golden vectors or known-answer files
for this path (its tests gate on tolerances / SNR only), and the reference itself (a ROCm
extension plus AMD Triton lowering) cannot execute on this hardware.  The byte-level behaviour
restated here is therefore pinned by the reference *kernel sources* cited on each function, and
cross-checked where possible against the reference's own torch test references
(tests/pytorch/ref/quantization_ref.py, tests/pytorch/ref/gemm_ref.py) through the committed
fixtures in tests/golden/.

All arithmetic: IEEE fp32, round-to-nearest-even division and multiplication, cast to FP8 by
round-to-nearest-even of an already clamped value (so the saturation mode of the cast is moot).
"""

from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch

# csrc/pytorch/quantization/quantization.cpp:21-35 (fp8 max table, OCP formats)
FP8_MAX = {torch.float8_e4m3fn: 448.0, torch.float8_e5m2: 57344.0}

EPS_TENSOR_ROW = 1e-12  # csrc/include/primus_turbo/quantization.h:15, quantization_rowwise.cu:71
EPS_BLOCK = 1e-4  # primus_turbo/triton/quantization/quant_blockwise.py:14, quantization_blockwise.cu:140,179,300


def _f32(v: float) -> torch.Tensor:
    return torch.tensor(v, dtype=torch.float32)


def _scale_pair(amax: torch.Tensor, fmax: float, eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """scale = fmax / max(amax, eps); scale_inv = 1.0f / scale  (two fp32 divisions).

    csrc/include/primus_turbo/device/quant_utils.cuh:60-72; quant_blockwise.py:11-18,57.
    """
    amax = amax.to(torch.float32)
    amax = torch.maximum(amax, _f32(eps))
    scale = _f32(fmax) / amax
    scale_inv = _f32(1.0) / scale
    return scale, scale_inv


def _quant(xf: torch.Tensor, scale: torch.Tensor, fmax: float, dtype: torch.dtype) -> torch.Tensor:
    """q = cast(clamp(xf * scale, -fmax, fmax)); quant_utils.cuh:31-38."""
    v = xf * scale
    v = torch.clamp(v, -fmax, fmax)
    return v.to(dtype)


def cdiv(a: int, b: int) -> int:
    return (a + b - 1) // b


# ----------------------------------------------------------------------------------------------
# quantize
# ----------------------------------------------------------------------------------------------
def quant_tensorwise(x: torch.Tensor, dtype: torch.dtype):
    """csrc/pytorch/quantization/quantization.cpp:42-88. Returns (q, scale_inv[]) ."""
    fmax = FP8_MAX[dtype]
    xf = x.to(torch.float32)
    amax = xf.abs().amax() if xf.numel() else _f32(0.0)
    scale, scale_inv = _scale_pair(amax, fmax, EPS_TENSOR_ROW)
    return _quant(xf, scale, fmax, dtype), scale_inv.reshape(())


def quant_rowwise(x: torch.Tensor, dtype: torch.dtype, axis: int):
    """csrc/pytorch/quantization/quantization.cpp:108-206; quantization_rowwise.cu:57-135,186-235.

    One scale for all elements that share every index except `axis`; scale_inv keeps the input
    shape with shape[axis] = 1.
    """
    fmax = FP8_MAX[dtype]
    axis = axis if axis >= 0 else x.dim() + axis
    xf = x.to(torch.float32)
    amax = xf.abs().amax(dim=axis, keepdim=True)
    scale, scale_inv = _scale_pair(amax, fmax, EPS_TENSOR_ROW)
    return _quant(xf, scale, fmax, dtype), scale_inv


def _pad_to(xf: torch.Tensor, mult: int) -> torch.Tensor:
    M, N = xf.shape[-2:]
    Mp, Np = cdiv(M, mult) * mult, cdiv(N, mult) * mult
    if (Mp, Np) == (M, N):
        return xf
    out = xf.new_zeros(*xf.shape[:-2], Mp, Np)
    out[..., :M, :N] = xf
    return out


def quant_block1d(x: torch.Tensor, dtype: torch.dtype, axis: int, block: int = 128):
    """quant_blockwise.py:22-62.  axis=1: one scale per (row, 128-col block) -> [M, ceil(N/128)];
    axis=0: one scale per (128-row block, col) -> [ceil(M/128), N].  Out-of-range elements of a
    partial block contribute 0 to the amax."""
    assert x.dim() == 2
    axis = axis % 2
    fmax = FP8_MAX[dtype]
    M, N = x.shape
    xf = _pad_to(x.to(torch.float32), block)
    Mp, Np = xf.shape
    if axis == 1:
        t = xf.reshape(Mp, Np // block, block)
        amax = t.abs().amax(dim=2, keepdim=True)
        scale, scale_inv = _scale_pair(amax, fmax, EPS_BLOCK)
        q = _quant(t, scale, fmax, dtype).reshape(Mp, Np)[:M, :N].contiguous()
        s = scale_inv.reshape(Mp, Np // block)[:M].contiguous()
    else:
        t = xf.reshape(Mp // block, block, Np)
        amax = t.abs().amax(dim=1, keepdim=True)
        scale, scale_inv = _scale_pair(amax, fmax, EPS_BLOCK)
        q = _quant(t, scale, fmax, dtype).reshape(Mp, Np)[:M, :N].contiguous()
        s = scale_inv.reshape(Mp // block, Np)[:, :N].contiguous()
    return q, s


def quant_block1d_dual(x: torch.Tensor, dtype: torch.dtype, block: int = 128):
    """quant_blockwise.py:65-112: row-block copy and col-block copy (both [M,N], un-transposed)."""
    q_row, s_row = quant_block1d(x, dtype, 1, block)
    q_col, s_col = quant_block1d(x, dtype, 0, block)
    return q_row, s_row, q_col, s_col


def quant_block2d(w: torch.Tensor, dtype: torch.dtype, block: int = 128):
    """quantization_blockwise.cu:246-332 / quant_blockwise.py:118-156: one scale per 128x128 tile
    of [M,N] or [B,M,N]; scale_inv [B, ceil(M/128), ceil(N/128)] (no B for 2-D input)."""
    assert w.dim() in (2, 3)
    fmax = FP8_MAX[dtype]
    squeeze = w.dim() == 2
    w3 = w.unsqueeze(0) if squeeze else w
    B, M, N = w3.shape
    xf = _pad_to(w3.to(torch.float32), block)
    Mp, Np = xf.shape[-2:]
    t = xf.reshape(B, Mp // block, block, Np // block, block)
    amax = t.abs().amax(dim=(2, 4), keepdim=True)
    scale, scale_inv = _scale_pair(amax, fmax, EPS_BLOCK)
    q = _quant(t, scale, fmax, dtype).reshape(B, Mp, Np)[:, :M, :N].contiguous()
    s = scale_inv.reshape(B, Mp // block, Np // block).contiguous()
    if squeeze:
        q, s = q[0], s[0]
    return q, s


def group_offs_from_lens(group_lens: torch.Tensor) -> torch.Tensor:
    """csrc/kernels/grouped_gemm/ck_grouped_gemm.cu:109-127: exclusive prefix sum, int64 [G+1]."""
    out = torch.zeros(group_lens.numel() + 1, dtype=torch.int64)
    out[1:] = torch.cumsum(group_lens.to(torch.int64), 0)
    return out


def quant_segment_row_col(
    x: torch.Tensor, dtype: torch.dtype, block: int, group_lens: torch.Tensor, group_offs: torch.Tensor
):
    """quant_blockwise.py:237-327 / quantization_blockwise.cu:58-213.

    Returns (q_row [M,N], q_col_padded [M+G*128,N], s_row [ceil(N/128), M] (transposed order),
    s_col_padded [ceil((M+G*128)/128), N], var_k_lens [G], var_k_offs [G+1], written_row_mask [M],
    padded_rows_written).  Rows of q_row / columns of s_row at or beyond group_offs[G], and rows of
    the padded outputs at or beyond var_k_offs[G], are never written by the reference; the oracle
    leaves them zero and reports the written extents so the test can ignore them.
    """
    assert x.dim() == 2
    fmax = FP8_MAX[dtype]
    M, N = x.shape
    G = group_lens.numel()
    lens = group_lens.to(torch.int64)
    offs = group_offs.to(torch.int64)
    var_k_lens = ((lens + block - 1) // block) * block
    var_k_offs = group_offs_from_lens(var_k_lens)
    m_pad_max = M + G * block
    m_used = int(offs[G])
    # row part: independent of grouping
    q_row_full, s_row_full = quant_block1d(x, dtype, 1, block)  # [M,N], [M, nb]
    q_row = torch.zeros((M, N), dtype=dtype)
    q_row[:m_used] = q_row_full[:m_used]
    s_row = torch.zeros((cdiv(N, block), M), dtype=torch.float32)
    s_row[:, :m_used] = s_row_full[:m_used].t()
    # col part: group-relative 128-row blocks, zero padded
    q_col = torch.zeros((m_pad_max, N), dtype=dtype)
    s_col = torch.zeros((cdiv(m_pad_max, block), N), dtype=torch.float32)
    xf = x.to(torch.float32)
    for g in range(G):
        lo, hi = int(offs[g]), int(offs[g + 1])
        if hi == lo:
            continue
        plo, plen = int(var_k_offs[g]), int(var_k_lens[g])
        seg = torch.zeros((plen, N), dtype=torch.float32)
        seg[: hi - lo] = xf[lo:hi]
        qs, ss = quant_block1d(seg, dtype, 0, block)
        q_col[plo : plo + plen] = qs
        s_col[plo // block : (plo + plen) // block] = ss
    written_rows = torch.zeros(M, dtype=torch.bool)
    written_rows[:m_used] = True
    return q_row, q_col, s_row, s_col, var_k_lens, var_k_offs, written_rows, int(var_k_offs[G])


# ----------------------------------------------------------------------------------------------
# dequantize: out = cast(float(q) * scale_inv)
# quant_blockwise.py:162-234; quantization_tensorwise.cu:37-44; quantization_rowwise.cu:430-438
# ----------------------------------------------------------------------------------------------
def dequant_tensorwise(q, scale_inv, out_dtype=torch.float32):
    return (q.to(torch.float32) * scale_inv.to(torch.float32)).to(out_dtype)


def dequant_rowwise(q, scale_inv, out_dtype=torch.float32):
    return (q.to(torch.float32) * scale_inv.to(torch.float32)).to(out_dtype)


def dequant_block1d(q, scale_inv, axis: int, out_dtype=torch.float32, block: int = 128):
    axis = axis % 2
    M, N = q.shape
    qf = q.to(torch.float32)
    if axis == 1:
        s = scale_inv.repeat_interleave(block, dim=1)[:, :N]
    else:
        s = scale_inv.repeat_interleave(block, dim=0)[:M, :]
    return (qf * s).to(out_dtype)


def dequant_block2d(q, scale_inv, out_dtype=torch.float32, block: int = 128):
    M, N = q.shape[-2:]
    s = scale_inv.repeat_interleave(block, dim=-2).repeat_interleave(block, dim=-1)[..., :M, :N]
    return (q.to(torch.float32) * s).to(out_dtype)


# ----------------------------------------------------------------------------------------------
# GEMM oracles: dequantize-then-matmul in fp32 on identical quantized inputs
# (reference semantics: primus_turbo/triton/gemm/gemm_fp8_kernel.py:165-167,229-230 tensorwise,
#  :525-528 rowwise, :945-954 blockwise; tests/pytorch/ref/gemm_ref.py:13-24 per-group matmul)
# ----------------------------------------------------------------------------------------------
def _mm(a_mk: torch.Tensor, b_nk: torch.Tensor) -> torch.Tensor:
    return a_mk.to(torch.float32) @ b_nk.to(torch.float32).t()


def gemm_tensorwise(aq, a_s, bq, b_s, trans_a=False, trans_b=True, out_dtype=torch.bfloat16):
    """C = (Aq.Bq^T) * (sa*sb).  aq is [M,K] ([K,M] if trans_a); bq is [N,K] if trans_b else [K,N]."""
    A = aq.to(torch.float32).t() if trans_a else aq.to(torch.float32)
    Bnk = bq.to(torch.float32) if trans_b else bq.to(torch.float32).t()
    return ((A @ Bnk.t()) * (a_s.to(torch.float32) * b_s.to(torch.float32))).to(out_dtype)


def gemm_rowwise(aq, a_s, bq, b_s, trans_a=False, trans_b=True, out_dtype=torch.bfloat16):
    """C[m,n] = (sum_k Aq Bq) * sa[m] * sb[n]; a_s / b_s are the keep-dim scale tensors produced by
    quant_rowwise along the contraction axis of each operand."""
    A = dequant_rowwise(aq, a_s)
    B = dequant_rowwise(bq, b_s)
    A = A.t() if trans_a else A
    Bnk = B if trans_b else B.t()
    return (A @ Bnk.t()).to(out_dtype)


def gemm_blockwise_nt(aq, a_s, bq, b_s, out_dtype=torch.bfloat16):
    """NT: A[M,K] with 1x128 scales [M,K/128]; B[N,K] with 128x128 scales [N/128,K/128]."""
    return _mm(dequant_block1d(aq, a_s, 1), dequant_block2d(bq, b_s)).to(out_dtype)


def gemm_blockwise_nn(aq, a_s, bq, b_s, out_dtype=torch.bfloat16):
    """NN (dgrad): A[M,K] 1x128 scales [M,K/128]; B[K,N] with 128x128 scales [K/128,N/128]."""
    return (dequant_block1d(aq, a_s, 1) @ dequant_block2d(bq, b_s)).to(out_dtype)


def gemm_blockwise_tn(aq, a_s, bq, b_s, out_dtype=torch.bfloat16):
    """TN (wgrad): A[K,M] with 128x1 scales [K/128,M]; B[K,N] with 128x1 scales [K/128,N];
    C[M,N] = A^T.B."""
    return (dequant_block1d(aq, a_s, 0).t() @ dequant_block1d(bq, b_s, 0)).to(out_dtype)


def grouped_gemm_blockwise(aq, a_s_t, bq, b_s, group_offs, trans_b=True, out_dtype=torch.bfloat16):
    """out[offs[g]:offs[g+1]] = A_g . W_g^T (trans_b) or A_g . W_g.
    aq [M_total,K]; a_s_t [ceil(K/128), M_total] (transposed order); bq [G,N,K] or [G,K,N];
    b_s [G, ceil(dim1/128), ceil(dim2/128)].  Rows >= offs[G] are zero."""
    M_total, K = aq.shape
    G = bq.shape[0]
    N = bq.shape[1] if trans_b else bq.shape[2]
    A = dequant_block1d(aq, a_s_t.t().contiguous(), 1)
    out = torch.zeros((M_total, N), dtype=torch.float32)
    for g in range(G):
        lo, hi = int(group_offs[g]), int(group_offs[g + 1])
        if hi == lo:
            continue
        W = dequant_block2d(bq[g], b_s[g])
        out[lo:hi] = A[lo:hi] @ (W.t() if trans_b else W)
    return out.to(out_dtype)


def grouped_gemm_blockwise_variable_k(lhs_q, lhs_s, rhs_q, rhs_s, var_k_offs, out_dtype=torch.bfloat16):
    """C[g] = lhs[po[g]:po[g+1]]^T . rhs[po[g]:po[g+1]] over segment-padded rows with 128x1 scales
    ([rows/128, cols]); empty group -> zeros.  Output [G, OUT_M, OUT_N]."""
    G = var_k_offs.numel() - 1
    OUT_M, OUT_N = lhs_q.shape[1], rhs_q.shape[1]
    out = torch.zeros((G, OUT_M, OUT_N), dtype=torch.float32)
    for g in range(G):
        lo, hi = int(var_k_offs[g]), int(var_k_offs[g + 1])
        if hi == lo:
            continue
        L = dequant_block1d(lhs_q[lo:hi], lhs_s[lo // 128 : hi // 128], 0)
        R = dequant_block1d(rhs_q[lo:hi], rhs_s[lo // 128 : hi // 128], 0)
        out[g] = L.t() @ R
    return out.to(out_dtype)


def grouped_gemm_rowwise(aq, a_s, bq, b_s, group_offs, trans_b=True, out_dtype=torch.bfloat16):
    """Grouped rowwise / tensorwise forward: a_s broadcastable to [M_total,1]; b_s broadcastable to
    bq with the contraction axis kept as 1 (or a scalar)."""
    M_total = aq.shape[0]
    G = bq.shape[0]
    N = bq.shape[1] if trans_b else bq.shape[2]
    A = aq.to(torch.float32) * a_s.to(torch.float32).reshape(-1, 1) if a_s.numel() > 1 else aq.to(torch.float32) * a_s
    Bd = bq.to(torch.float32) * b_s.to(torch.float32)
    out = torch.zeros((M_total, N), dtype=torch.float32)
    for g in range(G):
        lo, hi = int(group_offs[g]), int(group_offs[g + 1])
        if hi > lo:
            out[lo:hi] = A[lo:hi] @ (Bd[g].t() if trans_b else Bd[g])
    return out.to(out_dtype)


def grouped_gemm_variable_k_scaled(lhs_q, lhs_s, rhs_q, rhs_s, group_offs, out_dtype=torch.bfloat16):
    """Variable-K grouped GEMM with one scale per output row / column (rowwise) or one scalar each
    (tensorwise): C[g] = (lhs[offs[g]:offs[g+1]]^T . rhs[offs[g]:offs[g+1]]) * ls[:, None] * rs[None, :].
    The group boundaries are the unpadded row offsets, so a group's contraction range need not be a
    multiple of 128 (primus_turbo/pytorch/ops/grouped_gemm_fp8.py:345-393 rowwise wgrad, :522-568
    tensorwise wgrad; kernel semantics primus_turbo/triton/grouped_gemm/grouped_gemm_fp8_kernel.py,
    masked K loop).  Empty group -> zeros.  Output [G, OUT_M, OUT_N]."""
    G = group_offs.numel() - 1
    OUT_M, OUT_N = lhs_q.shape[1], rhs_q.shape[1]
    ls = lhs_s.to(torch.float32).reshape(-1, 1) if lhs_s.numel() > 1 else lhs_s.to(torch.float32).reshape(1, 1)
    rs = rhs_s.to(torch.float32).reshape(1, -1) if rhs_s.numel() > 1 else rhs_s.to(torch.float32).reshape(1, 1)
    out = torch.zeros((G, OUT_M, OUT_N), dtype=torch.float32)
    for g in range(G):
        lo, hi = int(group_offs[g]), int(group_offs[g + 1])
        if hi > lo:
            acc = lhs_q[lo:hi].to(torch.float32).t() @ rhs_q[lo:hi].to(torch.float32)
            out[g] = acc * (ls * rs)
    return out.to(out_dtype)


# ----------------------------------------------------------------------------------------------
# comparators (tests/pytorch/test_utils.py:37-74)
# ----------------------------------------------------------------------------------------------
def rel_frobenius(ref: torch.Tensor, got: torch.Tensor) -> float:
    ref, got = ref.double(), got.double()
    d = torch.linalg.norm(ref)
    return float(torch.linalg.norm(ref - got) / d) if d > 0 else float(torch.linalg.norm(got))


def snr_db(ref: torch.Tensor, got: torch.Tensor) -> float:
    ref, got = ref.double(), got.double()
    return float(10 * torch.log10(ref.pow(2).sum() / ((ref - got).pow(2).sum() + 1e-12)))


def bytes_equal(a: torch.Tensor, b: torch.Tensor) -> bool:
    return a.shape == b.shape and torch.equal(a.contiguous().view(torch.uint8), b.contiguous().view(torch.uint8))


def bits_equal_f32(a: torch.Tensor, b: torch.Tensor) -> bool:
    return a.shape == b.shape and torch.equal(a.contiguous().view(torch.int32), b.contiguous().view(torch.int32))


# ----------------------------------------------------------------------------------------------
# seeded synthetic inputs of the benchmark configurations
# ----------------------------------------------------------------------------------------------
def make_counts_softmax(num_experts: int, rows: int, gen: torch.Generator) -> torch.Tensor:
    logits = torch.randn(num_experts, generator=gen)
    p = torch.softmax(logits, 0)
    idx = torch.multinomial(p, rows, replacement=True, generator=gen)
    return torch.bincount(idx, minlength=num_experts).to(torch.int64)


def make_counts_zipf(num_experts: int, rows: int, gen: torch.Generator, s: float = 1.2, zeros: int = 8):
    perm = torch.randperm(num_experts, generator=gen)
    p = torch.arange(1, num_experts + 1, dtype=torch.float64).pow(-s)
    p = (p / p.sum()).to(torch.float32)
    pe = torch.empty(num_experts)
    pe[perm] = p
    idx = torch.multinomial(pe, rows, replacement=True, generator=gen)
    counts = torch.bincount(idx, minlength=num_experts).to(torch.int64)
    order = torch.argsort(counts, stable=True)
    moved = counts[order[:zeros]].sum()
    counts[order[:zeros]] = 0
    counts[order[-1]] += moved
    return counts
