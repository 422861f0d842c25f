"""GPU parity, second tier: the grouped rowwise / tensorwise kernels against the oracle on identical
quantised inputs (fp32 outputs, so only the accumulation order may differ), and the full-size
benchmark configurations checked on sampled groups / rows for forward, dgrad and wgrad.

Reference behaviour being matched: primus_turbo/pytorch/ops/grouped_gemm_fp8.py:214-393 (rowwise),
:396-568 (tensorwise), tests/pytorch/ops/test_grouped_gemm_fp8.py:157-175,493-520 (shape grid and
gates), tests/pytorch/ref/gemm_ref.py:13-41 (per-group reference)."""

import pytest
import torch

from oracle import fp8_oracle as O
from tests.gpu_util import DEV, E4, FROB_TOL, gen, randn, unbalanced_lens

pytestmark = pytest.mark.gpu

from primus_turbo_b200 import _lib  # noqa: E402
from primus_turbo_b200.pytorch.core.low_precision import ScalingGranularity as G  # noqa: E402
from primus_turbo_b200.pytorch.kernels.gemm_impl import (  # noqa: E402
    gemm_fp8_impl,
    grouped_gemm_fp8_impl,
    grouped_gemm_fp8_variable_k_impl,
)
from primus_turbo_b200.pytorch.kernels.quantization_impl import (  # noqa: E402
    quant_fp8_blockwise_for_weight_impl,
    quant_fp8_blockwise_segment_m_row_col_impl,
)

F32_TOL = 5e-6  # fp32 output: identical inputs, identical products, only the summation order differs


def _status_ok():
    torch.cuda.synchronize()
    assert _lib.gemm_status() == 0, "a device-side wait in the GEMM kernel ran out"


# ---- grouped rowwise / tensorwise kernels vs the oracle ------------------------------------------------
LENS_CASES = [
    [128, 256],
    [100, 0, 300, 1, 513],  # unpadded contraction ranges: 100, 300, 1, 513 rows
    [37] * 9 + [0, 0] + [700],
    [0, 0, 0],
    [1],
    [129, 127, 255, 257],
]


@pytest.mark.parametrize("gran", [G.ROWWISE, G.TENSORWISE])
@pytest.mark.parametrize("trans_b", [True, False])
@pytest.mark.parametrize("lens", LENS_CASES)
@pytest.mark.parametrize("nk", [(256, 384), (768, 512)])
def test_rowwise_tensorwise_kernels_vs_oracle(gran, trans_b, lens, nk):
    n, k = nk
    g = gen(len(lens) * 7 + n)
    gl = torch.tensor(lens, dtype=torch.int64)
    offs = O.group_offs_from_lens(gl)
    mu = int(offs[-1])
    m = mu + 3  # three rows past the last group
    ng = gl.numel()
    x = randn(g, m, k)
    w = randn(g, ng, n, k, scale=0.02) if trans_b else randn(g, ng, k, n, scale=0.02)
    gy = randn(g, m, n, scale=1e-3)
    w_k_axis, w_n_axis = (-1, -2) if trans_b else (-2, -1)
    if gran == G.ROWWISE:
        xq, x_s = O.quant_rowwise(x, E4, -1)  # [m,1]
        wq, w_s = O.quant_rowwise(w, E4, w_k_axis)  # forward: scales over K
        wq_b, w_s_b = O.quant_rowwise(w, E4, w_n_axis)  # dgrad: scales over N
        gq, g_s = O.quant_rowwise(gy, E4, -1)
        xq_t, x_s_t = O.quant_rowwise(x, E4, -2)  # wgrad operands: one scale per column over all rows
        gq_t, g_s_t = O.quant_rowwise(gy, E4, -2)
    else:
        xq, x_s = O.quant_tensorwise(x, E4)
        wq, w_s = O.quant_tensorwise(w, E4)
        wq_b, w_s_b = wq, w_s
        gq, g_s = O.quant_tensorwise(gy, E4)
        xq_t, x_s_t, gq_t, g_s_t = xq, x_s, gq, g_s
    gld, offd = gl.to(DEV), offs.to(DEV)
    # forward
    out = grouped_gemm_fp8_impl(xq.to(DEV), wq.to(DEV), x_s.to(DEV), w_s.to(DEV), gld, offd, False, trans_b,
                                torch.float32, gran.value)
    _status_ok()
    ref = O.grouped_gemm_rowwise(xq, x_s, wq, w_s, offs, trans_b, torch.float32)
    assert out.shape == (m, n)
    assert O.rel_frobenius(ref, out.cpu()) <= F32_TOL
    assert bool((out[mu:] == 0).all())
    # dgrad: grad_out . op(W)^-T with the weight as stored
    dx = grouped_gemm_fp8_impl(gq.to(DEV), wq_b.to(DEV), g_s.to(DEV), w_s_b.to(DEV), gld, offd, False, not trans_b,
                               torch.float32, gran.value)
    _status_ok()
    ref = O.grouped_gemm_rowwise(gq, g_s, wq_b, w_s_b, offs, not trans_b, torch.float32)
    assert dx.shape == (m, k)
    assert O.rel_frobenius(ref, dx.cpu()) <= F32_TOL
    assert bool((dx[mu:] == 0).all())
    # wgrad over the unpadded row ranges (the last contraction block of a group is masked in the kernel)
    dw = grouped_gemm_fp8_variable_k_impl(xq_t.to(DEV), gq_t.to(DEV), x_s_t.to(DEV), g_s_t.to(DEV), gld, offd, True,
                                          False, trans_b, torch.float32, gran.value)
    _status_ok()
    lq, ls, rq, rs = (gq_t, g_s_t, xq_t, x_s_t) if trans_b else (xq_t, x_s_t, gq_t, g_s_t)
    ref = O.grouped_gemm_variable_k_scaled(lq, ls, rq, rs, offs, torch.float32)
    assert dw.shape == w.shape
    assert O.rel_frobenius(ref, dw.cpu()) <= F32_TOL
    for gi in torch.nonzero(gl == 0).flatten().tolist():
        assert bool((dw[gi] == 0).all()), "an empty group must produce a zero weight gradient"


def test_variable_k_tail_ignores_rows_of_other_groups():
    """The last contraction block of an unpadded group overlaps the next group's rows (or rows past
    the last group) in both operands: whatever those rows hold -- including FP8 NaN bytes -- must not
    reach this group's result."""
    g = gen(77)
    lens = torch.tensor([70, 200, 3], dtype=torch.int64)
    offs = O.group_offs_from_lens(lens)
    mu, n, k = int(offs[-1]), 256, 384
    m = mu + 64
    x, gy = randn(g, m, k), randn(g, m, n, scale=1e-3)
    xq, x_s = O.quant_rowwise(x, E4, -2)
    gq, g_s = O.quant_rowwise(gy, E4, -2)
    xb, gb = xq.view(torch.uint8).clone(), gq.view(torch.uint8).clone()
    xb[mu:], gb[mu:] = 0x7F, 0xFF  # e4m3 NaN patterns in the rows past the last group
    dw = grouped_gemm_fp8_variable_k_impl(xb.view(E4).to(DEV), gb.view(E4).to(DEV), x_s.to(DEV), g_s.to(DEV),
                                          lens.to(DEV), offs.to(DEV), True, False, True, torch.float32, G.ROWWISE.value)
    _status_ok()
    ref = O.grouped_gemm_variable_k_scaled(gq, g_s, xq, x_s, offs, torch.float32)
    assert bool(torch.isfinite(dw).all())
    assert O.rel_frobenius(ref, dw.cpu()) <= F32_TOL


# ---- blockwise at sizes where a whole CPU reference is too slow: sampled groups ------------------------
def _blockwise_sampled(counts, n, k, sample, seed, w_scale=0.02, out_dtype=torch.bfloat16, tol=FROB_TOL):
    """forward, dgrad and wgrad launches at full size; oracle on the sampled groups only."""
    torch.manual_seed(seed)
    E = counts.numel()
    offs = O.group_offs_from_lens(counts)
    M = int(offs[-1])
    a = torch.randn(M, k, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(E, n, k, device=DEV, dtype=torch.bfloat16) * w_scale
    gy = torch.randn(M, n, device=DEV, dtype=torch.bfloat16) * 1e-3
    cd, od = counts.to(DEV), offs.to(DEV)
    a_row, a_col, a_s_row, a_s_col, _, _ = quant_fp8_blockwise_segment_m_row_col_impl(a, E4, 128, cd, od)
    wq, w_s = quant_fp8_blockwise_for_weight_impl(w, E4)
    del a, w
    out = grouped_gemm_fp8_impl(a_row, wq, a_s_row, w_s, cd, od, False, True, out_dtype, 3)
    g_row, g_col, g_s_row, g_s_col, vk_lens, vk_offs = quant_fp8_blockwise_segment_m_row_col_impl(gy, E4, 128, cd, od)
    dx = grouped_gemm_fp8_impl(g_row, wq, g_s_row, w_s, cd, od, False, False, out_dtype, 3)
    dw = grouped_gemm_fp8_variable_k_impl(a_col, g_col, a_s_col, g_s_col, vk_lens, vk_offs, True, False, True,
                                          out_dtype, 3)
    _status_ok()
    vko = vk_offs.cpu()
    for gi in sample:
        lo, hi = int(offs[gi]), int(offs[gi + 1])
        plo, phi = int(vko[gi]), int(vko[gi + 1])
        if hi == lo:
            assert plo == phi
            assert bool((dw[gi] == 0).all()), "an empty group must produce a zero weight gradient"
            continue
        W = O.dequant_block2d(wq[gi].cpu(), w_s[gi].cpu())
        A = O.dequant_block1d(a_row[lo:hi].cpu(), a_s_row[:, lo:hi].t().contiguous().cpu(), 1)
        assert O.rel_frobenius(A @ W.t(), out[lo:hi].float().cpu()) <= tol, f"forward, group {gi}"
        Gr = O.dequant_block1d(g_row[lo:hi].cpu(), g_s_row[:, lo:hi].t().contiguous().cpu(), 1)
        assert O.rel_frobenius(Gr @ W, dx[lo:hi].float().cpu()) <= tol, f"dgrad, group {gi}"
        L = O.dequant_block1d(g_col[plo:phi].cpu(), g_s_col[plo // 128 : phi // 128].cpu(), 0)
        R = O.dequant_block1d(a_col[plo:phi].cpu(), a_s_col[plo // 128 : phi // 128].cpu(), 0)
        assert O.rel_frobenius(L.t() @ R, dw[gi].float().cpu()) <= tol, f"wgrad, group {gi}"
    return out, dx, dw


def test_deepseek_v3_shape_sampled_fwd_dgrad_wgrad():
    """256 experts, K=7168, N=4096, 65536 rows, softmax-multinomial counts: all three launches at
    full size, each compared with the oracle on sampled groups (smallest, largest, four others)."""
    E, K, N, M = 256, 7168, 4096, 65536
    counts = O.make_counts_softmax(E, M, gen(0))
    sample = sorted({0, 17, 128, 255, int(counts.argmax()), int(counts.argmin())})
    _blockwise_sampled(counts, N, K, sample, seed=3)


def test_qwen3_shape_sampled_fwd_dgrad_wgrad():
    """128 experts, K=2048, N=1536, 32768 rows, Zipf(1.2) counts with >= 8 empty groups: sampled groups
    include an empty one and the largest one."""
    E, K, N, M = 128, 2048, 1536, 32768
    counts = O.make_counts_zipf(E, M, gen(0))
    empty = int(torch.nonzero(counts == 0)[0])
    sample = sorted({empty, int(counts.argmax()), 1, 64, 127, int(torch.nonzero(counts > 0)[0])})
    _blockwise_sampled(counts, N, K, sample, seed=4)


@pytest.mark.parametrize("b,m,nk", [(16, 512, (4096, 7168)), (32, 512, (4096, 7168)), (32, 512, (7168, 2048))])
def test_blockwise_unbalanced_reference_grid_large(b, m, nk):
    """The corners of the reference's shape grid whose whole CPU reference would take minutes: the same
    kernels at full size, the oracle on three sampled groups, fp32 outputs."""
    lens = unbalanced_lens(gen(b * m), b, m)
    sample = sorted({0, b // 2, b - 1})
    _blockwise_sampled(lens, nk[0], nk[1], sample, seed=b, out_dtype=torch.float32, tol=F32_TOL)


# ---- dense rowwise at the Llama-3-70B attention out-projection shape ------------------------------------
def test_llama70b_out_proj_rowwise_fwd_dgrad_wgrad_sampled():
    """X [16384, 8192], W [8192, 8192], dY [16384, 8192], per-row scales: forward (NT), dgrad (NN) and
    wgrad (TN) launches at full size on operands quantised by this library, compared with the fp32
    dequantise-then-matmul on sampled output rows."""
    m, n, k = 16384, 8192, 8192
    torch.manual_seed(5)
    x = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(n, k, device=DEV, dtype=torch.bfloat16) * 0.02
    gy = torch.randn(m, n, device=DEV, dtype=torch.bfloat16) * 1e-3
    from primus_turbo_b200.pytorch.kernels.quantization_impl import quantize_fp8_rowwise_impl as qr

    xq, x_s = qr(x, E4, -1)
    wq, w_s = qr(w, E4, -1)
    gq, g_s = qr(gy, E4, -1)
    wq_t, w_s_t = qr(w, E4, -2)  # [1, K] scales for dgrad
    xq_t, x_s_t = qr(x, E4, -2)  # [1, K]
    gq_t, g_s_t = qr(gy, E4, -2)  # [1, N]
    out = gemm_fp8_impl(xq, x_s, False, wq, w_s, True, torch.bfloat16, False, G.ROWWISE.value)
    dx = gemm_fp8_impl(gq, g_s, False, wq_t, w_s_t, False, torch.bfloat16, False, G.ROWWISE.value)
    dw = gemm_fp8_impl(gq_t, g_s_t, True, xq_t, x_s_t, False, torch.bfloat16, False, G.ROWWISE.value)
    _status_ok()
    assert out.shape == (m, n) and dx.shape == (m, k) and dw.shape == (n, k)
    rows = torch.arange(0, m, 331, device=DEV)
    ref = (xq[rows].float() * x_s[rows]) @ (wq.float() * w_s).t()
    assert O.rel_frobenius(ref.cpu(), out[rows].float().cpu()) <= FROB_TOL
    ref = (gq[rows].float() * g_s[rows]) @ (wq_t.float() * w_s_t)
    assert O.rel_frobenius(ref.cpu(), dx[rows].float().cpu()) <= FROB_TOL
    rows_n = torch.arange(0, n, 163, device=DEV)
    ref = (gq_t[:, rows_n].float() * g_s_t[:, rows_n]).t() @ (xq_t.float() * x_s_t)
    assert O.rel_frobenius(ref.cpu(), dw[rows_n].float().cpu()) <= FROB_TOL


# ---- weights quantised ahead of time ----------------------------------------------------------------------
@pytest.mark.parametrize("trans_b", [True, False])
def test_cached_blockwise_weight_is_bit_identical_to_the_raw_path(trans_b):
    """create_quantized_weight once, then grouped_gemm_fp8 / gemm_fp8 on the cached payload: the payload
    equals a fresh quantisation byte for byte, and out, grad_a and grad_w are bit-identical to the
    path that re-quantises the raw weight in every forward
    (primus_turbo/pytorch/core/quantized_tensor.py:884-956 in the reference)."""
    from primus_turbo_b200.pytorch.core.low_precision import Float8QuantConfig
    from primus_turbo_b200.pytorch.core.quantized_tensor import QuantizedTensorPair, create_quantized_weight
    from primus_turbo_b200.pytorch.ops import gemm_fp8, grouped_gemm_fp8

    cfg = Float8QuantConfig(granularity=G.BLOCKWISE, block_size=128)
    g = gen(31)
    lens = torch.tensor([200, 0, 300, 77, 1], dtype=torch.int64, device=DEV)
    m, n, k, E = int(lens.sum()), 512, 640, 5
    a = randn(g, m, k).to(DEV)
    w = (randn(g, E, n, k, scale=0.02) if trans_b else randn(g, E, k, n, scale=0.02)).to(DEV)
    go = randn(g, m, n, scale=1e-3).to(DEV)
    qw, qw_t = create_quantized_weight(w.clone().requires_grad_(True), E4, cfg, need_weight_transpose_cache=True)
    fresh_q, fresh_s = quant_fp8_blockwise_for_weight_impl(w, E4)
    assert torch.equal(qw.qdata.view(torch.uint8), fresh_q.view(torch.uint8))
    assert torch.equal(qw.scale_inv.view(torch.int32), fresh_s.view(torch.int32))
    assert qw.shape == w.shape and qw.dtype == torch.bfloat16 and qw.requires_grad

    def run(weight):
        aa = a.clone().requires_grad_(True)
        ww = weight if not torch.is_tensor(weight) or weight.requires_grad else weight.clone().requires_grad_(True)
        out = grouped_gemm_fp8(aa, ww, lens, trans_b=trans_b, config=cfg)
        leaf = ww.data if isinstance(ww, QuantizedTensorPair) else ww
        ga, gw = torch.autograd.grad(out, (aa, leaf), go)
        return out.detach(), ga, gw

    base = run(w)
    for cached in (qw, QuantizedTensorPair(qw, qw_t), QuantizedTensorPair(qw)):
        got = run(cached)
        for x, y in zip(base, got):
            assert x.shape == y.shape and torch.equal(x, y)
    _status_ok()
    # dense op, same hook
    qd, _ = create_quantized_weight(w[0], E4, cfg)
    a2 = a[:256].contiguous()
    assert torch.equal(gemm_fp8(a2, qd, trans_b=trans_b, out_dtype=torch.bfloat16, config=cfg),
                       gemm_fp8(a2, w[0], trans_b=trans_b, config=cfg))
