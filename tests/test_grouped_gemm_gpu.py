"""GPU parity: FP8 grouped GEMM (forward, dgrad, wgrad) through ``grouped_gemm_fp8`` and the C ABI
against the oracle on identical quantised inputs, with the reference's structural gates: unbalanced
and zero-length groups, zeroed tail rows, bitwise determinism
(tests/pytorch/ops/test_grouped_gemm_fp8.py:157-175, :1008-1070, :1073-1130, :304-389)."""

import pytest
import torch

from oracle import fp8_oracle as O
from tests.gpu_util import DEV, E4, FROB_TOL, SNR_E4M3_DB, gen, randn, unbalanced_lens

pytestmark = pytest.mark.gpu

from primus_turbo_b200 import _lib  # noqa: E402
from primus_turbo_b200.pytorch.core.low_precision import Float8QuantConfig  # noqa: E402
from primus_turbo_b200.pytorch.core.low_precision import ScalingGranularity as G  # noqa: E402
from primus_turbo_b200.pytorch.kernels.gemm_impl import (  # noqa: E402
    group_offs_from_lens,
    grouped_gemm_fp8_impl,
    grouped_gemm_fp8_variable_k_impl,
)
from primus_turbo_b200.pytorch.kernels.quantization_impl import (  # noqa: E402
    quant_fp8_blockwise_for_weight_impl,
    quant_fp8_blockwise_segment_m_row_col_impl,
)
from primus_turbo_b200.pytorch.ops import grouped_gemm_fp8  # noqa: E402

BLOCK = Float8QuantConfig(granularity=G.BLOCKWISE, block_size=128)


def _status_ok():
    torch.cuda.synchronize()
    assert _lib.gemm_status() == 0, "a device-side wait in the GEMM kernel ran out"


def _blockwise_kernels_vs_oracle(lens, n, k, trans_b, extra_rows=0, seed=0):
    """forward, dgrad and wgrad kernels on identical quantised inputs."""
    g = gen(seed)
    gl = torch.tensor(lens, dtype=torch.int64) if not torch.is_tensor(lens) else lens
    offs = O.group_offs_from_lens(gl)
    m = int(offs[-1]) + extra_rows
    ng = gl.numel()
    x = randn(g, m, k)
    w = randn(g, ng, n, k, scale=0.02) if trans_b else randn(g, ng, k, n, scale=0.02)
    gy = randn(g, m, n, scale=1e-3)
    gld, offd = gl.to(DEV), offs.to(DEV)
    a_row, a_col, a_s_row, a_s_col, _, _ = quant_fp8_blockwise_segment_m_row_col_impl(x.to(DEV), E4, 128, gld, offd)
    wq, w_s = quant_fp8_blockwise_for_weight_impl(w.to(DEV), E4)
    mu = int(offs[-1])
    # --- forward ---
    out = grouped_gemm_fp8_impl(a_row, wq, a_s_row, w_s, gld, offd, False, trans_b, torch.float32, 3)
    _status_ok()
    aq = a_row.cpu().view(torch.uint8).clone()
    aq[mu:] = 0
    ast = a_s_row.cpu().clone()
    ast[:, mu:] = 0
    ref = O.grouped_gemm_blockwise(aq.view(E4), ast, wq.cpu(), w_s.cpu(), offs, trans_b, torch.float32)
    assert O.rel_frobenius(ref, out.cpu()) <= 5e-6
    assert bool((out[mu:] == 0).all()), "rows past the last group must be zero"
    # --- dgrad: grad_out . op(W)^-T, the weight stays as stored ---
    g_row, g_col, g_s_row, g_s_col, vk_lens, vk_offs = quant_fp8_blockwise_segment_m_row_col_impl(
        gy.to(DEV), E4, 128, gld, offd
    )
    dx = grouped_gemm_fp8_impl(g_row, wq, g_s_row, w_s, gld, offd, False, not trans_b, torch.float32, 3)
    _status_ok()
    gq = g_row.cpu().view(torch.uint8).clone()
    gq[mu:] = 0
    gst = g_s_row.cpu().clone()
    gst[:, mu:] = 0
    ref = O.grouped_gemm_blockwise(gq.view(E4), gst, wq.cpu(), w_s.cpu(), offs, not trans_b, torch.float32)
    assert dx.shape == (m, k)
    assert O.rel_frobenius(ref, dx.cpu()) <= 5e-6
    # --- wgrad over the segment-padded column copies ---
    dw = grouped_gemm_fp8_variable_k_impl(
        a_col, g_col, a_s_col, g_s_col, vk_lens, vk_offs, True, False, trans_b, torch.float32, 3
    )
    _status_ok()
    pu = int(vk_offs[-1])
    lq, ls = (g_col, g_s_col) if trans_b else (a_col, a_s_col)
    rq, rs = (a_col, a_s_col) if trans_b else (g_col, g_s_col)
    ref = O.grouped_gemm_blockwise_variable_k(
        lq.cpu()[:pu], ls.cpu()[: pu // 128], rq.cpu()[:pu], rs.cpu()[: pu // 128], vk_offs.cpu(), torch.float32
    )
    assert dw.shape == w.shape
    assert O.rel_frobenius(ref, dw.cpu()) <= 5e-6
    for gi in torch.nonzero(gl == 0).flatten().tolist():
        assert bool((dw[gi] == 0).all()), "an empty group must produce a zero weight gradient"


@pytest.mark.parametrize("trans_b", [True, False])
@pytest.mark.parametrize(
    "lens,n,k",
    [
        ([128, 256], 256, 256),
        ([100, 0, 300, 1, 513], 512, 384),
        ([64] * 40 + [0] * 8 + [700], 768, 512),
        ([0, 0, 0], 256, 128),
        ([1], 128, 128),
        ([2047], 1536, 2048),
    ],
)
def test_blockwise_kernels(lens, n, k, trans_b):
    _blockwise_kernels_vs_oracle(lens, n, k, trans_b, extra_rows=5)


@pytest.mark.parametrize("b", [1, 2, 3, 8, 16, 32])
@pytest.mark.parametrize("m", [128, 512])
@pytest.mark.parametrize("nk", [(2048, 1536), (4096, 7168), (7168, 2048)])
def test_blockwise_unbalanced_reference_grid(b, m, nk):
    if b * m * nk[0] * nk[1] > 32 * 512 * 2048 * 1536 * 3:
        return  # a whole CPU reference takes minutes: test_grouped_gemm_parity_gpu.py checks these on sampled groups
    _blockwise_kernels_vs_oracle(unbalanced_lens(gen(b * m), b, m), nk[0], nk[1], True, seed=b)


def _op_fwd_bwd(a, w, lens, trans_b, cfg):
    a = a.clone().requires_grad_(True)
    w = w.clone().requires_grad_(True)
    out = grouped_gemm_fp8(a, w, lens, trans_b=trans_b, config=cfg)
    go = torch.randn_like(out) * 1e-3
    out.backward(go)
    return out.detach(), a.grad, w.grad, go


def _ref_fwd_bwd(a, w, lens, trans_b, go):
    """tests/pytorch/ref/gemm_ref.py:13-24: per-group fp32 matmul."""
    a = a.clone().float().requires_grad_(True)
    w = w.clone().float().requires_grad_(True)
    outs, start = [], 0
    for i, sz in enumerate(lens.tolist()):
        rhs = w[i].t() if trans_b else w[i]
        outs.append(a[start : start + sz] @ rhs)
        start += sz
    out = torch.cat(outs)
    out.backward(go.float()[: out.shape[0]])
    return out.detach(), a.grad, w.grad


@pytest.mark.parametrize("gran", [G.BLOCKWISE, G.ROWWISE, G.TENSORWISE])
@pytest.mark.parametrize("b,m", [(1, 256), (3, 128), (8, 512), (32, 256)])
@pytest.mark.parametrize("nk", [(2048, 1536), (4096, 7168), (7168, 2048)])
@pytest.mark.parametrize("trans_b", [True, False])
def test_op_fwd_bwd_snr(gran, b, m, nk, trans_b):
    n, k = nk
    g = gen(b + m)
    lens = unbalanced_lens(g, b, m)
    a = randn(g, b * m, k).to(DEV)
    w = (randn(g, b, n, k) if trans_b else randn(g, b, k, n)).to(DEV)
    cfg = Float8QuantConfig(granularity=gran, block_size=128 if gran == G.BLOCKWISE else None)
    out, ga, gw, go = _op_fwd_bwd(a, w, lens.to(DEV), trans_b, cfg)
    _status_ok()
    ro, rga, rgw = _ref_fwd_bwd(a, w, lens, trans_b, go)
    assert out.shape == (b * m, n) and ga.shape == a.shape and gw.shape == w.shape
    assert O.snr_db(ro.cpu(), out.float().cpu()) > SNR_E4M3_DB
    assert O.snr_db(rga.cpu(), ga.float().cpu()) > SNR_E4M3_DB
    assert O.snr_db(rgw.cpu(), gw.float().cpu()) > SNR_E4M3_DB


@pytest.mark.parametrize("gran", [G.BLOCKWISE, G.ROWWISE, G.TENSORWISE])
def test_zero_length_groups(gran):
    lens = torch.tensor([1024, 1024, 0, 0, 0, 0, 0, 0], dtype=torch.int64)
    g = gen(12)
    a = randn(g, 2048, 1024).to(DEV)
    w = randn(g, 8, 512, 1024).to(DEV)
    cfg = Float8QuantConfig(granularity=gran, block_size=128 if gran == G.BLOCKWISE else None)
    out, ga, gw, go = _op_fwd_bwd(a, w, lens.to(DEV), True, cfg)
    _status_ok()
    ro, rga, rgw = _ref_fwd_bwd(a, w, lens, True, go)
    assert O.snr_db(ro.cpu(), out.float().cpu()) > SNR_E4M3_DB
    assert O.snr_db(rga.cpu(), ga.float().cpu()) > SNR_E4M3_DB
    assert O.snr_db(rgw[:2].cpu(), gw[:2].float().cpu()) > SNR_E4M3_DB
    assert bool((gw[2:] == 0).all())


@pytest.mark.parametrize("gran", [G.BLOCKWISE, G.ROWWISE, G.TENSORWISE])
def test_padded_tail_is_zeroed(gran):
    """The output is allocated for all rows of ``a``; rows past sum(group_lens) must come back zero
    even when the allocator hands out memory full of a sentinel."""
    g = gen(13)
    m_alloc, used = 1536, [300, 500, 211]
    n, k = 512, 256
    poison = torch.full((m_alloc * n * 4,), 1234.5, device=DEV, dtype=torch.bfloat16)
    del poison  # returns the sentinel-filled block to the caching allocator
    a = randn(g, m_alloc, k).to(DEV)
    w = randn(g, 3, n, k).to(DEV)
    lens = torch.tensor(used, dtype=torch.int64, device=DEV)
    cfg = Float8QuantConfig(granularity=gran, block_size=128 if gran == G.BLOCKWISE else None)
    out = grouped_gemm_fp8(a, w, lens, trans_b=True, config=cfg)
    _status_ok()
    assert bool((out[sum(used) :] == 0).all())
    ro, _, _ = _ref_fwd_bwd(a[: sum(used)], w, lens.cpu(), True, torch.zeros(sum(used), n, device=DEV))
    assert O.snr_db(ro.cpu(), out[: sum(used)].float().cpu()) > SNR_E4M3_DB


@pytest.mark.parametrize("gran", [G.BLOCKWISE, G.ROWWISE, G.TENSORWISE])
def test_deterministic(gran):
    g = gen(14)
    lens = unbalanced_lens(g, 8, 256).to(DEV)
    a = randn(g, 2048, 1024).to(DEV)
    w = randn(g, 8, 768, 1024).to(DEV)
    cfg = Float8QuantConfig(granularity=gran, block_size=128 if gran == G.BLOCKWISE else None)

    def run():
        aa, ww = a.clone().requires_grad_(True), w.clone().requires_grad_(True)
        out = grouped_gemm_fp8(aa, ww, lens, trans_b=True, config=cfg)
        out.backward(torch.ones_like(out))
        return out.detach(), aa.grad, ww.grad

    first = run()
    for _ in range(9):
        for x, y in zip(first, run()):
            assert torch.equal(x, y)


def test_num_cu_cap_and_offsets_argument():
    g = gen(15)
    lens = torch.tensor([200, 56], dtype=torch.int64, device=DEV)
    a, w = randn(g, 256, 512).to(DEV), randn(g, 2, 384, 512).to(DEV)
    o1 = grouped_gemm_fp8(a, w, lens, config=BLOCK)
    o2 = grouped_gemm_fp8(a, w, lens, group_offs=group_offs_from_lens(lens), config=BLOCK, num_cu=16)
    assert torch.equal(o1, o2)


def test_qwen3_moe_shape_with_empty_groups():
    """128 experts, hidden 2048, gate+up 1536, 32768 rows, Zipf(1.2) counts with >= 8 empty groups:
    forward + backward through the op; SNR gates on every output, empty groups give zero dW."""
    E, K, N, M = 128, 2048, 1536, 32768
    counts = O.make_counts_zipf(E, M, gen(0))
    assert int((counts == 0).sum()) >= 8 and int(counts.sum()) == M
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(E, N, K, device=DEV, dtype=torch.bfloat16) * 0.02
    out, ga, gw, go = _op_fwd_bwd(a, w, counts.to(DEV), True, BLOCK)
    _status_ok()
    ro, rga, rgw = _ref_fwd_bwd(a, w, counts, True, go)
    assert O.snr_db(ro.cpu(), out.float().cpu()) > SNR_E4M3_DB
    assert O.snr_db(rga.cpu(), ga.float().cpu()) > SNR_E4M3_DB
    nz = counts > 0
    assert O.snr_db(rgw[nz].cpu(), gw[nz].float().cpu()) > SNR_E4M3_DB
    assert bool((gw[~nz] == 0).all())


def test_deepseek_v3_shape_properties():
    """256 experts, K=7168, N=4096, 65536 rows with softmax-multinomial counts.  A full CPU oracle is
    out of reach (11.5 TFLOP), so: (i) sampled groups against the oracle on identical quantised
    inputs, (ii) linearity: doubling the weight scales doubles the output exactly (powers of two)."""
    E, K, N, M = 256, 7168, 4096, 65536
    counts = O.make_counts_softmax(E, M, gen(0))
    offs = O.group_offs_from_lens(counts)
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(E, N, K, device=DEV, dtype=torch.bfloat16) * 0.02
    cd, od = counts.to(DEV), offs.to(DEV)
    a_row, _, a_s_row, _, _, _ = quant_fp8_blockwise_segment_m_row_col_impl(a, E4, 128, cd, od)
    wq, w_s = quant_fp8_blockwise_for_weight_impl(w, E4)
    out = grouped_gemm_fp8_impl(a_row, wq, a_s_row, w_s, cd, od, False, True, torch.bfloat16, 3)
    _status_ok()
    for gi in (0, 17, 128, 255):
        lo, hi = int(offs[gi]), int(offs[gi + 1])
        if hi == lo:
            continue
        A = O.dequant_block1d(a_row[lo:hi].cpu(), a_s_row[:, lo:hi].t().contiguous().cpu(), 1)
        W = O.dequant_block2d(wq[gi].cpu(), w_s[gi].cpu())
        assert O.rel_frobenius(A @ W.t(), out[lo:hi].float().cpu()) <= FROB_TOL
    out2 = grouped_gemm_fp8_impl(a_row, wq, a_s_row, w_s * 2, cd, od, False, True, torch.bfloat16, 3)
    assert torch.equal(out2, out * 2)
