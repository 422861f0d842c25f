"""MXFP8 (1x32 blocks, E8M0 scales): quantise / dequantise byte parity with the oracle, GEMM against
the oracle's dequantise-then-matmul, and the reference's own gates (tests/pytorch/ops/test_quantization.py:311-460,
test_gemm_fp8.py SNR gate)."""

import pytest
import torch

from oracle import fp8_oracle as O
from primus_turbo_b200.pytorch.core.low_precision import (
    Float8QuantConfig,
    Format,
    ScaleDtype,
    ScalingGranularity,
    ScalingRecipe,
)
from primus_turbo_b200.pytorch.ops import dequantize_fp8, gemm_fp8, quantize_fp8, quantize_fp8_with_trans

pytestmark = pytest.mark.gpu
MX = ScalingGranularity.MX_BLOCKWISE
DEV = "cuda"


def _mk(shape, dtype, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


def _same_bytes(a, b):
    return torch.equal(a.cpu().view(torch.uint8), b.cpu().view(torch.uint8))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("fp8", [torch.float8_e4m3fn, torch.float8_e5m2])
@pytest.mark.parametrize("shape", [(32, 32), (64, 256), (200, 96), (1, 64), (257, 1024), (1024, 32)])
@pytest.mark.parametrize("use_2d", [False, True])
def test_quantize_both_directions_match_oracle(dtype, fp8, shape, use_2d):
    x = _mk(shape, dtype, seed=shape[0] * 7 + shape[1])
    # a few blocks of special magnitudes: zeros, tiny, huge, exact powers of two
    x[0, :32] = 0
    if shape[0] > 3:
        x[1, :32] = 1e-30 if dtype == torch.bfloat16 else 6e-8
        x[2, :32] = 3e38 if dtype == torch.bfloat16 else 60000.0
        x[3, :32] = 2.0
    if shape[0] > 4 and dtype == torch.bfloat16:
        x[4, :32] = 0
        x[4, 0], x[4, 1] = 1e-37, -1e-37  # a maximum below 2^-119: scale byte 0, every value becomes a signed zero
    recipe = ScalingRecipe(use_2d_block=use_2d)
    q_row, s_row, q_col, s_col = quantize_fp8_with_trans(
        x.to(DEV), fp8, MX, block_size=32, scaling_recipe=recipe, scaling_recipe_for_trans=recipe
    )
    rq, rs = O.quant_mxfp8(x, fp8, 1, use_2d)
    cq, cs = O.quant_mxfp8(x, fp8, 0, use_2d)
    assert q_row.shape == rq.shape and s_row.shape == rs.shape and q_col.shape == cq.shape and s_col.shape == cs.shape
    assert s_row.dtype == torch.float8_e8m0fnu and s_col.dtype == torch.float8_e8m0fnu
    assert _same_bytes(s_row, rs), "row scale bytes"
    assert _same_bytes(s_col, cs), "column scale bytes"
    assert _same_bytes(q_row, rq), "row FP8 bytes"
    assert _same_bytes(q_col, cq), "column FP8 bytes"
    # single-direction calls give the same tensors
    q1, s1 = quantize_fp8(x.to(DEV), fp8, MX, block_size=32, axis=1, scaling_recipe=recipe)
    q0, s0 = quantize_fp8(x.to(DEV), fp8, MX, block_size=32, axis=0, scaling_recipe=recipe)
    assert _same_bytes(q1, q_row) and _same_bytes(s1, s_row) and _same_bytes(q0, q_col) and _same_bytes(s0, s_col)


@pytest.mark.parametrize("fp8", [torch.float8_e4m3fn, torch.float8_e5m2])
@pytest.mark.parametrize("axis", [0, 1])
def test_batched_quantize_and_dequantize(fp8, axis):
    x = _mk((3, 70, 96), torch.bfloat16, seed=5)
    q, s = quantize_fp8(x.to(DEV), fp8, MX, block_size=32, axis=axis + 1)
    for g in range(3):
        oq, os_ = O.quant_mxfp8(x[g], fp8, axis)
        assert _same_bytes(q[g], oq) and _same_bytes(s[g], os_)
    y = dequantize_fp8(q, torch.bfloat16, MX, block_size=32, axis=axis + 1, scale_inv=s)
    for g in range(3):
        oq, os_ = O.quant_mxfp8(x[g], fp8, axis)
        ref = O.dequant_mxfp8(oq, os_, axis, torch.bfloat16)
        assert y[g].shape == ref.shape and torch.equal(y[g].cpu(), ref)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("fp8", [torch.float8_e4m3fn, torch.float8_e5m2])
@pytest.mark.parametrize("shape", [(64, 256), (200, 96)])
def test_dequantize_matches_oracle_and_reference_tolerance(out_dtype, fp8, shape):
    x = _mk(shape, torch.bfloat16, seed=3)
    for axis in (0, 1):
        q, s = quantize_fp8(x.to(DEV), fp8, MX, block_size=32, axis=axis)
        y = dequantize_fp8(q, out_dtype, MX, block_size=32, axis=axis, scale_inv=s)
        oq, os_ = O.quant_mxfp8(x, fp8, axis)
        ref = O.dequant_mxfp8(oq, os_, axis, out_dtype)
        assert torch.equal(y.cpu(), ref)
        # the reference's own gate: dequantised values close to the zero-padded input
        pad = torch.zeros(ref.shape, dtype=torch.float32)
        pad[: shape[0], : shape[1]] = x.float()
        tol = dict(rtol=1e-1, atol=1e-1) if fp8 == torch.float8_e4m3fn else dict(rtol=2.5e-1, atol=2.5e-1)
        torch.testing.assert_close(y.float().cpu(), pad, **tol)


@pytest.mark.parametrize("fmt", [Format.E4M3, Format.E5M2, Format.HYBRID])
@pytest.mark.parametrize("mnk", [(128, 256, 128), (256, 512, 1024), (200, 320, 96), (1, 32, 32), (1000, 1056, 4096)])
def test_gemm_forward_backward_vs_oracle(fmt, mnk):
    M, N, K = mnk
    cfg = Float8QuantConfig(format=fmt, granularity=MX, block_size=32, scale_dtype=ScaleDtype.E8M0)
    a = _mk((M, K), torch.bfloat16, seed=1)
    b = _mk((N, K), torch.bfloat16, seed=2, scale=0.05)
    gy = _mk((M, N), torch.bfloat16, seed=3, scale=0.01)
    ad, bd = a.to(DEV).requires_grad_(), b.to(DEV).requires_grad_()
    out = gemm_fp8(ad, bd, trans_b=True, config=cfg)
    out.backward(gy.to(DEV))
    out = out.detach()
    fwd = torch.float8_e5m2 if fmt == Format.E5M2 else torch.float8_e4m3fn
    bwd = torch.float8_e4m3fn if fmt == Format.E4M3 else torch.float8_e5m2
    a_row, a_rs = O.quant_mxfp8(a, fwd, 1)
    a_col, a_cs = O.quant_mxfp8(a, fwd, 0)
    b_row, b_rs = O.quant_mxfp8(b, fwd, 1, True)
    b_col, b_cs = O.quant_mxfp8(b, fwd, 0, True)
    g_row, g_rs = O.quant_mxfp8(gy, bwd, 1)
    g_col, g_cs = O.quant_mxfp8(gy, bwd, 0)
    ref_out = O.gemm_mxfp8_nt(a_row, a_rs, b_row, b_rs)
    ref_ga = O.gemm_mxfp8_nt(g_row, g_rs, b_col, b_cs)
    ref_gb = O.gemm_mxfp8_nt(g_col, g_cs, a_col, a_cs)
    assert out.shape == (M, N) and ad.grad.shape == (M, K) and bd.grad.shape == (N, K)
    # parity bar for floating-point GEMMs: relative Frobenius error <= 1e-2 on identical quantised inputs
    assert O.rel_frobenius(ref_out, out.cpu()) <= 1e-2
    assert O.rel_frobenius(ref_ga, ad.grad.cpu()) <= 1e-2
    assert O.rel_frobenius(ref_gb, bd.grad.cpu()) <= 1e-2
    # the reference's gate: SNR against the high-precision product
    hp = a.float() @ b.float().t()
    assert O.snr_db(hp, out.float().cpu()) > (25 if fmt != Format.E5M2 else 20)


def test_gemm_is_deterministic():
    cfg = Float8QuantConfig(format=Format.E4M3, granularity=MX, block_size=32, scale_dtype=ScaleDtype.E8M0)
    a = _mk((300, 512), torch.bfloat16, 1).to(DEV)
    b = _mk((520, 512), torch.bfloat16, 2).to(DEV)
    first = gemm_fp8(a, b, trans_b=True, config=cfg)
    for _ in range(5):
        assert torch.equal(first, gemm_fp8(a, b, trans_b=True, config=cfg))


def test_argument_checks():
    x = _mk((64, 48), torch.bfloat16).to(DEV)
    with pytest.raises(AssertionError):
        quantize_fp8(x, torch.float8_e4m3fn, MX, block_size=32, axis=1)  # 48 is not a multiple of 32
    with pytest.raises(AssertionError):
        quantize_fp8(x[:, :32].contiguous(), torch.float8_e4m3fn, MX, block_size=128, axis=1)
    with pytest.raises(NotImplementedError):
        quantize_fp8(x[:, :32].contiguous(), torch.float8_e4m3fn, MX, block_size=32, axis=1,
                     scaling_recipe=ScalingRecipe(shuffle_scale=True))


# ---- grouped forms ------------------------------------------------------------------------------------------
from primus_turbo_b200.pytorch.kernels.quantization_impl import grouped_quantize_mxfp8_impl  # noqa: E402
from primus_turbo_b200.pytorch.ops import grouped_gemm_fp8  # noqa: E402
from primus_turbo_b200.pytorch.ops.quantization import grouped_quantize_fp8_with_trans  # noqa: E402

GROUPS = [[100, 0, 157, 43], [1], [128, 256, 384], [0, 0, 5], [33, 31, 32, 129, 1, 64]]


@pytest.mark.parametrize("fp8", [torch.float8_e4m3fn, torch.float8_e5m2])
@pytest.mark.parametrize("lens", GROUPS)
@pytest.mark.parametrize("use_2d", [False, True])
@pytest.mark.parametrize("row_align", [32, 1])
def test_grouped_quantize_matches_oracle(fp8, lens, use_2d, row_align):
    M, N = sum(lens), 96
    x = _mk((M, N), torch.bfloat16, seed=M)
    if M > 40:
        x[35:40] = 0  # a zero block inside a group: scale byte 127 in the grouped kernels
    gl = torch.tensor(lens, dtype=torch.int64)
    go = torch.cat([gl.new_zeros(1), gl.cumsum(0)])
    got = grouped_quantize_mxfp8_impl(x.to(DEV), fp8, 32, gl.to(DEV), go.to(DEV), use_2d, use_2d, row_align=row_align)
    q_row, s_row, q_col, s_col, row_lens, row_offs, col_lens, col_offs = got
    rq, rs, cq, cs, r_offs, c_offs, written = O.quant_mxfp8_grouped(x, fp8, go.tolist(), row_align, use_2d)
    assert row_offs.cpu().tolist() == r_offs and col_offs.cpu().tolist() == c_offs
    assert row_lens.cpu().tolist() == [b - a for a, b in zip(r_offs[:-1], r_offs[1:])]
    assert col_lens.cpu().tolist() == [b - a for a, b in zip(c_offs[:-1], c_offs[1:])]
    assert q_row.shape == rq.shape and s_row.shape == rs.shape and q_col.shape == cq.shape and s_col.shape == cs.shape
    w = written
    assert torch.equal(q_row.cpu().view(torch.uint8)[w], rq.view(torch.uint8)[w]), "row FP8 bytes"
    assert torch.equal(s_row.cpu().view(torch.uint8)[w], rs[w]), "row scale bytes"
    assert _same_bytes(q_col, cq), "column FP8 bytes"
    assert _same_bytes(s_col, cs), "column scale bytes"


def test_grouped_quantize_public_op_uses_the_reference_layout():
    lens = [40, 70]
    x = _mk((110, 64), torch.bfloat16, seed=9).to(DEV)
    gl = torch.tensor(lens, dtype=torch.int64, device=DEV)
    go = torch.cat([gl.new_zeros(1), gl.cumsum(0)])
    out = grouped_quantize_fp8_with_trans(x, torch.float8_e4m3fn, MX, gl, go, block_size=32)
    assert len(out) == 8
    assert out[0].shape == (192, 128) and out[2].shape == (64, 384)  # ceil((110 + 2*32)/32)*32, ceil((110 + 2*128)/128)*128
    assert out[5].cpu().tolist() == [0, 64, 160] and out[7].cpu().tolist() == [0, 128, 256]


@pytest.mark.parametrize("fmt", [Format.E4M3, Format.HYBRID])
@pytest.mark.parametrize("lens", [[100, 0, 157, 43], [128, 256, 384], [1, 0, 5, 300, 77, 33], [512] * 8])
@pytest.mark.parametrize("NK", [(256, 128), (320, 96), (1024, 1024)])
def test_grouped_gemm_forward_backward_vs_oracle(fmt, lens, NK):
    N, K = NK
    G, M = len(lens), sum(lens)
    cfg = Float8QuantConfig(format=fmt, granularity=MX, block_size=32, scale_dtype=ScaleDtype.E8M0)
    a = _mk((M, K), torch.bfloat16, seed=1)
    b = _mk((G, N, K), torch.bfloat16, seed=2, scale=0.05)
    gy = _mk((M, N), torch.bfloat16, seed=3, scale=0.01)
    gl = torch.tensor(lens, dtype=torch.int64)
    go = torch.cat([gl.new_zeros(1), gl.cumsum(0)]).tolist()
    ad, bd = a.to(DEV).requires_grad_(), b.to(DEV).requires_grad_()
    out = grouped_gemm_fp8(ad, bd, gl.to(DEV), trans_b=True, config=cfg)
    out.backward(gy.to(DEV))
    out = out.detach()
    fwd = torch.float8_e4m3fn
    bwd = torch.float8_e4m3fn if fmt == Format.E4M3 else torch.float8_e5m2
    a_row, a_rs, a_col, a_cs, _, c_offs, _ = O.quant_mxfp8_grouped(a, fwd, go, 1)
    g_row, g_rs, g_col, g_cs, _, _, _ = O.quant_mxfp8_grouped(gy, bwd, go, 1)
    b_row = [O.quant_mxfp8(b[g], fwd, 1, True) for g in range(G)]
    b_col = [O.quant_mxfp8(b[g], fwd, 0, True) for g in range(G)]
    stack = lambda pairs, i: torch.stack([p[i] for p in pairs])  # noqa: E731
    ref_out = O.grouped_gemm_mxfp8(a_row, a_rs, stack(b_row, 0), stack(b_row, 1), go)
    ref_ga = O.grouped_gemm_mxfp8(g_row, g_rs, stack(b_col, 0), stack(b_col, 1), go)
    ref_gb = O.grouped_gemm_mxfp8_variable_k(g_col, g_cs, a_col, a_cs, c_offs)
    assert out.shape == (M, N) and ad.grad.shape == (M, K) and bd.grad.shape == (G, N, K)
    assert O.rel_frobenius(ref_out, out.cpu()) <= 1e-2
    assert O.rel_frobenius(ref_ga, ad.grad.cpu()) <= 1e-2
    assert O.rel_frobenius(ref_gb, bd.grad.cpu()) <= 1e-2
    for g in range(G):  # an empty group's weight gradient is exactly zero
        if lens[g] == 0:
            assert bd.grad[g].abs().max().item() == 0.0
    hp = torch.cat([a[go[g] : go[g + 1]].float() @ b[g].float().t() for g in range(G)])
    assert O.snr_db(hp, out.float().cpu()) > 25


# ---- long contraction extents and many tiles per CTA: the scale ring goes round many times ------------------
from primus_turbo_b200 import _lib  # noqa: E402
from primus_turbo_b200.pytorch.kernels.gemm_impl import (  # noqa: E402
    gemm_mxfp8_impl,
    grouped_gemm_mxfp8_impl,
    grouped_gemm_mxfp8_variable_k_impl,
)


@pytest.mark.parametrize("mnk", [(512, 768, 8192), (4096, 4096, 2048), (300, 264, 7168 + 128)])
def test_gemm_long_k_and_many_tiles(mnk):
    M, N, K = mnk
    a = _mk((M, K), torch.bfloat16, seed=11)
    b = _mk((N, K), torch.bfloat16, seed=12, scale=0.05)
    aq, a_s = O.quant_mxfp8(a, torch.float8_e4m3fn, 1)
    bq, b_s = O.quant_mxfp8(b, torch.float8_e4m3fn, 1, True)
    _lib.gemm_status(reset=True)
    out = gemm_mxfp8_impl(aq.to(DEV), a_s.to(DEV), bq.to(DEV), b_s.to(DEV), torch.bfloat16)
    torch.cuda.synchronize()
    assert _lib.gemm_status() == 0, "a bounded wait inside the kernel ran out"
    ref = O.gemm_mxfp8_nt(aq, a_s, bq, b_s)
    assert O.rel_frobenius(ref, out.cpu()) <= 1e-2


def test_grouped_gemm_many_groups_long_k():
    g = torch.Generator().manual_seed(21)
    G, N, K = 96, 512, 7168
    lens = torch.randint(0, 90, (G,), generator=g)
    lens[5] = 0
    lens[17] = 300
    M = int(lens.sum())
    a = _mk((M, K), torch.bfloat16, seed=1)
    b = _mk((G, N, K), torch.bfloat16, seed=2, scale=0.05)
    gy = _mk((M, N), torch.bfloat16, seed=3, scale=0.01)
    go = torch.cat([lens.new_zeros(1), lens.cumsum(0)]).tolist()
    E4 = torch.float8_e4m3fn
    a_row, a_rs, a_col, a_cs, _, c_offs, _ = O.quant_mxfp8_grouped(a, E4, go, 1)
    g_row, g_rs, g_col, g_cs, _, _, _ = O.quant_mxfp8_grouped(gy, E4, go, 1)
    b_rows = [O.quant_mxfp8(b[i], E4, 1, True) for i in range(G)]
    bq, bs = torch.stack([p[0] for p in b_rows]), torch.stack([p[1] for p in b_rows])
    offs_dev = torch.tensor(go, dtype=torch.int64, device=DEV)
    _lib.gemm_status(reset=True)
    out = grouped_gemm_mxfp8_impl(a_row.to(DEV), a_rs.to(DEV), bq.to(DEV), bs.to(DEV), offs_dev, torch.bfloat16)
    gw = grouped_gemm_mxfp8_variable_k_impl(g_col.to(DEV), g_cs.to(DEV), a_col.to(DEV), a_cs.to(DEV),
                                            torch.tensor(c_offs, dtype=torch.int64, device=DEV), torch.bfloat16)
    torch.cuda.synchronize()
    assert _lib.gemm_status() == 0, "a bounded wait inside the kernel ran out"
    assert O.rel_frobenius(O.grouped_gemm_mxfp8(a_row, a_rs, bq, bs, go), out.cpu()) <= 1e-2
    assert O.rel_frobenius(O.grouped_gemm_mxfp8_variable_k(g_col, g_cs, a_col, a_cs, c_offs), gw.cpu()) <= 1e-2
