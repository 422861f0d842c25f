"""GPU parity: FP8 dense GEMM through ``gemm_fp8`` / ``gemm_fp8_impl`` (C ABI) against the oracle's
dequantise-then-matmul in fp32 on identical quantised inputs (relative Frobenius error <= 1e-2),
plus the reference's own gates: SNR vs the bf16 matmul, forward and backward, and bitwise
determinism (tests/pytorch/ops/test_gemm_fp8.py:101-114, :217-290, :574-661)."""

import pytest
import torch

from oracle import fp8_oracle as O
from tests.gpu_util import DEV, E4, E5, FROB_TOL, SNR_E4M3_DB, SNR_E5M2_DB, gen, randn

pytestmark = pytest.mark.gpu

from primus_turbo_b200 import _lib  # noqa: E402
from primus_turbo_b200.pytorch.core.low_precision import Float8QuantConfig, Format  # noqa: E402
from primus_turbo_b200.pytorch.core.low_precision import ScalingGranularity as G  # noqa: E402
from primus_turbo_b200.pytorch.core.low_precision import ScalingRecipe  # noqa: E402
from primus_turbo_b200.pytorch.core.quantized_tensor import QuantizedTensor, QuantizedTensorPair  # noqa: E402
from primus_turbo_b200.pytorch.kernels.gemm_impl import gemm_fp8_impl  # noqa: E402
from primus_turbo_b200.pytorch.ops import gemm_fp8, quantize_fp8, quantize_fp8_with_trans  # noqa: E402


def _status_ok():
    torch.cuda.synchronize()
    assert _lib.gemm_status() == 0, "a device-side wait in the GEMM kernel ran out"


def _operands(g, m, n, k, trans_a, trans_b, dtype=torch.bfloat16):
    a = randn(g, k, m, dtype=dtype) if trans_a else randn(g, m, k, dtype=dtype)
    b = randn(g, n, k, scale=0.02, dtype=dtype) if trans_b else randn(g, k, n, scale=0.02, dtype=dtype)
    return a, b


# ---- kernel-level parity on identical quantised inputs ------------------------------------------------
@pytest.mark.parametrize("layout", [(False, True), (False, False), (True, False), (True, True)])
@pytest.mark.parametrize("mnk", [(128, 256, 128), (255, 512, 576), (507, 1024, 2048), (512, 4096, 1024), (16, 48, 64)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_tensorwise_kernel(layout, mnk, out_dtype):
    ta, tb = layout
    m, n, k = mnk
    if ta and m % 16:  # a stored [K, M]: its leading dimension must be 16-byte aligned
        m = (m + 15) // 16 * 16
    a, b = _operands(gen(m + n), m, n, k, ta, tb)
    aq, a_s = O.quant_tensorwise(a, E4)
    bq, b_s = O.quant_tensorwise(b, E4)
    ref = O.gemm_tensorwise(aq, a_s, bq, b_s, ta, tb, torch.float32)
    out = gemm_fp8_impl(aq.to(DEV), a_s.to(DEV), ta, bq.to(DEV), b_s.to(DEV), tb, out_dtype, False, G.TENSORWISE.value)
    _status_ok()
    assert out.shape == (m, n)
    assert O.rel_frobenius(ref, out.float().cpu()) <= (2e-6 if out_dtype == torch.float32 else FROB_TOL)
    out_t = gemm_fp8_impl(aq.to(DEV), a_s.to(DEV), ta, bq.to(DEV), b_s.to(DEV), tb, out_dtype, True, G.TENSORWISE.value)
    assert torch.equal(out_t, out.t().contiguous())


@pytest.mark.parametrize("mnk", [(256, 512, 256), (255, 528, 576), (512, 2048, 1024)])
def test_rowwise_kernel_all_layouts(mnk):
    m, n, k = mnk
    g = gen(m)
    a, b = randn(g, m, k), randn(g, n, k, scale=0.02)
    # NT: scales along K
    aq, a_s = O.quant_rowwise(a, E4, -1)
    bq, b_s = O.quant_rowwise(b, E4, -1)
    ref = O.gemm_rowwise(aq, a_s, bq, b_s, False, True, torch.float32)
    out = gemm_fp8_impl(aq.to(DEV), a_s.to(DEV), False, bq.to(DEV), b_s.to(DEV), True, torch.float32, False, 2)
    _status_ok()
    assert O.rel_frobenius(ref, out.cpu()) <= 2e-6
    # NN (dgrad shape): b stored [K, N] with scales along K = axis -2
    bt = b.t().contiguous()  # [K, N]
    btq, bt_s = O.quant_rowwise(bt, E4, -2)
    ref = O.gemm_rowwise(aq, a_s, btq, bt_s, False, False, torch.float32)
    out = gemm_fp8_impl(aq.to(DEV), a_s.to(DEV), False, btq.to(DEV), bt_s.to(DEV), False, torch.float32, False, 2)
    assert O.rel_frobenius(ref, out.cpu()) <= 2e-6
    # TN (wgrad shape): both operands stored [K', *] with scales along K' = axis -2; m must be 16-aligned
    m2 = (m + 15) // 16 * 16
    x = randn(g, k, m2)
    y = randn(g, k, n)
    xq, x_s = O.quant_rowwise(x, E4, -2)
    yq, y_s = O.quant_rowwise(y, E4, -2)
    ref = O.gemm_rowwise(xq, x_s, yq, y_s, True, False, torch.float32)
    out = gemm_fp8_impl(xq.to(DEV), x_s.to(DEV), True, yq.to(DEV), y_s.to(DEV), False, torch.float32, False, 2)
    out_t = gemm_fp8_impl(xq.to(DEV), x_s.to(DEV), True, yq.to(DEV), y_s.to(DEV), False, torch.float32, True, 2)
    _status_ok()
    assert O.rel_frobenius(ref, out.cpu()) <= 2e-6
    assert torch.equal(out_t, out.t().contiguous())


@pytest.mark.parametrize("mnk", [(256, 512, 1024), (512, 1024, 256), (300, 640, 1152), (1024, 4096, 4096), (130, 384, 320)])
@pytest.mark.parametrize("fp8", [E4, E5])
def test_blockwise_kernel_nt_nn_tn(mnk, fp8):
    m, n, k = mnk
    g = gen(k)
    a, b = randn(g, m, k), randn(g, n, k, scale=0.02)
    a_row, a_s_row, a_col, a_s_col = O.quant_block1d_dual(a, fp8)
    bq, b_s = O.quant_block2d(b, fp8)
    dev = lambda *ts: [t.to(DEV) for t in ts]  # noqa: E731
    # NT forward
    ref = O.gemm_blockwise_nt(a_row, a_s_row, bq, b_s, torch.float32)
    out = gemm_fp8_impl(*dev(a_row, a_s_row), False, *dev(bq, b_s), True, torch.float32, False, 3)
    _status_ok()
    assert O.rel_frobenius(ref, out.cpu()) <= 5e-6
    out_bf16 = gemm_fp8_impl(*dev(a_row, a_s_row), False, *dev(bq, b_s), True, torch.bfloat16, False, 3)
    assert O.rel_frobenius(ref, out_bf16.float().cpu()) <= FROB_TOL
    # NN dgrad: grad [M, N] (1x128 along N) times b [N, K] stored un-transposed
    gy = randn(g, m, n, scale=1e-3)
    g_row, g_s_row, g_col, g_s_col = O.quant_block1d_dual(gy, fp8)
    ref = O.gemm_blockwise_nn(g_row, g_s_row, bq, b_s, torch.float32)
    out = gemm_fp8_impl(*dev(g_row, g_s_row), False, *dev(bq, b_s), False, torch.float32, False, 3)
    assert O.rel_frobenius(ref, out.cpu()) <= 5e-6
    # TN wgrad: a_col^T [K, M] . g_col [M, N]; trans_c gives [N, K]
    ref = O.gemm_blockwise_tn(a_col, a_s_col, g_col, g_s_col, torch.float32)
    out = gemm_fp8_impl(*dev(a_col, a_s_col), True, *dev(g_col, g_s_col), False, torch.float32, False, 3)
    out_t = gemm_fp8_impl(*dev(a_col, a_s_col), True, *dev(g_col, g_s_col), False, torch.float32, True, 3)
    _status_ok()
    assert out.shape == (k, n) and out_t.shape == (n, k)
    assert O.rel_frobenius(ref, out.cpu()) <= 5e-6
    assert O.rel_frobenius(ref.t(), out_t.cpu()) <= 5e-6


def test_config1_blockwise_against_golden(golden_dir):
    """A bf16 [256,1024] ~N(0,1), B bf16 [512,1024] ~N(0,0.02), seed 0: C = A.B^T in bf16."""
    g0 = gen(0)
    A = torch.randn(256, 1024, generator=g0).to(torch.bfloat16)
    B = (torch.randn(512, 1024, generator=g0) * 0.02).to(torch.bfloat16)
    cfg = Float8QuantConfig(granularity=G.BLOCKWISE, block_size=128)
    C = gemm_fp8(A.to(DEV), B.to(DEV), trans_b=True, config=cfg)
    _status_ok()
    a_row, a_s_row, _, _ = O.quant_block1d_dual(A, E4)
    bq, b_s = O.quant_block2d(B, E4)
    ref = O.gemm_blockwise_nt(a_row, a_s_row, bq, b_s, torch.float32)
    assert C.dtype == torch.bfloat16 and C.shape == (256, 512)
    assert O.rel_frobenius(ref, C.float().cpu()) <= FROB_TOL
    assert O.snr_db(A.float() @ B.float().t(), C.float().cpu()) > SNR_E4M3_DB


# ---- public op, forward + backward, reference gates ----------------------------------------------------
def _fwd_bwd(a, b, trans_a, trans_b, cfg):
    a = a.clone().requires_grad_(True)
    b = b.clone().requires_grad_(True)
    out = gemm_fp8(a, b, trans_a, trans_b, None, cfg)
    go = torch.randn_like(out)
    out.backward(go)
    return out.detach(), a.grad.detach(), b.grad.detach(), go


def _ref_fwd_bwd(a, b, trans_a, trans_b, go):
    a = a.clone().float().requires_grad_(True)
    b = b.clone().float().requires_grad_(True)
    out = (a.t() if trans_a else a) @ (b.t() if trans_b else b)
    out.backward(go.float())
    return out.detach(), a.grad, b.grad


@pytest.mark.parametrize("gran", [G.TENSORWISE, G.ROWWISE, G.BLOCKWISE])
@pytest.mark.parametrize("fmt", [Format.E4M3, Format.HYBRID])
@pytest.mark.parametrize("mnk", [(256, 512, 256), (512, 1024, 576), (512, 4096, 1024)])
@pytest.mark.parametrize("trans_b", [True, False])
def test_gemm_fp8_fwd_bwd_snr(gran, fmt, mnk, trans_b):
    m, n, k = mnk
    if gran == G.BLOCKWISE and k % 128:
        k = 640
    a, b = _operands(gen(m * 3 + n), m, n, k, False, trans_b)
    a, b = a.to(DEV), (b * 50).to(DEV)
    cfg = Float8QuantConfig(format=fmt, granularity=gran, block_size=128 if gran == G.BLOCKWISE else None)
    out, ga, gb, go = _fwd_bwd(a, b, False, trans_b, cfg)
    _status_ok()
    ro, rga, rgb = _ref_fwd_bwd(a, b, False, trans_b, go)
    bwd_gate = SNR_E5M2_DB if fmt == Format.HYBRID else SNR_E4M3_DB
    assert out.dtype == torch.bfloat16 and ga.shape == a.shape and gb.shape == b.shape
    assert O.snr_db(ro.cpu(), out.float().cpu()) > SNR_E4M3_DB
    assert O.snr_db(rga.cpu(), ga.float().cpu()) > bwd_gate
    assert O.snr_db(rgb.cpu(), gb.float().cpu()) > bwd_gate


def test_gemm_fp8_tensorwise_trans_a():
    a, b = _operands(gen(1), 256, 512, 384, True, False)
    cfg = Float8QuantConfig()
    out, ga, gb, go = _fwd_bwd(a.to(DEV), b.to(DEV), True, False, cfg)
    ro, rga, rgb = _ref_fwd_bwd(a.to(DEV), b.to(DEV), True, False, go)
    assert ga.shape == a.shape
    for r, x in ((ro, out), (rga, ga), (rgb, gb)):
        assert O.snr_db(r.cpu(), x.float().cpu()) > SNR_E4M3_DB


def test_rowwise_backward_uses_requantised_operands():
    """The rowwise backward operands are quantised from the *dequantised* forward operands
    (reference ops/gemm_fp8.py:259-291): reproduce that schedule with the oracle."""
    g = gen(21)
    m, n, k = 256, 384, 512
    a, b = randn(g, m, k), randn(g, n, k, scale=0.02)
    go = randn(g, m, n, scale=1e-3)
    cfg = Float8QuantConfig(granularity=G.ROWWISE)
    ad, bd = a.to(DEV).requires_grad_(True), b.to(DEV).requires_grad_(True)
    out = gemm_fp8(ad, bd, trans_b=True, config=cfg)
    out.backward(go.to(DEV))
    _status_ok()
    aq, a_s = O.quant_rowwise(a, E4, -1)
    bq, b_s = O.quant_rowwise(b, E4, -1)
    a_t_q, a_t_s = O.quant_rowwise(O.dequant_rowwise(aq, a_s, torch.bfloat16), E4, -2)
    b_t_q, b_t_s = O.quant_rowwise(O.dequant_rowwise(bq, b_s, torch.bfloat16), E4, -2)
    gq, g_s = O.quant_rowwise(go, E4, -1)
    gtq, gt_s = O.quant_rowwise(go, E4, -2)
    ref_ga = O.gemm_rowwise(gq, g_s, b_t_q, b_t_s, False, False, torch.float32)  # [M,N].[N,K]
    ref_gb = O.gemm_rowwise(gtq, gt_s, a_t_q, a_t_s, True, False, torch.float32)  # g^T [N,M].[M,K]
    assert O.rel_frobenius(ref_ga, ad.grad.float().cpu()) <= FROB_TOL
    assert O.rel_frobenius(ref_gb, bd.grad.float().cpu()) <= FROB_TOL


def test_prequantized_inputs():
    g = gen(8)
    a, b = randn(g, 256, 512).to(DEV), randn(g, 384, 512, scale=0.02).to(DEV)
    cfg = Float8QuantConfig()
    qa = QuantizedTensor.quantize(a, E4, G.TENSORWISE)
    qb = QuantizedTensor.quantize(b, E4, G.TENSORWISE)
    o1 = gemm_fp8(a, b, trans_b=True, config=cfg)
    o2 = gemm_fp8(qa, qb, trans_b=True, out_dtype=torch.bfloat16, config=cfg)
    o3 = gemm_fp8(QuantizedTensorPair(qa), QuantizedTensorPair(qb, qb.t()), trans_b=True, out_dtype=torch.bfloat16, config=cfg)
    assert torch.equal(o1, o2) and torch.equal(o1, o3)
    assert torch.equal(qa.t().qdata.view(torch.uint8), qa.qdata.view(torch.uint8).t().contiguous())
    torch.testing.assert_close(qa.dequantize().float(), a.float(), rtol=1e-1, atol=1e-1)
    cfgb = Float8QuantConfig(granularity=G.BLOCKWISE, block_size=128)
    qwb = QuantizedTensor.quantize(b, E4, G.BLOCKWISE, axis=-1, block_size=128, scaling_recipe=ScalingRecipe(use_2d_block=True))
    o4 = gemm_fp8(a, qwb, trans_b=True, out_dtype=torch.bfloat16, config=cfgb)
    o5 = gemm_fp8(a, b, trans_b=True, config=cfgb)
    assert torch.equal(o4, o5)


@pytest.mark.parametrize("gran", [G.TENSORWISE, G.ROWWISE, G.BLOCKWISE])
def test_deterministic(gran):
    a, b = _operands(gen(2), 512, 1024, 1024, False, True)
    a, b = a.to(DEV), b.to(DEV)
    cfg = Float8QuantConfig(granularity=gran, block_size=128 if gran == G.BLOCKWISE else None)
    first = _fwd_bwd_fixed(a, b, cfg)
    for _ in range(9):
        again = _fwd_bwd_fixed(a, b, cfg)
        for x, y in zip(first, again):
            assert torch.equal(x, y)


def _fwd_bwd_fixed(a, b, cfg):
    a = a.clone().requires_grad_(True)
    b = b.clone().requires_grad_(True)
    out = gemm_fp8(a, b, False, True, None, cfg)
    out.backward(torch.ones_like(out))
    return out.detach(), a.grad, b.grad


def test_errors():
    a = torch.zeros(4, 8, 16, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(AssertionError):
        gemm_fp8(a, a)
    x = torch.zeros(64, 24, device=DEV, dtype=torch.bfloat16)  # K = 24 is not 16-byte aligned
    with pytest.raises(RuntimeError):
        gemm_fp8(x, x, trans_b=True)
    with pytest.raises(AssertionError):
        gemm_fp8(x, x, trans_a=True, trans_b=True, config=Float8QuantConfig(granularity=G.ROWWISE))


def test_llama_mlp_shape_tensorwise():
    """Llama-3-8B MLP up-projection shape, forward only: [8192,4096] x [14336,4096]^T."""
    m, n, k = 8192, 14336, 4096
    x = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(n, k, device=DEV, dtype=torch.bfloat16) * 0.02
    out = gemm_fp8(x, w, trans_b=True)
    _status_ok()
    xq, x_s = quantize_fp8(x, E4, G.TENSORWISE)
    wq, w_s = quantize_fp8(w, E4, G.TENSORWISE)
    # identical quantised inputs, fp32 reference on a row / column sample (full fp32 matmul is 1 TFLOP)
    rows = torch.arange(0, m, 97, device=DEV)
    ref = (xq[rows].float() @ wq.float().t()) * (x_s * w_s)
    assert O.rel_frobenius(ref.cpu(), out[rows].float().cpu()) <= FROB_TOL
    assert O.snr_db((x[rows].float() @ w.float().t()).cpu(), out[rows].float().cpu()) > SNR_E4M3_DB


def test_bounded_wait_gives_up_and_reports():
    """A wait that nothing satisfies returns after its 2 s limit: the kernel ends normally, the
    status word holds the self-test's code, and the library keeps working afterwards."""
    import time

    import ctypes

    from primus_turbo_b200 import _lib

    assert _lib.gemm_status(reset=True) == 0
    t0 = time.time()
    _lib.check(_lib.lib.ptb_gemm_wait_selftest(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "selftest")
    torch.cuda.synchronize()
    waited = time.time() - t0
    assert 1.5 < waited < 10.0, waited
    assert _lib.gemm_status(reset=True) == 9
    assert _lib.gemm_status(reset=False) == 0
    # the context is intact: a small GEMM still runs and is correct
    a = torch.randn(128, 256, device="cuda").to(torch.float8_e4m3fn)
    b = torch.randn(256, 256, device="cuda").to(torch.float8_e4m3fn)
    one = torch.ones((), device="cuda")
    out = gemm_fp8_impl(a, one, False, b, one, True, torch.float32, False, 1)
    ref = a.float() @ b.float().t()
    assert O.rel_frobenius(ref.cpu(), out.cpu()) < 1e-5
    assert _lib.gemm_status(reset=True) == 0
