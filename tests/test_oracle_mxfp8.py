"""CPU checks of the MXFP8 part of the oracle: known answers of the scale rule worked out by hand from
the reference source (csrc/kernels/quantization/quantization_mxfp8.cu:71-110), layouts
(csrc/pytorch/quantization/quantization.cpp:736-966) and the reference tests' closeness gate
(tests/pytorch/ops/test_quantization.py:311-360)."""

import pytest
import torch

from oracle import fp8_oracle as O

E4, E5 = torch.float8_e4m3fn, torch.float8_e5m2


def test_scale_rule_known_answers():
    # e4m3: exponent of the maximum (mantissa rounded to 3 bits) minus 8, biased by 127
    amax = torch.tensor([448.0, 1.0, 0.0, 1.9375, 1.93, 2.0, 2.0 ** -140, 3.0e38, 0.75])
    byte, native = O.mx_scale(amax, E4)
    assert byte.tolist() == [127, 119, 0, 120, 119, 120, 0, 246, 118]
    assert native[0].item() == 1.0 and native[1].item() == 2.0 ** -8 and native[2].item() == 0.0
    # e5m2: mantissa rounded to 2 bits, exponent minus 15
    amax = torch.tensor([57344.0, 1.0, 1.875, 1.87])
    byte, _ = O.mx_scale(amax, E5)
    assert byte.tolist() == [127, 112, 113, 112]


@pytest.mark.parametrize("fp8", [E4, E5])
@pytest.mark.parametrize("use_2d", [False, True])
def test_layouts_padding_and_transposed_copy(fp8, use_2d):
    g = torch.Generator().manual_seed(1)
    x = torch.randn(70, 96, generator=g).bfloat16()
    q1, s1 = O.quant_mxfp8(x, fp8, 1, use_2d)
    q0, s0 = O.quant_mxfp8(x, fp8, 0, use_2d)
    assert q1.shape == (70, 128) and s1.shape == (70, 4) and q0.shape == (96, 128) and s0.shape == (96, 4)
    assert q1.view(torch.uint8)[:, 96:].eq(0).all() and s1[:, 3].eq(0).all()
    assert q0.view(torch.uint8)[:, 70:].eq(0).all() and s0[:, 3].eq(0).all()
    if not use_2d:
        # blocks along a column of x are blocks along a row of x^T
        qt, st = O.quant_mxfp8(x[:64].t().contiguous(), fp8, 1, False)
        assert torch.equal(qt.view(torch.uint8)[:, :64], q0.view(torch.uint8)[:, :64]) and torch.equal(st[:, :2], s0[:, :2])
    else:
        # one scale per 32x32 tile: both directions carry the same byte for a tile
        assert torch.equal(s1[:64:32, :3], s0[:96:32, :2].t())


@pytest.mark.parametrize("fp8,tol", [(E4, 1e-1), (E5, 2.5e-1)])
def test_round_trip_meets_the_reference_gate(fp8, tol):
    g = torch.Generator().manual_seed(2)
    x = torch.randn(256, 64, generator=g).bfloat16()
    for axis in (0, 1):
        q, s = O.quant_mxfp8(x, fp8, axis)
        y = O.dequant_mxfp8(q, s, axis, torch.bfloat16)
        ref = torch.zeros(y.shape, dtype=torch.bfloat16)
        ref[:256, :64] = x
        torch.testing.assert_close(y, ref, rtol=tol, atol=tol)


def test_values_are_clamped_not_overflowed():
    # a block maximum of 1.9 keeps the exponent of 1.0: 1.9 * 2^8 = 486 > 448 must saturate at 448
    x = torch.zeros(1, 32, dtype=torch.bfloat16)
    x[0, 0], x[0, 1] = 1.9, -1.9
    q, s = O.quant_mxfp8(x, E4, 1)
    assert s[0, 0].item() == 119
    assert q[0, 0].float().item() == 448.0 and q[0, 1].float().item() == -448.0


def test_gemm_matches_plain_matmul_of_dequantised_operands():
    g = torch.Generator().manual_seed(3)
    a, b = torch.randn(40, 64, generator=g).bfloat16(), torch.randn(24, 64, generator=g).bfloat16()
    aq, as_ = O.quant_mxfp8(a, E4, 1)
    bq, bs_ = O.quant_mxfp8(b, E4, 1, True)
    out = O.gemm_mxfp8_nt(aq, as_, bq, bs_, torch.float32)
    assert out.shape == (40, 24)
    assert O.snr_db(a.float() @ b.float().t(), out) > 25
