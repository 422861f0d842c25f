"""GPU: ``Float8Linear`` against ``torch.nn.Linear`` in bf16 — the reference's module test gate
(SNR of output, input gradient, weight gradient and bias gradient) at each granularity."""

import pytest
import torch

from oracle import fp8_oracle as O
from primus_turbo_b200.pytorch.core.low_precision import Float8QuantConfig, Format, ScalingGranularity
from primus_turbo_b200.pytorch.modules import Float8Linear

pytestmark = pytest.mark.gpu


def _cfg(gran, fmt=Format.E4M3):
    if gran == ScalingGranularity.BLOCKWISE:
        return Float8QuantConfig(format=fmt, granularity=gran, block_size=128)
    return Float8QuantConfig(format=fmt, granularity=gran)


@pytest.mark.parametrize("gran", [ScalingGranularity.TENSORWISE, ScalingGranularity.ROWWISE, ScalingGranularity.BLOCKWISE])
@pytest.mark.parametrize("bias", [True, False])
@pytest.mark.parametrize("lead,k,n", [((4, 96), 512, 384), ((256,), 1024, 768)])
def test_float8_linear_matches_bf16_linear(gran, bias, lead, k, n):
    torch.manual_seed(3)
    ref = torch.nn.Linear(k, n, bias=bias, device="cuda", dtype=torch.bfloat16)
    mod = Float8Linear.from_float(ref, _cfg(gran), inplace=False)
    x = torch.randn(*lead, k, device="cuda", dtype=torch.bfloat16)
    x1 = x.clone().requires_grad_(True)
    x2 = x.clone().requires_grad_(True)
    gy = torch.randn(*lead, n, device="cuda", dtype=torch.bfloat16)
    y1 = ref(x1)
    y2 = mod(x2)
    assert y2.shape == y1.shape and y2.dtype == torch.bfloat16
    y1.backward(gy)
    y2.backward(gy)
    assert O.snr_db(y1.detach().float().cpu(), y2.detach().float().cpu()) > 25
    assert O.snr_db(x1.grad.float().cpu(), x2.grad.float().cpu()) > 25
    assert O.snr_db(ref.weight.grad.float().cpu(), mod.weight.grad.float().cpu()) > 25
    if bias:
        assert O.snr_db(ref.bias.grad.float().cpu(), mod.bias.grad.float().cpu()) > 40


def test_float8_linear_hybrid_format_backward_in_e5m2():
    torch.manual_seed(4)
    ref = torch.nn.Linear(512, 256, device="cuda", dtype=torch.bfloat16)
    mod = Float8Linear.from_float(ref, _cfg(ScalingGranularity.TENSORWISE, Format.HYBRID), inplace=False)
    x = torch.randn(128, 512, device="cuda", dtype=torch.bfloat16)
    x1, x2 = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    gy = torch.randn(128, 256, device="cuda", dtype=torch.bfloat16)
    ref(x1).backward(gy)
    mod(x2).backward(gy)
    assert O.snr_db(x1.grad.float().cpu(), x2.grad.float().cpu()) > 20  # e5m2 gradients: 2 mantissa bits
