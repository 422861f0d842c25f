"""GPU: a rank of an expert-parallel job that receives no row at all.

With one local expert per rank and an expert nobody routes to, the grouped path runs on tensors of zero
rows: their data pointers are null, the group offsets are all zero.  The segment quantisers must still
write the padded layout (every group empty), the forward and the activation gradient are empty, and the
weight gradient is exactly zero.  The reference reaches the same state through torch's empty tensors
(its kernels launch over zero blocks).
"""

import pytest
import torch

pytestmark = pytest.mark.gpu

from primus_turbo_b200 import _lib  # noqa: E402
from primus_turbo_b200.pytorch.core.low_precision import Float8QuantConfig, ScaleDtype, ScalingGranularity  # noqa: E402

DEV = "cuda"
E4 = torch.float8_e4m3fn


def _groups(G):
    lens = torch.zeros(G, dtype=torch.int64, device=DEV)
    offs = torch.zeros(G + 1, dtype=torch.int64, device=DEV)
    return lens, offs


@pytest.mark.parametrize("G", [1, 4])
def test_segment_quantiser_without_rows_writes_an_empty_layout(G):
    from primus_turbo_b200.pytorch.kernels.quantization_impl import quant_fp8_blockwise_segment_m_row_col_impl

    lens, offs = _groups(G)
    x = torch.empty((0, 512), dtype=torch.bfloat16, device=DEV)
    q_row, q_col, s_row, s_col, vk_lens, vk_offs = quant_fp8_blockwise_segment_m_row_col_impl(x, E4, 128, lens, offs)
    torch.cuda.synchronize()
    assert q_row.shape == (0, 512) and q_col.shape == (G * 128, 512)
    assert s_row.shape == (4, 0) and s_col.shape == (G, 512)
    assert vk_lens.tolist() == [0] * G and vk_offs.tolist() == [0] * (G + 1)


def test_fused_activation_quantiser_without_rows():
    from primus_turbo_b200.pytorch.ops.activation import swiglu_with_probs_quant_segment

    lens, offs = _groups(2)
    x = torch.empty((0, 1024), dtype=torch.bfloat16, device=DEV)
    probs = torch.empty(0, dtype=torch.float32, device=DEV)
    out = swiglu_with_probs_quant_segment(x, probs, E4, lens, offs)
    torch.cuda.synchronize()
    assert out[0].shape == (0, 512) and out[1].shape == (256, 512)
    assert out[4].tolist() == [0, 0] and out[5].tolist() == [0, 0, 0]


@pytest.mark.parametrize("granularity", [ScalingGranularity.BLOCKWISE, ScalingGranularity.MX_BLOCKWISE])
@pytest.mark.parametrize("G", [1, 2])
def test_grouped_gemm_without_rows_gives_a_zero_weight_gradient(granularity, G):
    from primus_turbo_b200.pytorch.ops import grouped_gemm_fp8

    K, N = 512, 384
    if granularity == ScalingGranularity.BLOCKWISE:
        cfg = Float8QuantConfig(granularity=granularity, block_size=128)
    else:
        cfg = Float8QuantConfig(granularity=granularity, block_size=32, scale_dtype=ScaleDtype.E8M0)
    lens, _ = _groups(G)
    a = torch.empty((0, K), dtype=torch.bfloat16, device=DEV, requires_grad=True)
    w = (torch.randn(G, N, K, device=DEV) * 0.02).to(torch.bfloat16).requires_grad_(True)
    out = grouped_gemm_fp8(a, w, lens, config=cfg)
    assert out.shape == (0, N)
    out.backward(torch.empty((0, N), dtype=torch.bfloat16, device=DEV))
    torch.cuda.synchronize()
    assert _lib.gemm_status() == 0
    assert a.grad.shape == (0, K)
    assert w.grad.shape == w.shape and bool((w.grad == 0).all())
