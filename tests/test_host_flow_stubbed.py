"""CPU: the Python side of the grouped FP8 path with every C-ABI call replaced by a recorder.

What is checked is host logic only -- which entry points a forward + backward of ``grouped_gemm_fp8`` invokes,
in which order, and the shapes it allocates around them -- for ordinary inputs and for the zero-row case (an
expert-parallel rank whose experts received nothing), whose tensors are empty and whose data pointers are
null.  No arithmetic happens here; the numbers are the GPU tests' business.
"""

import contextlib
import sys

import pytest
import torch

from primus_turbo_b200 import _lib
from primus_turbo_b200.pytorch.core.low_precision import Float8QuantConfig, ScaleDtype, ScalingGranularity

E4 = torch.float8_e4m3fn
MODULES = (
    "primus_turbo_b200.pytorch.kernels.quantization_impl",
    "primus_turbo_b200.pytorch.kernels.gemm_impl",
    "primus_turbo_b200.pytorch.ops.activation",
    "primus_turbo_b200.pytorch.ops.grouped_gemm_fp8",
)


@pytest.fixture
def recorded_calls(monkeypatch):
    """Every ``_lib.call`` lands in the returned list as (entry point, arguments); device checks are lifted."""
    import importlib

    for m in MODULES:
        importlib.import_module(m)
    calls = []
    monkeypatch.setattr(_lib, "call", lambda name, *a: calls.append((name, a)))
    monkeypatch.setattr(torch.cuda, "device", lambda d: contextlib.nullcontext())
    for m in MODULES:
        mod = sys.modules[m]
        if hasattr(mod, "require_cuda"):
            monkeypatch.setattr(mod, "require_cuda", lambda *t: None)
        if hasattr(mod, "stream_of"):
            monkeypatch.setattr(mod, "stream_of", lambda t: 0)
    return calls


def _names(calls):
    return [c[0] for c in calls]


@pytest.mark.parametrize("rows", [0, 300])
def test_segment_quantiser_allocations(recorded_calls, rows):
    from primus_turbo_b200.pytorch.kernels.quantization_impl import quant_fp8_blockwise_segment_m_row_col_impl

    G = 3
    lens = torch.tensor([rows, 0, 0], dtype=torch.int64)
    offs = torch.cat([lens.new_zeros(1), lens.cumsum(0)])
    x = torch.empty((rows, 512), dtype=torch.bfloat16)
    q_row, q_col, s_row, s_col, vk_lens, vk_offs = quant_fp8_blockwise_segment_m_row_col_impl(x, E4, 128, lens, offs)
    assert q_row.shape == (rows, 512) and q_col.shape == (rows + G * 128, 512)
    assert s_row.shape == (4, rows) and s_col.shape == ((rows + G * 128 + 127) // 128, 512)
    assert vk_lens.shape == (G,) and vk_offs.shape == (G + 1,)
    (name, args), = recorded_calls
    assert name == "ptb_quant_fp8_segment_row_col"
    # x, M, N, G as the C entry point sees them: an empty x is a null pointer
    assert args[2:5] == (rows, 512, G) and (args[0] == 0) == (rows == 0)


def test_fused_activation_quantiser_allocations_without_rows(recorded_calls):
    from primus_turbo_b200.pytorch.ops.activation import swiglu_with_probs_quant_segment

    lens, offs = torch.zeros(2, dtype=torch.int64), torch.zeros(3, dtype=torch.int64)
    out = swiglu_with_probs_quant_segment(torch.empty((0, 1024), dtype=torch.bfloat16), torch.empty(0), E4, lens, offs)
    assert out[0].shape == (0, 512) and out[1].shape == (256, 512) and out[2].shape == (4, 0)
    assert _names(recorded_calls) == ["ptb_swiglu_quant_fp8_segment_row_col"]


@pytest.mark.parametrize("rows", [0, 200])
@pytest.mark.parametrize("granularity", [ScalingGranularity.BLOCKWISE, ScalingGranularity.MX_BLOCKWISE])
def test_grouped_gemm_call_sequence(recorded_calls, granularity, rows):
    grouped = sys.modules["primus_turbo_b200.pytorch.ops.grouped_gemm_fp8"]
    G, K, N = 2, 512, 384
    if granularity == ScalingGranularity.BLOCKWISE:
        cfg = Float8QuantConfig(granularity=granularity, block_size=128)
        forward = ["ptb_quant_fp8_segment_row_col", "ptb_quant_fp8_block2d", "ptb_grouped_gemm_fp8"]
        backward = ["ptb_quant_fp8_segment_row_col", "ptb_grouped_gemm_fp8", "ptb_grouped_gemm_fp8_variable_k"]
    else:
        cfg = Float8QuantConfig(granularity=granularity, block_size=32, scale_dtype=ScaleDtype.E8M0)
        forward = ["ptb_quant_mxfp8_grouped", "ptb_quant_mxfp8", "ptb_grouped_gemm_mxfp8"]
        backward = ["ptb_quant_mxfp8_grouped", "ptb_grouped_gemm_mxfp8", "ptb_grouped_gemm_mxfp8_variable_k"]
    lens = torch.tensor([rows, 0], dtype=torch.int64)
    a = torch.zeros((rows, K), dtype=torch.bfloat16, requires_grad=True)
    w = torch.zeros((G, N, K), dtype=torch.bfloat16, requires_grad=True)
    offs = torch.cat([lens.new_zeros(1), lens.cumsum(0)])
    out = grouped.grouped_gemm_fp8(a, w, lens, offs, config=cfg)
    assert out.shape == (rows, N) and out.dtype == torch.bfloat16
    assert _names(recorded_calls) == forward
    del recorded_calls[:]
    out.backward(torch.zeros((rows, N), dtype=torch.bfloat16))
    assert _names(recorded_calls) == backward
    assert a.grad.shape == (rows, K) and w.grad.shape == (G, N, K)
