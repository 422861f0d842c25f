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


# ---- MXFP8 payloads in QuantizedTensor ----------------------------------------------------------------------
MX_MODULES = MODULES + ("primus_turbo_b200.pytorch.ops.gemm_fp8",)
MX = ScalingGranularity.MX_BLOCKWISE


def _mx_cfg():
    return Float8QuantConfig(granularity=MX, block_size=32, scale_dtype=ScaleDtype.E8M0)


def test_mx_quantized_tensor_layouts(recorded_calls):
    """Logical shape outside, padded payload inside: axis -1 keeps rows and pads the inner extent to 128, axis -2
    holds the transposed copy; dequantize drops the padding; a view (same number of dimensions) re-splits the leading
    extents of payload and scale bytes alike; ``.t()`` is the other-direction copy of the same logical tensor."""
    from primus_turbo_b200.pytorch.core.low_precision import ScalingRecipe
    from primus_turbo_b200.pytorch.core.quantized_tensor import QuantizedTensor

    x = torch.zeros((96, 160), dtype=torch.bfloat16)
    with pytest.raises(AssertionError, match="scaling_recipe must be provided"):
        QuantizedTensor.quantize(x, E4, MX, axis=-1, block_size=32)
    row = QuantizedTensor.quantize(x, E4, MX, axis=-1, block_size=32, scaling_recipe=ScalingRecipe())
    assert row.shape == (96, 160) and row.qdata.shape == (96, 256) and row.scale_inv.shape == (96, 8)
    assert row.scale_inv.dtype == torch.float8_e8m0fnu and row.quantized_axis == 1
    col = QuantizedTensor.quantize(x, E4, MX, axis=-2, block_size=32, scaling_recipe=ScalingRecipe())
    assert col.shape == (96, 160) and col.qdata.shape == (160, 128) and col.scale_inv.shape == (160, 4)
    assert row.dequantize().shape == (96, 160) and col.dequantize().shape == (96, 160)
    del recorded_calls[:]
    t = row.t()
    assert t.quantized_axis == 0 and t.qdata.shape == (160, 128) and t.shape == (96, 160)
    assert _names(recorded_calls) == ["ptb_dequant_mxfp8", "ptb_quant_mxfp8"]
    w = torch.zeros((3, 64, 128), dtype=torch.bfloat16)
    qw = QuantizedTensor.quantize(w, E4, MX, axis=-1, block_size=32, scaling_recipe=ScalingRecipe(use_2d_block=True))
    assert qw.qdata.shape == (3, 64, 128) and qw.scale_inv.shape == (3, 64, 4)
    v = qw.view(6, 32, 128)  # same number of dimensions, leading extents re-split
    assert v.shape == (6, 32, 128) and v.qdata.shape == (6, 32, 128) and v.scale_inv.shape == (6, 32, 4)
    x3 = QuantizedTensor.quantize(torch.zeros((2, 48, 160), dtype=torch.bfloat16), E4, MX, axis=-1, block_size=32,
                                  scaling_recipe=ScalingRecipe())
    v = x3.reshape(4, 24, 160)  # the payload's inner extent stays padded to 128
    assert v.shape == (4, 24, 160) and v.qdata.shape == (4, 24, 256) and v.scale_inv.shape == (4, 24, 8)
    qw_t = QuantizedTensor.quantize(w, E4, MX, axis=-2, block_size=32, scaling_recipe=ScalingRecipe(use_2d_block=True))
    assert qw_t.qdata.shape == (3, 128, 128) and qw_t.scale_inv.shape == (3, 128, 4)
    assert qw_t.dequantize().shape == (3, 64, 128)


def test_mx_create_quantized_weight(recorded_calls):
    from primus_turbo_b200.pytorch.core.low_precision import ScalingRecipe
    from primus_turbo_b200.pytorch.core.quantized_tensor import create_quantized_weight

    w = torch.zeros((256, 512), dtype=torch.bfloat16, requires_grad=True)
    qw, qw_t = create_quantized_weight(w, E4, _mx_cfg(), need_weight_transpose_cache=True)
    assert qw.scaling_recipe == ScalingRecipe(use_2d_block=True) == qw_t.scaling_recipe
    assert qw.quantized_axis == 1 and qw_t.quantized_axis == 0
    assert qw.qdata.shape == (256, 512) and qw_t.qdata.shape == (512, 256)
    # both copies are 32x32-tile quantisations: the 2-D flag is argument 9 (row) / 10 (column) of the entry point
    assert [(c[0], c[1][9], c[1][10]) for c in recorded_calls] == [("ptb_quant_mxfp8", 1, 1)] * 2


@pytest.mark.parametrize("with_transposed", [False, True])
def test_mx_gemm_with_quantized_operands(monkeypatch, recorded_calls, with_transposed):
    """Pre-quantised operands bring their row copies; the column copies come from the pair's second member or from
    a dequantise -> re-quantise along the other axis (the reference's schedule)."""
    from primus_turbo_b200.pytorch.core.low_precision import ScalingRecipe
    from primus_turbo_b200.pytorch.core.quantized_tensor import QuantizedTensor, QuantizedTensorPair

    import importlib

    gemm = importlib.import_module("primus_turbo_b200.pytorch.ops.gemm_fp8")
    impl = sys.modules["primus_turbo_b200.pytorch.kernels.gemm_impl"]
    for mod in (gemm, impl):
        for n in ("require_cuda", "stream_of"):
            if hasattr(mod, n):
                monkeypatch.setattr(mod, n, (lambda *t: None) if n == "require_cuda" else (lambda t: 0))
    M, N, K = 256, 352, 160
    a = torch.zeros((M, K), dtype=torch.bfloat16, requires_grad=True)
    b = torch.zeros((N, K), dtype=torch.bfloat16, requires_grad=True)
    ra, rb = ScalingRecipe(), ScalingRecipe(use_2d_block=True)
    qa = QuantizedTensor.quantize(a, E4, MX, axis=-1, block_size=32, scaling_recipe=ra)
    qb = QuantizedTensor.quantize(b, E4, MX, axis=-1, block_size=32, scaling_recipe=rb)
    qa_t = QuantizedTensor.quantize(a, E4, MX, axis=-2, block_size=32, scaling_recipe=ra) if with_transposed else None
    qb_t = QuantizedTensor.quantize(b, E4, MX, axis=-2, block_size=32, scaling_recipe=rb) if with_transposed else None
    del recorded_calls[:]
    out = gemm.gemm_fp8(QuantizedTensorPair(qa, qa_t), QuantizedTensorPair(qb, qb_t), False, True, torch.bfloat16, _mx_cfg())
    assert out.shape == (M, N)
    requant = [] if with_transposed else ["ptb_dequant_mxfp8", "ptb_quant_mxfp8"] * 2
    assert _names(recorded_calls) == requant + ["ptb_gemm_mxfp8"]
    del recorded_calls[:]
    out.backward(torch.zeros((M, N), dtype=torch.bfloat16))
    assert _names(recorded_calls) == ["ptb_quant_mxfp8", "ptb_gemm_mxfp8", "ptb_gemm_mxfp8"]
    assert qa.grad.shape == (M, K) and qb.grad.shape == (N, K)
    # a row-direction operand handed over as the column copy is refused
    with pytest.raises(AssertionError, match="quantized_axis"):
        gemm.gemm_fp8(QuantizedTensorPair(qa, qa), QuantizedTensorPair(qb, qb_t), False, True, torch.bfloat16, _mx_cfg())


def test_mx_grouped_gemm_with_quantized_weight(recorded_calls):
    from primus_turbo_b200.pytorch.core.quantized_tensor import QuantizedTensorPair, create_quantized_weight

    grouped = sys.modules["primus_turbo_b200.pytorch.ops.grouped_gemm_fp8"]
    G, K, N, rows = 2, 512, 384, 200
    w = torch.zeros((G, N, K), dtype=torch.bfloat16, requires_grad=True)
    qw, qw_t = create_quantized_weight(w, E4, _mx_cfg(), need_weight_transpose_cache=True)
    lens = torch.tensor([rows, 0], dtype=torch.int64)
    offs = torch.cat([lens.new_zeros(1), lens.cumsum(0)])
    a = torch.zeros((rows, K), dtype=torch.bfloat16, requires_grad=True)
    del recorded_calls[:]
    out = grouped.grouped_gemm_fp8(a, QuantizedTensorPair(qw, qw_t), lens, offs, config=_mx_cfg())
    assert out.shape == (rows, N)
    assert _names(recorded_calls) == ["ptb_quant_mxfp8_grouped", "ptb_grouped_gemm_mxfp8"]
    del recorded_calls[:]
    out.backward(torch.zeros((rows, N), dtype=torch.bfloat16))
    assert _names(recorded_calls) == ["ptb_quant_mxfp8_grouped", "ptb_grouped_gemm_mxfp8", "ptb_grouped_gemm_mxfp8_variable_k"]
    assert a.grad.shape == (rows, K) and qw.grad.shape == (G, N, K)


# ---- grouped MX activations -----------------------------------------------------------------------------------
def _emulate_group_layout(calls):
    """Stand-in for the layout kernel of ``ptb_quant_mxfp8_grouped``: reads the group offsets and writes the
    padded lengths / offsets of both layouts through the (host) pointers the call was given."""
    import ctypes

    def at(ptr, n):
        return (ctypes.c_int64 * n).from_address(ptr)

    name, a = calls[-1]
    assert name == "ptb_quant_mxfp8_grouped"
    G, row_align = a[5], a[6]
    offs = list(at(a[4], G + 1))
    for lens_ptr, offs_ptr, align in ((a[11], a[12], row_align), (a[13], a[14], 128)):
        run = 0
        for g in range(G):
            padded = -(-(offs[g + 1] - offs[g]) // align) * align
            at(lens_ptr, G)[g] = padded
            at(offs_ptr, G + 1)[g] = run
            run += padded
        at(offs_ptr, G + 1)[G] = run


def test_packed_row_index():
    from primus_turbo_b200.pytorch.kernels.quantization_impl import packed_row_index

    offs = torch.tensor([0, 100, 100, 257, 300])
    padded = torch.tensor([0, 128, 128, 288, 352])  # groups padded to 32 rows
    idx = packed_row_index(offs, padded, 300).tolist()
    want = list(range(0, 100)) + list(range(128, 128 + 157)) + list(range(288, 288 + 43))
    assert idx == want
    # rows past the last group stay inside the padded layout
    assert packed_row_index(offs, padded, 304).tolist()[-4:] == [331, 332, 333, 334]


def test_mx_grouped_activation_as_quantized_tensor(monkeypatch, recorded_calls):
    """A grouped activation quantised ahead of time: padded layouts inside, packed rows outside; the grouped GEMM
    runs over the padded row copy and gathers the rows that exist."""
    from primus_turbo_b200.pytorch.core.low_precision import ScalingRecipe
    from primus_turbo_b200.pytorch.core.quantized_tensor import QuantizedTensor, QuantizedTensorPair

    gemm_impl = sys.modules["primus_turbo_b200.pytorch.kernels.gemm_impl"]
    grouped = sys.modules["primus_turbo_b200.pytorch.ops.grouped_gemm_fp8"]
    qt_mod = sys.modules["primus_turbo_b200.pytorch.core.quantized_tensor"]
    offsets = lambda lens: torch.cat([lens.new_zeros(1), lens.cumsum(0)])  # noqa: E731
    monkeypatch.setattr(gemm_impl, "group_offs_from_lens", offsets)
    monkeypatch.setattr(grouped, "group_offs_from_lens", offsets)

    def call(name, *a):
        recorded_calls.append((name, a))
        if name == "ptb_quant_mxfp8_grouped":
            _emulate_group_layout(recorded_calls)

    monkeypatch.setattr(_lib, "call", call)
    # the group tensors live on the host here
    monkeypatch.setattr(torch.Tensor, "is_cuda", property(lambda self: True))
    G, K, N = 4, 160, 96
    lens = torch.tensor([100, 0, 157, 43], dtype=torch.int64)
    M = int(lens.sum())
    a = torch.zeros((M, K), dtype=torch.bfloat16, requires_grad=True)
    w = torch.zeros((G, N, K), dtype=torch.bfloat16, requires_grad=True)
    qa = QuantizedTensor.quantize(a, E4, MX, axis=-1, block_size=32, scaling_recipe=ScalingRecipe(), group_lens=lens)
    assert qa.shape == (M, K) and qa._is_grouped_tensor
    assert qa.qdata.shape == (448, 256) and qa.scale_inv.shape == (448, 8)  # ceil((300 + 4*32) / 32) * 32 rows
    assert qa.group_lens.tolist() == [128, 0, 160, 64] and qa.group_offs.tolist() == [0, 128, 128, 288, 352]
    assert qa._orig_group_offs.tolist() == [0, 100, 100, 257, 300]
    qa_t = QuantizedTensor.quantize(a, E4, MX, axis=-2, block_size=32, scaling_recipe=ScalingRecipe(), group_lens=lens)
    assert qa_t.qdata.shape == (K, 896) and qa_t.group_offs.tolist() == [0, 128, 128, 384, 512]
    assert qa.dequantize().shape == (M, K) and qa_t.dequantize().shape == (M, K)
    del recorded_calls[:]
    out = grouped.grouped_gemm_fp8(QuantizedTensorPair(qa, None), w, lens, config=_mx_cfg())
    assert out.shape == (M, N)
    assert _names(recorded_calls) == ["ptb_dequant_mxfp8", "ptb_quant_mxfp8_grouped", "ptb_quant_mxfp8",
                                      "ptb_grouped_gemm_mxfp8"]
    gemm_args = recorded_calls[-1][1]
    assert gemm_args[13] == 448, "the GEMM runs over the padded row layout"
    del recorded_calls[:]
    out.backward(torch.zeros((M, N), dtype=torch.bfloat16))
    assert _names(recorded_calls) == ["ptb_quant_mxfp8_grouped", "ptb_grouped_gemm_mxfp8", "ptb_grouped_gemm_mxfp8_variable_k"]
    assert recorded_calls[1][1][13] == M, "dgrad runs over the packed rows"
    assert qa.grad.shape == (M, K) and w.grad.shape == (G, N, K)


@pytest.mark.parametrize("granularity", [ScalingGranularity.TENSORWISE, ScalingGranularity.ROWWISE])
def test_grouped_gemm_tensorwise_rowwise_with_quantized_operands(monkeypatch, recorded_calls, granularity):
    """A grouped activation and a weight quantised ahead of time skip exactly their own quantisation."""
    from primus_turbo_b200.pytorch.core.quantized_tensor import QuantizedTensor

    gemm_impl = sys.modules["primus_turbo_b200.pytorch.kernels.gemm_impl"]
    grouped = sys.modules["primus_turbo_b200.pytorch.ops.grouped_gemm_fp8"]
    import importlib

    custom = importlib.import_module("primus_turbo_b200.pytorch.kernels.custom_ops")
    offsets = lambda lens: torch.cat([lens.new_zeros(1), lens.cumsum(0)])  # noqa: E731
    for mod in (gemm_impl, grouped, custom):
        if hasattr(mod, "group_offs_from_lens"):
            monkeypatch.setattr(mod, "group_offs_from_lens", offsets)
    monkeypatch.setattr(torch.Tensor, "is_cuda", property(lambda self: True))
    G, K, N, rows = 2, 256, 384, 200
    lens = torch.tensor([rows, 0], dtype=torch.int64)
    cfg = Float8QuantConfig(granularity=granularity)

    def sequence(a_op, w_op):
        del recorded_calls[:]
        out = grouped.grouped_gemm_fp8(a_op, w_op, lens, config=cfg)
        fwd = _names(recorded_calls)
        del recorded_calls[:]
        out.backward(torch.zeros((rows, N), dtype=torch.bfloat16))
        return out, fwd, _names(recorded_calls)

    a = torch.zeros((rows, K), dtype=torch.bfloat16, requires_grad=True)
    w = torch.zeros((G, N, K), dtype=torch.bfloat16, requires_grad=True)
    out, fwd_raw, bwd_raw = sequence(a, w)
    assert out.shape == (rows, N)
    qa = QuantizedTensor.quantize(a.detach().clone().requires_grad_(), E4, granularity, axis=-1, group_lens=lens)
    qw = QuantizedTensor.quantize(w.detach().clone().requires_grad_(), E4, granularity, axis=-1)
    assert qa._is_grouped_tensor and qa.group_offs.tolist() == [0, rows, rows]
    out, fwd_q, bwd_q = sequence(qa, qw)
    assert out.shape == (rows, N) and qa.grad.shape == (rows, K) and qw.grad.shape == (G, N, K)
    # forward: the two operand quantisations are gone, everything after them is unchanged
    assert fwd_raw[:2] == [fwd_raw[0]] * 2 and fwd_raw[0].startswith("ptb_quant_fp8_")
    assert fwd_q == fwd_raw[2:] and fwd_q[0] == "ptb_grouped_gemm_fp8"
    assert bwd_q == bwd_raw
