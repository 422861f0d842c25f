"""GPU: MXFP8 payloads inside ``QuantizedTensor`` and as pre-quantised operands of the MX GEMMs.

The reference's checks for this (tests/pytorch/core/test_quantized_tensor.py, tests/pytorch/ops/test_gemm_fp8.py:
348-470,513-545, tests/pytorch/ops/test_grouped_gemm_fp8.py:778-860) are a dequantise round trip and an SNR gate
against the high-precision product.  Here the row copies are also compared byte for byte with the plain
quantise op, and a GEMM whose operands bring both of their copies must equal the raw-tensor GEMM bit for bit
(same payloads, same kernel).
"""

import pytest
import torch

from oracle import fp8_oracle as O
from primus_turbo_b200 import _lib
from primus_turbo_b200.pytorch.core.low_precision import (
    Float8QuantConfig,
    Format,
    ScaleDtype,
    ScalingGranularity,
    ScalingRecipe,
)
from primus_turbo_b200.pytorch.core.quantized_tensor import QuantizedTensor, QuantizedTensorPair, create_quantized_weight
from primus_turbo_b200.pytorch.ops import gemm_fp8, grouped_gemm_fp8, quantize_fp8

pytestmark = pytest.mark.gpu
MX = ScalingGranularity.MX_BLOCKWISE
DEV = "cuda"
E4 = torch.float8_e4m3fn


def _mk(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(torch.bfloat16).to(DEV)


def _same_bytes(a, b):
    return a.shape == b.shape and torch.equal(a.contiguous().view(torch.uint8), b.contiguous().view(torch.uint8))


def _cfg(fmt=Format.E4M3):
    return Float8QuantConfig(format=fmt, granularity=MX, block_size=32, scale_dtype=ScaleDtype.E8M0)


@pytest.mark.parametrize("shape", [(96, 160), (256, 512), (3, 64, 128)])
@pytest.mark.parametrize("use_2d", [False, True])
def test_payload_matches_the_plain_op_and_round_trips(shape, use_2d):
    x = _mk(shape, seed=sum(shape))
    recipe = ScalingRecipe(use_2d_block=use_2d)
    nd = len(shape)
    for axis in (-1, -2):
        qt = QuantizedTensor.quantize(x, E4, MX, axis=axis, block_size=32, scaling_recipe=recipe)
        q, s = quantize_fp8(x, E4, MX, block_size=32, axis=axis + nd, scaling_recipe=recipe)
        assert qt.shape == x.shape and qt.dtype == x.dtype
        assert _same_bytes(qt.qdata, q) and _same_bytes(qt.scale_inv, s)
        back = qt.dequantize()
        assert back.shape == x.shape and back.dtype == x.dtype
        # one e4m3 rounding of a value scaled into the block's binade: relative error <= 2^-4 of the block maximum
        assert O.rel_frobenius(x.float().cpu(), back.float().cpu()) <= 0.04
    t = QuantizedTensor.quantize(x, E4, MX, axis=-1, block_size=32, scaling_recipe=recipe).transpose(-2, -1)
    assert t.quantized_axis == nd - 2 and t.qdata.shape[-2] == shape[-1]


@pytest.mark.parametrize("fmt", [Format.E4M3, Format.HYBRID])
@pytest.mark.parametrize("mnk", [(256, 352, 160), (512, 1024, 1024)])
def test_gemm_with_pre_quantised_operands(fmt, mnk):
    M, N, K = mnk
    cfg = _cfg(fmt)
    a, b, gy = _mk((M, K), 1), _mk((N, K), 2, 0.05), _mk((M, N), 3, 0.01)
    ra, rb = ScalingRecipe(), ScalingRecipe(use_2d_block=True)

    def run(a_op, b_op, a_leaf, b_leaf):
        out = gemm_fp8(a_op, b_op, False, True, torch.bfloat16, cfg)
        out.backward(gy)
        return out.detach(), a_leaf.grad, b_leaf.grad

    a0, b0 = a.clone().requires_grad_(), b.clone().requires_grad_()
    ref = run(a0, b0, a0, b0)
    # both copies handed over: the same payloads reach the same kernels
    a1, b1 = a.clone().requires_grad_(), b.clone().requires_grad_()
    qa, qa_t = (QuantizedTensor.quantize(a1, E4, MX, axis=ax, block_size=32, scaling_recipe=ra) for ax in (-1, -2))
    qb, qb_t = create_quantized_weight(b1, E4, cfg, need_weight_transpose_cache=True)
    got = run(QuantizedTensorPair(qa, qa_t), QuantizedTensorPair(qb, qb_t), qa, qb)
    assert _lib.gemm_status() == 0
    for r, g in zip(ref, got):
        assert torch.equal(r, g)
    # row copies only: the column copies are re-quantised from the dequantised row copies (the reference's
    # schedule), so the forward is still identical and the gradients pass the reference's SNR gate
    qa2 = QuantizedTensor.quantize(a.clone().requires_grad_(), E4, MX, axis=-1, block_size=32, scaling_recipe=ra)
    qb2 = QuantizedTensor.quantize(b.clone().requires_grad_(), E4, MX, axis=-1, block_size=32, scaling_recipe=rb)
    got2 = run(QuantizedTensorPair(qa2, None), QuantizedTensorPair(qb2, None), qa2, qb2)
    assert _lib.gemm_status() == 0
    assert torch.equal(ref[0], got2[0])
    ga = gy.float() @ b.float()
    gb = gy.float().t() @ a.float()
    floor = 20 if fmt == Format.HYBRID else 25
    assert O.snr_db(ga.cpu(), got2[1].float().cpu()) > floor - 5
    assert O.snr_db(gb.cpu(), got2[2].float().cpu()) > floor - 5


def test_grouped_gemm_with_pre_quantised_weight():
    G, K, N = 4, 128, 256  # shapes the raw-tensor grouped MX tests cover
    lens = torch.tensor([100, 0, 157, 43], dtype=torch.int64, device=DEV)
    rows = int(lens.sum())
    cfg = _cfg()
    a, w, gy = _mk((rows, K), 4), _mk((G, N, K), 5, 0.05), _mk((rows, N), 6, 0.01)

    def run(a_leaf, w_op, w_leaf):
        out = grouped_gemm_fp8(a_leaf, w_op, lens, config=cfg)
        out.backward(gy)
        return out.detach(), a_leaf.grad, w_leaf.grad

    a0, w0 = a.clone().requires_grad_(), w.clone().requires_grad_()
    ref = run(a0, w0, w0)
    a1 = a.clone().requires_grad_()
    qw, qw_t = create_quantized_weight(w.clone().requires_grad_(), E4, cfg, need_weight_transpose_cache=True)
    got = run(a1, QuantizedTensorPair(qw, qw_t), qw)
    assert _lib.gemm_status() == 0
    for r, g in zip(ref, got):
        assert torch.equal(r, g)
    with pytest.raises(AssertionError, match="grouped tensor"):
        qa = QuantizedTensor.quantize(a, E4, MX, axis=-1, block_size=32, scaling_recipe=ScalingRecipe())
        grouped_gemm_fp8(qa, w, lens, config=cfg)


def test_grouped_activation_as_quantized_tensor():
    """The reference's grouped MX activation tensor (row copy padded to 32 rows per group, transposed column copy
    padded to 128): layout metadata, round trip, and the grouped GEMM over it against the raw-tensor call."""
    G, K, N = 4, 96, 320  # shapes the raw-tensor grouped MX tests cover
    lens_host = [100, 0, 157, 43]
    lens = torch.tensor(lens_host, dtype=torch.int64, device=DEV)
    M = sum(lens_host)
    cfg = _cfg()
    a, w, gy = _mk((M, K), 7), _mk((G, N, K), 8, 0.05), _mk((M, N), 9, 0.01)
    a1 = a.clone().requires_grad_()
    qa = QuantizedTensor.quantize(a1, E4, MX, axis=-1, block_size=32, scaling_recipe=ScalingRecipe(), group_lens=lens)
    qa_t = QuantizedTensor.quantize(a1, E4, MX, axis=-2, block_size=32, scaling_recipe=ScalingRecipe(), group_lens=lens)
    assert qa.shape == (M, K) and qa.qdata.shape == (448, 128)
    assert qa.group_lens.tolist() == [128, 0, 160, 64] and qa.group_offs.tolist() == [0, 128, 128, 288, 352]
    assert qa_t.qdata.shape == (K, 896) and qa_t.group_offs.tolist() == [0, 128, 128, 384, 512]
    for t in (qa, qa_t):
        back = t.dequantize()
        assert back.shape == (M, K)
        assert O.rel_frobenius(a.float().cpu(), back.float().cpu()) <= 0.04

    def run(a_op, a_leaf, w_leaf):
        out = grouped_gemm_fp8(a_op, w_leaf, lens, config=cfg)
        out.backward(gy)
        return out.detach(), a_leaf.grad, w_leaf.grad

    a0, w0 = a.clone().requires_grad_(), w.clone().requires_grad_()
    ref = run(a0, a0, w0)
    w1 = w.clone().requires_grad_()
    got = run(QuantizedTensorPair(qa, qa_t), qa, w1)
    assert _lib.gemm_status() == 0
    for r, g in zip(ref, got):  # same bytes per row and per column block reach the same kernels
        assert torch.equal(r, g)
    # without the column copy it is re-quantised from the dequantised rows: same forward, gated weight gradient
    qa2 = QuantizedTensor.quantize(a.clone().requires_grad_(), E4, MX, axis=-1, block_size=32,
                                   scaling_recipe=ScalingRecipe(), group_lens=lens)
    w2 = w.clone().requires_grad_()
    got2 = run(QuantizedTensorPair(qa2, None), qa2, w2)
    assert _lib.gemm_status() == 0
    assert torch.equal(ref[0], got2[0]) and torch.equal(ref[1], got2[1])
    assert O.rel_frobenius(ref[2].float().cpu(), got2[2].float().cpu()) <= 0.05


@pytest.mark.parametrize("granularity", [ScalingGranularity.TENSORWISE, ScalingGranularity.ROWWISE])
def test_grouped_gemm_tensorwise_rowwise_with_pre_quantised_operands(granularity):
    """The reference's ``test_grouped_gemm_fp8_{tensorwise,rowwise}_quantized_tensor``: a grouped activation and a
    weight quantised ahead of time go through the code the raw tensors take after their own quantisation, so the
    three results are the raw-tensor call's bit for bit."""
    G, K, N = 4, 256, 384
    lens = torch.tensor([100, 0, 157, 43], dtype=torch.int64, device=DEV)
    rows = int(lens.sum())
    cfg = Float8QuantConfig(granularity=granularity)
    a, w, gy = _mk((rows, K), 10), _mk((G, N, K), 11, 0.05), _mk((rows, N), 12, 0.01)

    def run(a_op, w_op, a_leaf, w_leaf):
        out = grouped_gemm_fp8(a_op, w_op, lens, config=cfg)
        out.backward(gy)
        return out.detach(), a_leaf.grad, w_leaf.grad

    a0, w0 = a.clone().requires_grad_(), w.clone().requires_grad_()
    ref = run(a0, w0, a0, w0)
    qa = QuantizedTensor.quantize(a.clone().requires_grad_(), E4, granularity, axis=-1, group_lens=lens)
    qw = QuantizedTensor.quantize(w.clone().requires_grad_(), E4, granularity, axis=-1)
    got = run(qa, qw, qa, qw)
    assert _lib.gemm_status() == 0
    for r, g in zip(ref, got):
        assert torch.equal(r, g)
    hp = torch.cat([a[o : o + n].float() @ w[i].float().t() for i, (o, n) in enumerate(zip([0, 100, 100, 257], [100, 0, 157, 43]))])
    assert O.snr_db(hp.cpu(), got[0].float().cpu()) > 25


def test_grouped_gemm_replays_from_a_cuda_graph_with_new_group_lens():
    """The reference's (currently skipped) graph tests, tests/pytorch/ops/test_grouped_gemm_fp8.py:802-929: forward
    and backward captured once, replayed after ``group_lens`` was rewritten in place.  Nothing on the host
    depends on the group lengths (offsets, padded layouts and tile schedules are computed on the device), so the
    replay must give exactly what an eager call with the new lengths gives."""
    G, K, N, M = 4, 512, 384, 1024
    cfg = Float8QuantConfig(granularity=ScalingGranularity.BLOCKWISE, block_size=128)
    a, w, gy = _mk((M, K), 13).requires_grad_(), _mk((G, N, K), 14, 0.05).requires_grad_(), _mk((M, N), 15, 0.01)
    first, second = [300, 0, 500, 224], [256, 256, 256, 256]
    lens = torch.tensor(first, dtype=torch.int64, device=DEV)

    def step(group_lens):
        out = grouped_gemm_fp8(a, w, group_lens, config=cfg)
        return (out,) + torch.autograd.grad(out, (a, w), gy)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):  # warm-up outside the capture: one-time kernel attributes, allocator pools
        for _ in range(2):
            step(lens)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = step(lens)
    for values in (first, second, first):
        lens.copy_(torch.tensor(values, dtype=torch.int64, device=DEV))
        graph.replay()
        torch.cuda.synchronize()
        got = [t.clone() for t in captured]
        want = step(torch.tensor(values, dtype=torch.int64, device=DEV))
        torch.cuda.synchronize()
        assert _lib.gemm_status() == 0
        for g, e in zip(got, want):
            assert torch.equal(g, e)


def test_drop_and_pad_routing_on_the_device():
    """Capacity-padded routing is a chain of torch ops (as in the reference): the device result must be the host's."""
    from primus_turbo_b200.pytorch.ops.moe.permutation import capacity_indices, token_permute, token_unpermute

    g = torch.Generator().manual_seed(0)
    T, E, H, capacity = 300, 8, 64, 20
    routing = torch.rand(T, E, generator=g) < 0.1
    probs = torch.rand(T, E, generator=g)
    x = torch.randn(T, H, generator=g)
    rows, slot_probs, sorted_indices, tpe = token_permute(
        x.to(DEV), E * capacity, probs=probs.to(DEV), routing_map=routing.to(DEV), drop_and_pad=True)
    want = capacity_indices(routing, capacity)
    assert torch.equal(sorted_indices.cpu(), want) and tpe.cpu().tolist() == routing.sum(0).tolist()
    assert torch.equal(rows.cpu(), x[want])
    back = token_unpermute(rows, sorted_indices, merging_probs=probs.to(DEV), restore_shape=(T, H),
                           routing_map=routing.to(DEV), drop_and_pad=True)
    ref = torch.zeros(T, H).index_add_(0, want, x[want] * slot_probs.cpu().unsqueeze(1))
    torch.testing.assert_close(back.cpu(), ref, rtol=1e-5, atol=1e-5)
