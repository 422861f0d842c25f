"""CPU: config / enum semantics and the backend-manager shim of the ops surface."""

import pytest
import torch

from primus_turbo_b200.pytorch.core.backend import BackendType, GlobalBackendManager, PrecisionType
from primus_turbo_b200.pytorch.core.low_precision import (
    Float8QuantConfig,
    Format,
    ScaleDtype,
    ScalingGranularity,
    ScalingRecipe,
    float8_e4m3,
    float8_e5m2,
)


def test_enum_values_match_c_abi():
    from primus_turbo_b200 import _lib

    assert ScalingGranularity.TENSORWISE.value == _lib.PTB_TENSORWISE
    assert ScalingGranularity.ROWWISE.value == _lib.PTB_ROWWISE
    assert ScalingGranularity.BLOCKWISE.value == _lib.PTB_BLOCKWISE
    assert float8_e4m3 is torch.float8_e4m3fn and float8_e5m2 is torch.float8_e5m2


def test_config_defaults_and_asserts():
    c = Float8QuantConfig()
    assert c.format == Format.E4M3 and c.granularity == ScalingGranularity.TENSORWISE and c.block_size is None
    with pytest.raises(AssertionError):
        Float8QuantConfig(granularity=ScalingGranularity.BLOCKWISE)
    Float8QuantConfig(granularity=ScalingGranularity.BLOCKWISE, block_size=128)
    with pytest.raises(AssertionError):
        Float8QuantConfig(granularity=ScalingGranularity.MX_BLOCKWISE, block_size=32, scale_dtype=ScaleDtype.FP32)
    assert ScalingRecipe().use_2d_block is False and ScalingRecipe(use_2d_block=True).use_2d_block


def test_backend_manager_shim_records_and_resets(monkeypatch):
    GlobalBackendManager.reset()
    assert GlobalBackendManager.get_gemm_backend(PrecisionType.FP8) is None
    GlobalBackendManager.set_gemm_backend(BackendType.TRITON)
    GlobalBackendManager.set_grouped_gemm_backend(BackendType.CK, PrecisionType.FP8)
    assert GlobalBackendManager.get_gemm_backend(PrecisionType.FP8) == BackendType.TRITON
    assert GlobalBackendManager.get_grouped_gemm_backend(PrecisionType.FP8) == BackendType.CK
    GlobalBackendManager.set_auto_tune(True)
    assert GlobalBackendManager.auto_tune_enabled()
    GlobalBackendManager.reset()
    assert GlobalBackendManager.get_gemm_backend() is None and not GlobalBackendManager.auto_tune_enabled()
    monkeypatch.setenv("PRIMUS_TURBO_GEMM_BACKEND", "hipblaslt")
    assert GlobalBackendManager.get_gemm_backend() == BackendType.HIPBLASLT


def test_drop_in_alias():
    import primus_turbo_b200

    primus_turbo_b200.install_as_primus_turbo()
    import primus_turbo.pytorch as turbo
    from primus_turbo.pytorch.core.low_precision import Float8QuantConfig as C2
    from primus_turbo.pytorch.ops import gemm_fp8, grouped_gemm_fp8, quantize_fp8  # noqa: F401

    assert C2 is Float8QuantConfig and turbo.float8_e4m3 is torch.float8_e4m3fn


def test_float8_linear_conversion_mechanics():
    """Construction and ``from_float`` (in place and copying) need no GPU; the forward does."""
    from primus_turbo_b200.pytorch.modules import Float8Linear

    lin = torch.nn.Linear(16, 8, bias=True)
    w0, b0 = lin.weight.detach().clone(), lin.bias.detach().clone()
    cfg = Float8QuantConfig(granularity=ScalingGranularity.BLOCKWISE, block_size=128)
    copy = Float8Linear.from_float(lin, cfg, inplace=False)
    assert type(lin) is torch.nn.Linear and isinstance(copy, Float8Linear) and copy.config is cfg
    assert torch.equal(copy.weight, w0) and torch.equal(copy.bias, b0) and copy.weight is not lin.weight
    same = Float8Linear.from_float(lin)
    assert same is lin and isinstance(lin, Float8Linear)
    assert lin.config.granularity == ScalingGranularity.TENSORWISE
    assert "config=" in repr(lin)
    nb = Float8Linear(4, 4, bias=False)
    assert nb.bias is None and nb.config.granularity == ScalingGranularity.TENSORWISE
    with pytest.raises(AssertionError):
        Float8Linear.from_float(torch.nn.ReLU())


def _cpu_qt(shape=(4, 6), gran=None, requires_grad=False):
    import torch

    from primus_turbo_b200.pytorch.core.low_precision import ScalingGranularity
    from primus_turbo_b200.pytorch.core.quantized_tensor import QuantizedTensor

    data = torch.arange(shape[0] * shape[1], dtype=torch.uint8).reshape(shape).view(torch.float8_e4m3fn)
    return QuantizedTensor(
        data, torch.full((), 0.5), shape=data.shape, orig_dtype=torch.bfloat16, dest_dtype=torch.float8_e4m3fn,
        granularity=gran or ScalingGranularity.TENSORWISE, quantized_axis=-1, requires_grad=requires_grad,
    )


def test_quantized_tensor_view_and_reshape_keep_payload_and_metadata():
    """view / reshape move the FP8 payload without dequantising, keep the scale and the wrapper's
    metadata, and send the gradient back in the original shape
    (primus_turbo/pytorch/core/quantized_tensor.py:700-740,838-881)."""
    import torch

    from primus_turbo_b200.pytorch.core.quantized_tensor import QuantizedTensor

    q = _cpu_qt(requires_grad=True)
    for v in (q.view(6, 4), q.view((3, 8)), q.reshape(-1, 12), q.reshape(2, -1)):
        assert isinstance(v, QuantizedTensor) and v.qdata.shape == v.shape and v.numel() == 24
        assert torch.equal(v.qdata.view(torch.uint8).reshape(-1), q.qdata.view(torch.uint8).reshape(-1))
        assert v.scale_inv is q.scale_inv and v.granularity == q.granularity and v.real_dtype == q.real_dtype
        assert v.dtype == torch.bfloat16 and v.quantized_axis == q.quantized_axis
    same = q.view(4, 6)
    assert same.qdata.data_ptr() == q.qdata.data_ptr()
    v = q.view(6, 4)
    assert v.grad_fn is not None
    (gin,) = v.grad_fn.apply(torch.ones(6, 4))[:1]
    assert gin.shape == (4, 6)
    import pytest

    with pytest.raises(AssertionError):
        q.view(24)  # the number of dimensions is kept, as in the reference


def test_quantized_tensor_flatten_unflatten_round_trip():
    """__tensor_flatten__ / __tensor_unflatten__ (what torch.compile and FSDP use to take the wrapper
    apart and rebuild it) reproduce payload, scales and every piece of metadata."""
    import torch

    from primus_turbo_b200.pytorch.core.low_precision import ScalingGranularity, ScalingRecipe
    from primus_turbo_b200.pytorch.core.quantized_tensor import QuantizedTensor

    data = torch.zeros(8, 16, dtype=torch.float8_e5m2)
    lens = torch.tensor([3, 5])
    offs = torch.tensor([0, 3, 8])
    q = QuantizedTensor(
        data, torch.ones(8, 1), shape=data.shape, orig_dtype=torch.float16, dest_dtype=torch.float8_e5m2,
        granularity=ScalingGranularity.ROWWISE, block_size=None, scaling_recipe=ScalingRecipe(), quantized_axis=-1,
        group_lens=lens, group_offs=offs, orig_group_lens=lens, orig_group_offs=offs, is_grouped_tensor=True,
    )
    names, meta = q.__tensor_flatten__()
    assert names[:2] == ["_data", "_scale_inv"] and set(names[2:]) == {
        "_orig_group_lens", "_orig_group_offs", "_group_lens", "_group_offs"}
    r = QuantizedTensor.__tensor_unflatten__({n: getattr(q, n) for n in names}, meta, q.shape, q.stride())
    assert r.shape == q.shape and r.dtype == torch.float16 and r.real_dtype == torch.float8_e5m2
    assert r.granularity == ScalingGranularity.ROWWISE and r.quantized_axis == r.qdata.ndim - 1 and r._is_grouped_tensor
    assert r.qdata is q.qdata and r.scale_inv is q.scale_inv and r.group_lens is lens and r.group_offs is offs
    plain = _cpu_qt()
    names, meta = plain.__tensor_flatten__()
    assert names == ["_data", "_scale_inv"]
    r = QuantizedTensor.__tensor_unflatten__({n: getattr(plain, n) for n in names}, meta, plain.shape, None)
    assert r.group_lens is None and not r._is_grouped_tensor


def test_logger_level_once_and_rank_filters(capsys):
    """PRIMUS_TURBO_LOG_LEVEL-style logger (primus_turbo/common/logger.py:29-130): once= and rank= filters."""
    import logging

    from primus_turbo_b200.common import logger

    logger.set_level(logging.INFO)
    logger.info("hello %d", 1)
    logger.info("only once", once=True)
    logger.info("only once", once=True)
    logger.info("other rank", rank=3)
    logger.debug("below the level")
    err = capsys.readouterr().err
    assert err.count("hello 1") == 1 and err.count("only once") == 1
    assert "other rank" not in err and "below the level" not in err
    logger.set_level(logging.WARNING)


def test_drop_and_pad_routing_matches_a_slot_by_slot_evaluation(monkeypatch):
    """Capacity-padded routing (primus_turbo/pytorch/ops/moe/permutation.py:332-349,408-436 in the reference) is
    a chain of torch ops there and here, so it can be checked on the CPU: every expert takes exactly
    ``capacity`` slots -- its routed tokens in token order, then unrouted ones in token order -- and the way back
    adds every slot's row, times the slot's probability, to its token."""
    import sys

    import primus_turbo_b200.pytorch.ops.moe.permutation  # noqa: F401

    perm = sys.modules["primus_turbo_b200.pytorch.ops.moe.permutation"]
    monkeypatch.setattr(perm, "require_cuda", lambda *t: None)
    g = torch.Generator().manual_seed(0)
    T, E, H, capacity = 11, 4, 6, 3
    routing = torch.rand(T, E, generator=g) < 0.35
    routing[:, 2] = False  # an expert nobody routes to: all of its slots are padding
    routing[:, 0] = True   # more routed tokens than capacity: the later ones are dropped
    probs = torch.rand(T, E, generator=g, dtype=torch.float64)
    x = torch.randn(T, H, generator=g, dtype=torch.float64, requires_grad=True)
    rows, slot_probs, sorted_indices, tpe = perm.token_permute(
        x, E * capacity, probs=probs, routing_map=routing, drop_and_pad=True)
    want = []
    for e in range(E):
        routed = [t for t in range(T) if routing[t, e]]
        padding = [t for t in range(T) if not routing[t, e]]
        want += (routed + padding)[:capacity]
    assert sorted_indices.tolist() == want and tpe.tolist() == routing.sum(0).tolist()
    assert torch.equal(rows, x.detach()[want])
    assert torch.equal(slot_probs, torch.stack([probs[t, i // capacity] for i, t in enumerate(want)]))
    y = rows * 2.0
    back = perm.token_unpermute(y, sorted_indices, merging_probs=probs, restore_shape=(T, H), routing_map=routing,
                                drop_and_pad=True)
    ref = torch.zeros(T, H, dtype=torch.float64)
    for i, t in enumerate(want):
        ref[t] += 2.0 * x.detach()[t] * probs[t, i // capacity]
    torch.testing.assert_close(back.detach(), ref, rtol=1e-12, atol=1e-12)
    back.sum().backward()
    weight = torch.zeros(T, dtype=torch.float64)
    for i, t in enumerate(want):
        weight[t] += 2.0 * probs[t, i // capacity]
    torch.testing.assert_close(x.grad, weight.unsqueeze(1).expand(T, H), rtol=1e-12, atol=1e-12)
