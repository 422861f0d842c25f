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
