"""``torch.nn.Linear`` whose matmuls (forward, dgrad, wgrad) run through ``gemm_fp8``.

Mirrors primus_turbo/pytorch/modules/linear_fp8.py:20-119: same constructor, same ``from_float``
conversion (in place by re-classing the module, or into a fresh copy), bias added after the FP8
GEMM in the activation dtype, any leading batch dimensions flattened into the row axis.
"""

from __future__ import annotations

from typing import Optional

import torch

from primus_turbo_b200.pytorch.core.low_precision import Float8QuantConfig, ScalingGranularity
from primus_turbo_b200.pytorch.ops.gemm_fp8 import gemm_fp8

__all__ = ["Float8Linear"]


def _default_config() -> Float8QuantConfig:
    return Float8QuantConfig(granularity=ScalingGranularity.TENSORWISE)


class Float8Linear(torch.nn.Linear):
    def __init__(self, in_features: int, out_features: int, bias: bool = True,
                 config: Optional[Float8QuantConfig] = None, **kwargs):
        super().__init__(in_features, out_features, bias, **kwargs)
        self.config = config if config is not None else _default_config()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        y = gemm_fp8(x.reshape(-1, self.in_features), self.weight, trans_a=False, trans_b=True,
                     out_dtype=x.dtype, config=self.config)
        if self.bias is not None:
            y = y + self.bias
        return y.view(*lead, self.out_features)

    @classmethod
    @torch.no_grad()
    def from_float(cls, mod: torch.nn.Linear, config: Optional[Float8QuantConfig] = None,
                   inplace: bool = True) -> "Float8Linear":
        assert isinstance(mod, torch.nn.Linear), f"Expected torch.nn.Linear, got {type(mod)}"
        config = config if config is not None else _default_config()
        if inplace:
            mod.__class__ = cls
            mod.config = config
            return mod
        new = cls(mod.in_features, mod.out_features, bias=mod.bias is not None, config=config,
                  device=mod.weight.device, dtype=mod.weight.dtype)
        new.weight.copy_(mod.weight)
        if mod.bias is not None:
            new.bias.copy_(mod.bias)
        return new

    def extra_repr(self) -> str:
        return f"{super().extra_repr()}, config={getattr(self, 'config', None)}"
