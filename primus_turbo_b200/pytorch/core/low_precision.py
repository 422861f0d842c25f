"""FP8 formats, scaling granularities and the quantisation config of the ops surface.

Mirrors the names and semantics of primus_turbo/pytorch/core/low_precision.py:105-186 so that code
written against the reference keeps working.  On B200 the FP8 types are always the OCP ones
(e4m3fn / e5m2); the reference's FNUZ selection (low_precision.py:77-84) has no counterpart here.
MXFP8 (1x32 blocks, E8M0 scales) has kernels for quantise / dequantise and the dense GEMM; the FP4
recipes are declared for API compatibility but have no kernels.
"""

from __future__ import annotations

from dataclasses import dataclass
from enum import Enum, auto
from typing import NamedTuple, Optional, Tuple

import torch

__all__ = ["float8_e4m3", "float8_e5m2"]

float8_e4m3 = torch.float8_e4m3fn
float8_e5m2 = torch.float8_e5m2
float4_e2m1fn_x2 = getattr(torch, "float4_e2m1fn_x2", None)

MXFP8_BLOCK_SIZE = 32
MXFP4_BLOCK_SIZE = 32
MXFP8_PADDING_ALIGN_SIZE = 128
MXFP4_PADDING_ALIGN_SIZE = 128
DEFAULT_BLOCK_SIZE = 128

_FP8_DTYPES = (torch.float8_e4m3fn, torch.float8_e4m3fnuz, torch.float8_e5m2, torch.float8_e5m2fnuz)


def is_fp8_dtype(dtype) -> bool:
    return dtype in _FP8_DTYPES


def is_fp4_dtype(dtype) -> bool:
    return float4_e2m1fn_x2 is not None and dtype == float4_e2m1fn_x2


def check_fp8_support() -> Tuple[bool, str]:
    if torch.cuda.is_available() and torch.cuda.get_device_capability() >= (10, 0):
        return True, ""
    return False, "An sm_100a (B200) device is required for FP8 execution."


def check_fp8_ocp_support() -> Tuple[bool, str]:
    return check_fp8_support()


def check_mxfp8_support() -> Tuple[bool, str]:
    return check_fp8_support()


def check_mxfp4_support() -> Tuple[bool, str]:
    return False, "MXFP4 kernels are not part of this build."


class Format(Enum):
    E4M3 = auto()
    E5M2 = auto()
    E2M1_X2 = auto()
    HYBRID = auto()  # e4m3 forward, e5m2 for gradients


class ScaleDtype(Enum):
    FP32 = auto()
    E8M0 = auto()


class ScalingGranularity(Enum):
    TENSORWISE = auto()  # == PTB_TENSORWISE (1)
    ROWWISE = auto()  # == PTB_ROWWISE (2)
    BLOCKWISE = auto()  # == PTB_BLOCKWISE (3)
    MX_BLOCKWISE = auto()


class ScalingStrategy(Enum):
    DYNAMIC = auto()


class ScalingRecipe(NamedTuple):
    use_2d_block: bool = False  # one scale per 128x128 tile (weights)
    use_sr: bool = False
    use_rht: bool = False
    shuffle_scale: bool = False
    shuffle_out: bool = False


@dataclass
class Float8QuantConfig:
    format: Format = Format.E4M3
    granularity: ScalingGranularity = ScalingGranularity.TENSORWISE
    strategy: ScalingStrategy = ScalingStrategy.DYNAMIC
    scale_dtype: ScaleDtype = ScaleDtype.FP32
    block_size: Optional[int] = None

    def __post_init__(self):
        if self.granularity == ScalingGranularity.BLOCKWISE:
            assert self.block_size is not None, "block_size must be set when granularity is BLOCKWISE"
        if self.granularity == ScalingGranularity.MX_BLOCKWISE:
            assert self.block_size in [MXFP8_BLOCK_SIZE], (
                f"block_size should be {[MXFP8_BLOCK_SIZE]} when granularity is MX_BLOCKWISE"
            )
            assert self.scale_dtype == ScaleDtype.E8M0, (
                f"scale_dtype should be {ScaleDtype.E8M0} when granularity is MX_BLOCKWISE"
            )


class Float4QuantConfig:
    """Present so that code importing the name keeps importing (low_precision.py:189-214 in the reference);
    FP4 kernels are not part of this build, so a configuration cannot be made."""

    def __init__(self, *args, **kwargs):
        raise NotImplementedError("MXFP4 kernels are not part of this build.")

