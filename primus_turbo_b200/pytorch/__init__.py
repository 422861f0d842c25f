"""Mirror of ``primus_turbo.pytorch`` for the FP8 quantize / GEMM / grouped-GEMM path."""

import primus_turbo_b200._lib  # noqa: F401  (loads the CUDA library; raises if it is missing)
from primus_turbo_b200.pytorch import core, modules, ops  # noqa: F401
from primus_turbo_b200.pytorch.core import low_precision

float8_e4m3 = low_precision.float8_e4m3
float8_e5m2 = low_precision.float8_e5m2
