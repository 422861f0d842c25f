"""Backend-manager shim.

The reference selects among several GEMM backends (primus_turbo/pytorch/core/backend.py:59-270).
This build has exactly one implementation, so the manager only records what callers ask for: every
setter is accepted, nothing changes which kernel runs, and code or tests that pin a backend keep
working unchanged.
"""

from __future__ import annotations

import os
from enum import Enum, auto
from typing import Dict, Optional

__all__ = ["BackendType", "PrecisionType", "GlobalBackendManager"]

ENV_GEMM_BACKEND = "PRIMUS_TURBO_GEMM_BACKEND"
ENV_GROUPED_GEMM_BACKEND = "PRIMUS_TURBO_GROUPED_GEMM_BACKEND"
ENV_AUTO_TUNE = "PRIMUS_TURBO_AUTO_TUNE"


class PrecisionType(Enum):
    FP4 = auto()
    FP8 = auto()
    BF16_FP16_FP32 = auto()


class BackendType(Enum):
    CK = auto()
    HIPBLASLT = auto()
    AITER = auto()
    TRITON = auto()
    DEEP_EP = auto()
    TURBO = auto()
    FLYDSL = auto()


class GlobalBackendManager:
    """Records requested backends; all of them map to the one CUDA implementation."""

    _gemm: Dict[PrecisionType, Optional[BackendType]] = {}
    _grouped: Dict[PrecisionType, Optional[BackendType]] = {}
    _auto_tune: Optional[bool] = None

    @classmethod
    def _set(cls, table, backend, precision):
        assert backend is None or isinstance(backend, BackendType)
        for p in ([precision] if precision is not None else list(PrecisionType)):
            table[p] = backend

    @classmethod
    def set_gemm_backend(cls, backend: Optional[BackendType], precision: Optional[PrecisionType] = None) -> None:
        cls._set(cls._gemm, backend, precision)

    @classmethod
    def set_grouped_gemm_backend(
        cls, backend: Optional[BackendType], precision: Optional[PrecisionType] = None
    ) -> None:
        cls._set(cls._grouped, backend, precision)

    @classmethod
    def set_auto_tune(cls, enabled: Optional[bool]) -> None:
        cls._auto_tune = enabled

    @classmethod
    def _from_env(cls, key: str) -> Optional[BackendType]:
        v = os.environ.get(key)
        if not v or ":" in v:
            return None
        return BackendType.__members__.get(v.strip().upper())

    @classmethod
    def get_gemm_backend(cls, precision: PrecisionType = PrecisionType.FP8) -> Optional[BackendType]:
        return cls._gemm.get(precision) or cls._from_env(ENV_GEMM_BACKEND)

    @classmethod
    def get_grouped_gemm_backend(cls, precision: PrecisionType = PrecisionType.FP8) -> Optional[BackendType]:
        return cls._grouped.get(precision) or cls._from_env(ENV_GROUPED_GEMM_BACKEND)

    @classmethod
    def auto_tune_enabled(cls) -> bool:
        if cls._auto_tune is not None:
            return cls._auto_tune
        return os.environ.get(ENV_AUTO_TUNE, "0") == "1"

    @classmethod
    def reset(cls) -> None:
        cls._gemm, cls._grouped, cls._auto_tune = {}, {}, None
