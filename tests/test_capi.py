"""CPU: the C-ABI library loads, exports every symbol include/ptb.h declares, and rejects bad
arguments before touching the device (so these calls are safe without a GPU)."""

import ctypes
import re
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent


def _declared_symbols():
    text = (REPO / "include" / "ptb.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ptb_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_expected_entry_points():
    syms = _declared_symbols()
    for s in (
        "ptb_quant_fp8_tensorwise", "ptb_quant_fp8_rowwise", "ptb_quant_fp8_block1d", "ptb_quant_fp8_block1d_dual",
        "ptb_quant_fp8_block2d", "ptb_quant_fp8_segment_row_col", "ptb_dequant_fp8_tensorwise",
        "ptb_dequant_fp8_rowwise", "ptb_dequant_fp8_block1d", "ptb_dequant_fp8_block2d", "ptb_group_offs",
        "ptb_transpose_2d_u8", "ptb_gemm_fp8", "ptb_grouped_gemm_fp8", "ptb_grouped_gemm_fp8_variable_k",
        "ptb_last_error", "ptb_version",
    ):
        assert s in syms


def test_library_exports_every_declared_symbol():
    from primus_turbo_b200 import _lib

    for name in _declared_symbols():
        assert hasattr(_lib.lib, name), f"{name} declared in include/ptb.h but not exported"
    assert set(_lib.EXPORTS) <= set(_declared_symbols()) | {"ptb_version", "ptb_last_error"}
    assert _lib.lib.ptb_version() == 100


def test_argument_errors_are_reported_without_a_device():
    from primus_turbo_b200 import _lib

    L = _lib.lib
    rc = L.ptb_quant_fp8_tensorwise(None, _lib.PTB_BF16, -1, None, _lib.PTB_E4M3, None, None, None)
    assert rc == -1 and b"n < 0" in L.ptb_last_error()
    rc = L.ptb_quant_fp8_block1d(None, _lib.PTB_BF16, 4, 4, 7, None, _lib.PTB_E4M3, None, None)
    assert rc == -1
    # K == 0 is rejected before any pointer is looked at
    rc = L.ptb_gemm_fp8(None, 3, 0, 0, None, 3, 1, 0, None, 2, 0, 128, 128, 0, 1, None, 0, 0, None, 0, 0, 1, 0, None)
    assert rc == -1 and b"bad shape" in L.ptb_last_error()
    # more groups than the device-side tile table holds
    rc = L.ptb_grouped_gemm_fp8(None, 3, 0, None, 3, 1, None, 2, 0, None, 5000, 16, 16, 16, 3, None, 0, 0, None, 0, 0, 0,
                                0, None)
    assert rc == -5 and b"groups" in L.ptb_last_error()
    with pytest.raises(_lib.PtbError):
        _lib.check(rc, "ptb_grouped_gemm_fp8")
    # a misaligned FP8 output of a blockwise quantise is an error code, never a device fault
    # (the pointers are only inspected on the host; nothing is launched)
    rc = L.ptb_quant_fp8_block1d(0x1000, _lib.PTB_BF16, 128, 128, 1, 0x2004, _lib.PTB_E4M3, 0x3000, None)
    assert rc == -3 and b"8-byte" in L.ptb_last_error()
    rc = L.ptb_quant_fp8_block2d(0x1000, _lib.PTB_BF16, 1, 128, 128, 0x2001, _lib.PTB_E4M3, 0x3000, None)
    assert rc == -3
    # empty problems succeed trivially
    assert L.ptb_quant_fp8_block2d(None, 2, 0, 128, 128, None, 3, None, None) == 0
    assert L.ptb_transpose_2d_u8(None, 1, 0, 8, None, None) == 0


def test_no_cpu_fallback_for_cpu_tensors():
    import torch

    from primus_turbo_b200 import _lib
    from primus_turbo_b200.pytorch.ops import quantize_fp8
    from primus_turbo_b200.pytorch.core.low_precision import ScalingGranularity

    with pytest.raises(_lib.PtbError):
        quantize_fp8(torch.zeros(4, 4, dtype=torch.bfloat16), torch.float8_e4m3fn, ScalingGranularity.TENSORWISE)
