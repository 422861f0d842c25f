"""ctypes binding of the C ABI declared in ``include/ptb.h``.

The shared library is the only compute backend: if it is missing or fails to load, importing this
module raises.  There is no fallback path.
"""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_int, c_int64, c_void_p
from pathlib import Path

import torch

import os

# PTB_LIB_PATH points the binding at another build of the same library (e.g. a tuning build)
_LIB_PATH = Path(os.environ.get("PTB_LIB_PATH") or Path(__file__).resolve().parent / "_C" / "libptb_b200.so")

# element type codes (include/ptb.h)
PTB_F32, PTB_F16, PTB_BF16, PTB_E4M3, PTB_E5M2 = 0, 1, 2, 3, 4
PTB_TENSORWISE, PTB_ROWWISE, PTB_BLOCKWISE = 1, 2, 3
PTB_TENSORWISE_WS_BYTES = 256

_DTYPE_CODE = {
    torch.float32: PTB_F32,
    torch.float16: PTB_F16,
    torch.bfloat16: PTB_BF16,
    torch.float8_e4m3fn: PTB_E4M3,
    torch.float8_e5m2: PTB_E5M2,
}

_P, _I, _L = c_void_p, c_int, c_int64

# name -> argument types; every function returns int except where noted
_PROTOS = {
    "ptb_quant_fp8_tensorwise": [_P, _I, _L, _P, _I, _P, _P, _P],
    "ptb_quant_fp8_tensorwise_with_scale": [_P, _I, _L, _P, _P, _I, _P, _P],
    "ptb_quant_fp8_rowwise": [_P, _I, _L, _L, _L, _P, _I, _P, _P, _P],
    "ptb_quant_fp8_rowwise_noalloc": [_P, _I, _L, _L, _L, _P, _I, _P, _P],
    "ptb_quant_fp8_block1d": [_P, _I, _L, _L, _I, _P, _I, _P, _P],
    "ptb_quant_fp8_block1d_dual": [_P, _I, _L, _L, _P, _P, _P, _P, _I, _P],
    "ptb_quant_fp8_block2d": [_P, _I, _L, _L, _L, _P, _I, _P, _P],
    "ptb_quant_fp8_segment_row_col": [_P, _I, _L, _L, _L, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _P],
    "ptb_dequant_fp8_tensorwise": [_P, _I, _L, _P, _P, _I, _P],
    "ptb_dequant_fp8_rowwise": [_P, _I, _L, _L, _L, _P, _P, _I, _P],
    "ptb_dequant_fp8_block1d": [_P, _I, _L, _L, _I, _P, _P, _I, _P],
    "ptb_dequant_fp8_block2d": [_P, _I, _L, _L, _L, _P, _P, _I, _P],
    "ptb_group_offs": [_P, _L, _P, _P],
    "ptb_transpose_2d_u8": [_P, _L, _L, _L, _P, _P],
    "ptb_gemm_fp8": [_P, _I, _I, _L, _P, _I, _I, _L, _P, _I, _L, _L, _L, _L, _I, _P, _L, _L, _P, _L, _L, _I, _I, _P],
    "ptb_grouped_gemm_fp8": [_P, _I, _L, _P, _I, _I, _P, _I, _L, _P, _L, _L, _L, _L, _I, _P, _L, _L, _P, _L, _L, _L,
                             _I, _P],
    "ptb_grouped_gemm_fp8_variable_k": [_P, _I, _L, _P, _I, _L, _P, _I, _P, _L, _L, _L, _L, _I, _P, _P, _I, _P],
    "ptb_copy_segments": [_P, _P, _I, _P, _L, _L, _I, _P],
    "ptb_copy_segments_signal": [_P, _P, _I, _P, _L, _L, _I, _P, _P, ctypes.c_uint32, _P],
    "ptb_wait_flags": [_P, _I, ctypes.c_uint32, _P],
    "ptb_copy_segments_status": [ctypes.POINTER(c_int), _I],
    "ptb_enable_peer_access": [_I],
    "ptb_gather_rows": [_P, _P, _L, _L, _L, _P, _P],
    "ptb_swiglu_probs_fwd": [_P, _I, _P, _P, _L, _L, _P, _P],
    "ptb_swiglu_probs_bwd": [_P, _P, _I, _P, _P, _L, _L, _P, _P, _P],
    "ptb_swiglu_quant_fp8_segment_row_col": [_P, _I, _P, _L, _L, _L, _P, _P, _P, _P, _P, _P, _P, _P, _I, _P],
    "ptb_moe_row_id_map": [_P, _L, _L, _L, _P, _P, _P, _P, _P],
    "ptb_gather_rows_scaled": [_P, _I, _P, _P, _L, _L, _L, _P, _P],
    "ptb_unpermute_rows": [_P, _I, _P, _P, _L, _L, _L, _P, _P],
    "ptb_unpermute_rows_bwd": [_P, _I, _P, _P, _P, _L, _L, _L, _P, _P, _P],
    "ptb_quant_mxfp8": [_P, _I, _L, _L, _L, _P, _P, _P, _P, _I, _I, _I, _P],
    "ptb_dequant_mxfp8": [_P, _I, _L, _L, _P, _I, _P, _I, _P],
    "ptb_quant_mxfp8_grouped": [_P, _I, _L, _L, _P, _L, _L, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P],
    "ptb_grouped_gemm_mxfp8": [_P, _I, _L, _P, _L, _P, _I, _P, _P, _I, _L, _P, _L, _L, _L, _L, _I, _P],
    "ptb_grouped_gemm_mxfp8_variable_k": [_P, _I, _L, _P, _L, _P, _I, _L, _P, _L, _P, _I, _P, _L, _L, _L, _L, _I, _P],
    "ptb_gemm_mxfp8": [_P, _I, _L, _P, _L, _P, _I, _L, _P, _L, _P, _I, _L, _L, _L, _L, _I, _P],
    "ptb_gemm_status": [ctypes.POINTER(c_int), _I],
    "ptb_gemm_wait_selftest": [_P],
}

EXPORTS = ["ptb_version", "ptb_last_error", *_PROTOS.keys()]


def _load() -> ctypes.CDLL:
    if not _LIB_PATH.exists():
        raise ImportError(
            f"{_LIB_PATH} is missing: build it with `python -m primus_turbo_b200.build` "
            "(there is no fallback implementation)"
        )
    lib = ctypes.CDLL(str(_LIB_PATH))
    lib.ptb_version.restype = c_int
    lib.ptb_version.argtypes = []
    lib.ptb_last_error.restype = c_char_p
    lib.ptb_last_error.argtypes = []
    for name, args in _PROTOS.items():
        fn = getattr(lib, name)
        fn.restype = c_int
        fn.argtypes = args
    return lib


lib = _load()


class PtbError(RuntimeError):
    """A C-ABI call returned a non-zero status (RuntimeError, like the reference's C++ checks)."""


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib.ptb_last_error().decode("utf-8", "replace")
        raise PtbError(f"{what} failed with status {rc}: {msg}")


# kernels enqueued by one successful call of each entry point (memset nodes not counted)
KERNELS_PER_CALL = {"ptb_quant_fp8_tensorwise": 2, "ptb_quant_fp8_rowwise": 2, "ptb_quant_fp8_rowwise_noalloc": 2,
                    "ptb_quant_fp8_segment_row_col": 2, "ptb_quant_mxfp8_grouped": 2, "ptb_moe_row_id_map": 3, "ptb_swiglu_quant_fp8_segment_row_col": 2,
                    "ptb_gemm_status": 0, "ptb_copy_segments_status": 0, "ptb_enable_peer_access": 0}
# PTB_DEBUG_STATUS=1: after every GEMM call, wait for the device and raise if a bounded wait inside the
# kernel ran out (status codes in include/ptb.h).  Off by default: the check synchronises.
_DEBUG_STATUS = os.environ.get("PTB_DEBUG_STATUS", "0") not in ("", "0")
_GEMM_ENTRY_POINTS = ("ptb_gemm_fp8", "ptb_gemm_mxfp8", "ptb_grouped_gemm_fp8", "ptb_grouped_gemm_fp8_variable_k",
                      "ptb_grouped_gemm_mxfp8", "ptb_grouped_gemm_mxfp8_variable_k")
# PTB_NVTX=1: one NVTX range per C-ABI call, named after the entry point (timeline tools show them)
_NVTX = os.environ.get("PTB_NVTX", "0") not in ("", "0")
launch_count = 0  # running total of kernels this process enqueued through the C ABI
_event_log = None  # when a dict: name -> [(start_event, stop_event), ...] on the launching stream


def call(name: str, *args) -> None:
    """Invoke one C-ABI entry point: count its launches, optionally bracket it with CUDA events on
    the current stream (see record_kernel_times), raise PtbError on a non-zero status."""
    global launch_count
    fn = getattr(lib, name)
    if _NVTX:
        torch.cuda.nvtx.range_push(name)
        try:
            rc = fn(*args)
        finally:
            torch.cuda.nvtx.range_pop()
        check(rc, name)
        launch_count += KERNELS_PER_CALL.get(name, 1)
        return
    if _event_log is not None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        rc = fn(*args)
        e1.record()
        _event_log.setdefault(name, []).append((e0, e1))
    else:
        rc = fn(*args)
    check(rc, name)
    launch_count += KERNELS_PER_CALL.get(name, 1)
    if _DEBUG_STATUS and name in _GEMM_ENTRY_POINTS and not torch.cuda.is_current_stream_capturing():
        # (a stream that is being captured into a graph cannot be waited for: the check is skipped there)
        torch.cuda.synchronize()
        code = gemm_status(reset=True)
        if code != 0:
            raise PtbError(f"{name}: a device-side wait ran out (status {code}); the output is incomplete")


class timed_region:
    """Brackets other device work (a collective, a torch copy) with events under ``name`` while
    ``record_kernel_times`` is active, so that a step's timeline can be accounted for; otherwise free."""

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        self.log = _event_log
        if self.log is not None:
            self.e0 = torch.cuda.Event(enable_timing=True)
            self.e0.record()
        return self

    def __exit__(self, *exc):
        if self.log is not None:
            e1 = torch.cuda.Event(enable_timing=True)
            e1.record()
            self.log.setdefault(self.name, []).append((self.e0, e1))
        return False


class record_kernel_times:
    """Context manager: per-entry-point device durations (ms) of every call made inside it."""

    def __enter__(self):
        global _event_log
        self._prev, _event_log = _event_log, {}
        self.log = _event_log
        return self

    def __exit__(self, *exc):
        global _event_log
        _event_log = self._prev
        return False

    def durations_ms(self):
        torch.cuda.synchronize()
        return {k: [a.elapsed_time(b) for a, b in v] for k, v in self.log.items()}


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dt]
    except KeyError:
        raise PtbError(f"dtype {dt} is not supported by the B200 FP8 library") from None


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def stream_of(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise PtbError("tensors must live on a CUDA device: this library has no CPU path")


def copy_segments_status(reset: bool = True) -> int:
    out = c_int(0)
    check(lib.ptb_copy_segments_status(ctypes.byref(out), 1 if reset else 0), "ptb_copy_segments_status")
    return out.value


def gemm_status(reset: bool = True) -> int:
    out = c_int(0)
    check(lib.ptb_gemm_status(ctypes.byref(out), 1 if reset else 0), "ptb_gemm_status")
    return out.value
