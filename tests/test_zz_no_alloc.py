"""GPU: the rowwise quantize entry point that owns its scratch (``ptb_quant_fp8_rowwise_noalloc``).

Some hosts give a library nothing but the input and output buffers of a call and keep every other
byte of the device for themselves, so the library cannot be handed (and must not create) a
workspace.  This entry point serves them from a fixed array inside the library.  It must produce
exactly what the workspace variant produces -- FP8 bytes and scale bits -- on back-to-back calls
(the second call sees the first call's leftovers in the shared array and has to clear them), and
it must refuse shapes that do not fit the array.
"""

import pytest
import torch

from oracle import fp8_oracle as O

pytestmark = pytest.mark.gpu

from primus_turbo_b200 import _lib  # noqa: E402

E4 = torch.float8_e4m3fn


def _run(entry: str, x: torch.Tensor, with_workspace: bool):
    B, M, N = x.shape
    q = torch.empty(x.shape, dtype=E4, device=x.device)
    s = torch.empty((B, 1, N), dtype=torch.float32, device=x.device)
    stream = torch.cuda.current_stream().cuda_stream
    args = [x.data_ptr(), _lib.dtype_code(x.dtype), B, M, N, q.data_ptr(), _lib.PTB_E4M3, s.data_ptr()]
    if with_workspace:
        ws = torch.empty(B * N, dtype=torch.float32, device=x.device)
        args.append(ws.data_ptr())
    args.append(stream)
    rc = getattr(_lib.lib, entry)(*args)
    assert rc == 0, _lib.lib.ptb_last_error()
    torch.cuda.synchronize()
    return q, s


def test_noalloc_matches_workspace_variant_twice_in_a_row():
    torch.manual_seed(0)
    big = torch.randn(3, 257, 1000, device="cuda", dtype=torch.bfloat16) * 40.0
    small = torch.randn(3, 257, 1000, device="cuda", dtype=torch.bfloat16) * 1e-3  # smaller amax everywhere
    for x in (big, small):  # second call must not see the first call's larger column maxima
        q_ref, s_ref = _run("ptb_quant_fp8_rowwise", x, with_workspace=True)
        q, s = _run("ptb_quant_fp8_rowwise_noalloc", x, with_workspace=False)
        assert torch.equal(s.view(torch.int32), s_ref.view(torch.int32))
        assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8))
        # and the entry point stands on its own against the CPU oracle of the reference arithmetic
        q_cpu, s_cpu = O.quant_rowwise(x.cpu(), E4, 1)
        assert O.bits_equal_f32(s.cpu(), s_cpu) and O.bytes_equal(q.cpu(), q_cpu)
    # innermost-axis case (N == 1) goes through the same entry point and needs no scratch at all
    rows = torch.randn(300, 515, 1, device="cuda", dtype=torch.float16)
    q_ref, s_ref = _run("ptb_quant_fp8_rowwise", rows, with_workspace=True)
    q, s = _run("ptb_quant_fp8_rowwise_noalloc", rows, with_workspace=False)
    assert torch.equal(s.view(torch.int32), s_ref.view(torch.int32)) and torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8))
    q_cpu, s_cpu = O.quant_rowwise(rows.cpu(), E4, 1)
    assert O.bits_equal_f32(s.cpu(), s_cpu) and O.bytes_equal(q.cpu(), q_cpu)
    # that case has no size limit: more rows than the scratch has words
    many = torch.randn(70000, 64, 1, device="cuda", dtype=torch.bfloat16)
    q, s = _run("ptb_quant_fp8_rowwise_noalloc", many, with_workspace=False)
    q_cpu, s_cpu = O.quant_rowwise(many.cpu(), E4, 1)
    assert O.bits_equal_f32(s.cpu(), s_cpu) and O.bytes_equal(q.cpu(), q_cpu)


def test_noalloc_rejects_shapes_beyond_its_scratch():
    x = torch.zeros(1, 2, 65537, device="cuda", dtype=torch.bfloat16)
    q = torch.empty(x.shape, dtype=E4, device="cuda")
    s = torch.empty((1, 1, 65537), dtype=torch.float32, device="cuda")
    rc = _lib.lib.ptb_quant_fp8_rowwise_noalloc(
        x.data_ptr(), _lib.PTB_BF16, 1, 2, 65537, q.data_ptr(), _lib.PTB_E4M3, s.data_ptr(),
        torch.cuda.current_stream().cuda_stream,
    )
    assert rc == -5 and b"65536" in _lib.lib.ptb_last_error()
    # sizes whose product wraps a 64-bit integer are refused as well (no pointer is touched)
    rc = _lib.lib.ptb_quant_fp8_rowwise_noalloc(None, _lib.PTB_BF16, 1 << 32, 2, 1 << 32, None, _lib.PTB_E4M3, None, None)
    assert rc == -5
