"""CPU: the registered custom ops trace under FakeTensorMode with the output shapes and dtypes of
the reference's meta functions (no kernel runs)."""

import torch
from torch._subclasses.fake_tensor import FakeTensorMode

from primus_turbo_b200.pytorch.kernels import custom_ops as C

E4 = torch.float8_e4m3fn


def test_fake_shapes():
    with FakeTensorMode():
        x = torch.empty(300, 333, dtype=torch.bfloat16, device="cuda")
        q, s = C.quantize_fp8_tensorwise(x, E4)
        assert q.shape == x.shape and q.dtype == E4 and s.shape == () and s.dtype == torch.float32
        q, s = C.quantize_fp8_rowwise(x, E4, 0)
        assert s.shape == (1, 333)
        q, s = C.quant_fp8_blockwise(x, E4, 1)
        assert s.shape == (300, 3)
        r = C.quant_fp8_blockwise_dual(x, E4)
        assert [tuple(t.shape) for t in r] == [(300, 333), (300, 3), (300, 333), (3, 333)]
        w = torch.empty(4, 256, 512, dtype=torch.bfloat16, device="cuda")
        q, s = C.quant_fp8_blockwise_for_weight(w, E4)
        assert s.shape == (4, 2, 4)
        lens = torch.empty(4, dtype=torch.int64, device="cuda")
        offs = torch.empty(5, dtype=torch.int64, device="cuda")
        r = C.quant_fp8_blockwise_segment_m_row_col(x, E4, 128, lens, offs)
        assert [tuple(t.shape) for t in r] == [(300, 333), (812, 333), (3, 300), (7, 333), (4,), (5,)]
        a = torch.empty(256, 512, dtype=E4, device="cuda")
        b = torch.empty(384, 512, dtype=E4, device="cuda")
        one = torch.empty((), device="cuda")
        assert C.gemm_fp8_impl(a, one, False, b, one, True, torch.bfloat16, False, 1).shape == (256, 384)
        assert C.gemm_fp8_impl(a, one, False, b, one, True, torch.bfloat16, True, 1).shape == (384, 256)
        wq = torch.empty(4, 384, 512, dtype=E4, device="cuda")
        out = C.grouped_gemm_fp8_impl(a, wq, one, one, lens, offs, False, True, torch.bfloat16, 1)
        assert out.shape == (256, 384)
        g = torch.empty(256, 384, dtype=E4, device="cuda")
        dw = C.grouped_gemm_fp8_variable_k_impl(a, g, one, one, lens, offs, True, False, True, torch.bfloat16, 1)
        assert dw.shape == (4, 384, 512)
