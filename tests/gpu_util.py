"""Helpers shared by the GPU parity tests: seeded inputs generated on the CPU (so oracle and GPU
see identical bits) and the comparators of the parity gates."""

import torch

from oracle import fp8_oracle as O

E4, E5 = torch.float8_e4m3fn, torch.float8_e5m2
DEV = "cuda"
FROB_TOL = 1e-2  # GEMM gate: relative Frobenius error vs dequantise-then-matmul in fp32
SNR_E4M3_DB = 25.0  # reference gate vs the bf16 matmul (tests/pytorch/ops/test_gemm_fp8.py:101-114)
SNR_E5M2_DB = 20.0


def gen(seed: int) -> torch.Generator:
    return torch.Generator().manual_seed(seed)


def randn(g, *shape, scale=1.0, dtype=torch.bfloat16):
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def assert_quant_equal(q_gpu, s_gpu, q_ref, s_ref, what=""):
    assert O.bits_equal_f32(s_gpu.cpu(), s_ref), f"{what}: scale bits differ"
    assert O.bytes_equal(q_gpu.cpu(), q_ref), f"{what}: fp8 bytes differ"


def unbalanced_lens(g, b, m):
    """tests/pytorch/ref/gemm_ref.py:77-86 (reference's unbalanced group lengths)."""
    dist = 0.2 + 0.8 * torch.rand(b, generator=g)
    dist /= dist.sum()
    lens = (dist * b * m).to(torch.int64)
    lens[-1] += b * m - lens.sum()
    return lens
