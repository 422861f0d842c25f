"""GPU: SwiGLU with routing probabilities (forward, backward, row mask) against the fp32 formulas of the
reference kernels (primus_turbo/triton/activation/swiglu_kernel.py:145-248; reference test
tests/pytorch/ops/test_activation.py), and the fused activation + grouped quantise against running the
two steps one after the other (bytes and scale bits must be identical)."""

import pytest
import torch

from oracle import fp8_oracle as O
from tests.gpu_util import DEV, E4, gen

pytestmark = pytest.mark.gpu

from primus_turbo_b200.pytorch.kernels.gemm_impl import group_offs_from_lens  # noqa: E402
from primus_turbo_b200.pytorch.kernels.quantization_impl import quant_fp8_blockwise_segment_m_row_col_impl  # noqa: E402
from primus_turbo_b200.pytorch.ops.activation import swiglu_with_probs, swiglu_with_probs_quant_segment  # noqa: E402


def _ref(x, probs, mask):
    h = x.shape[-1] // 2
    up, down = x[..., :h].float(), x[..., h:].float()
    out = (up / (1.0 + torch.exp(-up))) * down * probs.float().unsqueeze(-1)
    if mask is not None:
        out = out * (mask != 0).unsqueeze(-1)
    return out


@pytest.mark.parametrize("rows,h", [(1, 8), (300, 2048), (1000, 768), (4096, 1536)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("masked", [False, True])
def test_swiglu_with_probs_forward_and_backward(rows, h, dtype, masked):
    g = gen(rows + h)
    x = torch.randn(rows, 2 * h, generator=g).to(dtype)
    probs = torch.rand(rows, generator=g)
    mask = (torch.rand(rows, generator=g) > 0.3).to(torch.int64) if masked else None
    go = torch.randn(rows, h, generator=g).to(dtype)
    xd, pd = x.to(DEV).requires_grad_(True), probs.to(DEV).requires_grad_(True)
    out = swiglu_with_probs(xd, pd, None if mask is None else mask.to(DEV))
    out.backward(go.to(DEV))
    xr, pr = x.float().requires_grad_(True), probs.clone().requires_grad_(True)
    ref = _ref(xr, pr, mask)
    ref.backward(go.float())
    assert out.dtype == dtype and out.shape == (rows, h)
    tol = dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=4e-3, atol=4e-3)
    torch.testing.assert_close(out.float().cpu(), ref.detach(), **tol)
    # exactly the fp32 result rounded once, except where the device exp differs from the host's in the last place
    exact = (out.cpu() == ref.detach().to(dtype)).float().mean()
    assert exact > 0.98, exact
    torch.testing.assert_close(xd.grad.float().cpu(), xr.grad, **tol)
    torch.testing.assert_close(pd.grad.cpu(), pr.grad, rtol=2e-2, atol=2e-2 * (h ** 0.5))
    if masked:
        assert bool((out[mask.to(DEV) == 0] == 0).all())


@pytest.mark.parametrize("lens,n", [([100, 0, 300, 1, 129], 256), ([128, 128], 128), ([513], 1536), ([64] * 20 + [0] * 3 + [700], 768)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_fused_swiglu_quantise_equals_the_two_steps(lens, n, dtype):
    gl = torch.tensor(lens, dtype=torch.int64)
    m = int(gl.sum()) + 4
    g = gen(n + len(lens))
    x = torch.randn(m, 2 * n, generator=g).to(dtype).to(DEV)
    probs = torch.rand(m, generator=g).to(DEV)
    gld = gl.to(DEV)
    offs = group_offs_from_lens(gld)
    act = swiglu_with_probs(x, probs)
    two = quant_fp8_blockwise_segment_m_row_col_impl(act, E4, 128, gld, offs)
    one = swiglu_with_probs_quant_segment(x, probs, E4, gld, offs)
    mu, pu = int(gl.sum()), int(two[5][-1])
    assert torch.equal(one[5], two[5]) and torch.equal(one[4], two[4])
    assert torch.equal(one[0][:mu].view(torch.uint8), two[0][:mu].view(torch.uint8))
    assert torch.equal(one[1][:pu].view(torch.uint8), two[1][:pu].view(torch.uint8))
    assert torch.equal(one[2][:, :mu].view(torch.int32), two[2][:, :mu].view(torch.int32))
    assert torch.equal(one[3][: pu // 128].view(torch.int32), two[3][: pu // 128].view(torch.int32))
    # and the quantised activation is the oracle's quantisation of the activation
    ro = O.quant_segment_row_col(act.cpu(), E4, 128, gl, O.group_offs_from_lens(gl))
    assert O.bytes_equal(one[0].cpu()[:mu], ro[0][:mu]) and O.bytes_equal(one[1].cpu()[:pu], ro[1][:pu])
