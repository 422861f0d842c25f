"""GPU parity: MoE token permutation against the CPU restatement of the reference's torch definition
(primus_turbo/pytorch/ops/moe/permutation.py:281-436; reference tests tests/pytorch/ops/test_permutation.py):
row ids, token order, tokens per expert, permuted rows and probabilities bit-exact; the merge of
``token_unpermute`` bit-exact against a sequential fp32 scatter-add; gradients against autograd on the
reference formulas."""

import pytest
import torch

from oracle import fp8_oracle as O
from tests.gpu_util import DEV, gen

pytestmark = pytest.mark.gpu

from primus_turbo_b200.pytorch.ops.moe import token_permute, token_unpermute  # noqa: E402


def _routing(g, T, E, topk):
    scores = torch.rand(T, E, generator=g)
    idx = scores.topk(topk, dim=1).indices
    mask = torch.zeros(T, E, dtype=torch.bool)
    mask.scatter_(1, idx, True)
    probs = torch.softmax(torch.randn(T, E, generator=g), dim=1) * mask
    return mask, probs.float()


@pytest.mark.parametrize("T,E,topk,H", [(1, 4, 2, 64), (300, 8, 2, 512), (1000, 64, 6, 7168), (4096, 256, 8, 2048), (513, 1024, 3, 128)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("map_dtype", [torch.bool, torch.int32])
def test_permute_and_unpermute_match_the_reference_definition(T, E, topk, H, dtype, map_dtype):
    g = gen(T + E)
    mask, probs = _routing(g, T, E, topk)
    mask[:, 1] = False  # an expert nobody routes to
    probs = probs * mask
    x = torch.randn(T, H, generator=g).to(dtype)
    n = int(mask.sum())
    rows_ref, pp_ref, si_ref, tpe_ref = O.token_permute_ref(x, mask, probs)
    rows, pp, si, tpe = token_permute(x.to(DEV), n, probs=probs.to(DEV), routing_map=mask.to(map_dtype).to(DEV))
    assert torch.equal(si.cpu(), si_ref) and torch.equal(tpe.cpu(), tpe_ref)
    assert torch.equal(rows.cpu(), rows_ref) and torch.equal(pp.cpu(), pp_ref)
    # all routed rows without giving the count (one host read), and fewer rows than are routed (the rest dropped)
    rows_all, _, si_all, _ = token_permute(x.to(DEV), -1, routing_map=mask.to(DEV))
    assert torch.equal(rows_all.cpu(), rows_ref) and torch.equal(si_all.cpu(), si_ref)
    if n > 3:
        rows_cut, _, si_cut, tpe_cut = token_permute(x.to(DEV), n - 3, routing_map=mask.to(DEV))
        assert torch.equal(rows_cut.cpu(), rows_ref[: n - 3]) and torch.equal(tpe_cut.cpu(), tpe_ref)
    # expert outputs back to token order, merged with the routing probabilities
    y = torch.randn(n, H, generator=g).to(dtype)
    for mp in (probs, None):
        ref = O.token_unpermute_ref(y, si_ref, (T, H), mp, mask)
        got = token_unpermute(y.to(DEV), si, merging_probs=None if mp is None else mp.to(DEV), restore_shape=(T, H),
                              routing_map=mask.to(DEV))
        assert got.dtype == dtype and torch.equal(got.cpu(), ref)


def test_gradients_match_autograd_on_the_reference_formulas():
    g = gen(5)
    T, E, topk, H = 257, 16, 4, 96
    mask, probs = _routing(g, T, E, topk)
    x = torch.randn(T, H, generator=g)
    w = torch.randn(int(mask.sum()), H, generator=g)
    # reference: permute -> scale by a fixed per-row weight -> unpermute with probs -> weighted sum
    xr, pr = x.clone().requires_grad_(True), probs.clone().requires_grad_(True)
    rows_ref, pp_ref, si_ref, _ = O.token_permute_ref(xr, mask, pr)
    mid_ref = rows_ref * w + pp_ref.unsqueeze(-1)
    p_sel = pr.t().contiguous().masked_select(mask.t().contiguous())
    out_ref = torch.zeros(T, H).index_add_(0, si_ref, mid_ref * p_sel.unsqueeze(-1))
    coeff = torch.randn(T, H, generator=g)
    (out_ref * coeff).sum().backward()
    xd, pd = x.to(DEV).requires_grad_(True), probs.to(DEV).requires_grad_(True)
    rows, pp, si, _ = token_permute(xd, int(mask.sum()), probs=pd, routing_map=mask.to(DEV))
    mid = rows * w.to(DEV) + pp.unsqueeze(-1)
    out = token_unpermute(mid, si, merging_probs=pd, restore_shape=(T, H), routing_map=mask.to(DEV))
    (out * coeff.to(DEV)).sum().backward()
    torch.testing.assert_close(out.detach().cpu(), out_ref.detach(), rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(xd.grad.cpu(), xr.grad, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(pd.grad.cpu(), pr.grad, rtol=1e-4, atol=1e-4)


def test_empty_and_argument_errors():
    x = torch.zeros(0, 32, device=DEV, dtype=torch.bfloat16)
    m = torch.zeros(0, 4, dtype=torch.bool, device=DEV)
    rows, pp, si, tpe = token_permute(x, 0, routing_map=m)
    assert rows.shape == (0, 32) and tpe.tolist() == [0, 0, 0, 0]
    with pytest.raises(ValueError):
        token_permute(torch.zeros(2, 32, device=DEV), 2)
