"""GPU parity: every quantize / dequantize entry point, through the public ops and therefore the
C ABI, must reproduce the oracle's FP8 bytes and fp32 scale bits exactly."""

import hashlib

import numpy as np
import pytest
import torch

from oracle import fp8_oracle as O
from tests.gpu_util import DEV, E4, E5, assert_quant_equal, gen, randn

pytestmark = pytest.mark.gpu

from primus_turbo_b200.pytorch.core.low_precision import ScalingGranularity as G  # noqa: E402
from primus_turbo_b200.pytorch.core.low_precision import ScalingRecipe  # noqa: E402
from primus_turbo_b200.pytorch.kernels.gemm_impl import group_offs_from_lens  # noqa: E402
from primus_turbo_b200.pytorch.kernels.quantization_impl import (  # noqa: E402
    quant_fp8_blockwise_segment_m_row_col_impl,
    transpose_2d_fp8,
)
from primus_turbo_b200.pytorch.ops import dequantize_fp8, quantize_fp8, quantize_fp8_with_trans  # noqa: E402

HP = [torch.bfloat16, torch.float16, torch.float32]


@pytest.mark.parametrize("dtype", HP)
@pytest.mark.parametrize("fp8", [E4, E5])
@pytest.mark.parametrize("numel", [1, 111, 7168, 8193, 1048576, 1048576 + 3])
def test_tensorwise(dtype, fp8, numel):
    x = randn(gen(numel), numel, scale=2.5, dtype=dtype)
    q, s = quantize_fp8(x.to(DEV), fp8, G.TENSORWISE)
    assert s.shape == () and q.shape == x.shape
    assert_quant_equal(q, s, *O.quant_tensorwise(x, fp8))


def test_tensorwise_amax_spike_and_zero():
    """amax regression: one large element anywhere must set the scale; all-zero input uses the floor."""
    x = randn(gen(5), 3, 4099)
    for pos in (0, 4098, 3 * 4099 - 1):
        y = x.clone().reshape(-1)
        y[pos] = 1000.0
        y = y.reshape(3, 4099)
        assert_quant_equal(*quantize_fp8(y.to(DEV), E4, G.TENSORWISE), *O.quant_tensorwise(y, E4))
    z = torch.zeros(17, 33, dtype=torch.bfloat16)
    assert_quant_equal(*quantize_fp8(z.to(DEV), E4, G.TENSORWISE), *O.quant_tensorwise(z, E4))


@pytest.mark.parametrize("dtype", HP)
@pytest.mark.parametrize("shape", [(1, 1), (111, 7168), (2, 8193), (4, 96, 520), (3, 2, 40, 24)])
def test_rowwise_all_axes(dtype, shape):
    x = randn(gen(len(shape)), *shape, dtype=dtype)
    for axis in list(range(len(shape))) + [-1, -2][: len(shape)]:
        q, s = quantize_fp8(x.to(DEV), E4, G.ROWWISE, axis=axis)
        qo, so = O.quant_rowwise(x, E4, axis)
        assert s.shape == so.shape
        assert_quant_equal(q, s, qo, so, f"axis={axis}")
        d = dequantize_fp8(q, torch.float32, G.ROWWISE, axis=axis, scale_inv=s)
        assert torch.equal(d.cpu(), O.dequant_rowwise(qo, so))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(128, 128), (256, 1024), (320, 256), (300, 333), (1, 7), (129, 7168)])
def test_blockwise_1d_dual_2d(dtype, shape):
    x = randn(gen(shape[0]), *shape, dtype=dtype)
    xd = x.to(DEV)
    for axis in (0, 1, -1, -2):
        q, s = quantize_fp8(xd, E4, G.BLOCKWISE, block_size=128, axis=axis)
        qo, so = O.quant_block1d(x, E4, axis)
        assert_quant_equal(q, s, qo, so, f"block1d axis={axis}")
        d = dequantize_fp8(q, dtype, G.BLOCKWISE, block_size=128, axis=axis, scale_inv=s)
        assert torch.equal(d.cpu(), O.dequant_block1d(qo, so, axis, dtype))
        torch.testing.assert_close(d.cpu().float(), x.float(), rtol=1e-1, atol=1e-1)
    r = quantize_fp8_with_trans(xd, E4, G.BLOCKWISE, block_size=128)
    ro = O.quant_block1d_dual(x, E4)
    assert_quant_equal(r[0], r[1], ro[0], ro[1], "dual row")
    assert_quant_equal(r[2], r[3], ro[2], ro[3], "dual col")
    recipe = ScalingRecipe(use_2d_block=True)
    for w in (x, torch.stack([x, -x * 0.02, x * 3])):
        q, s = quantize_fp8(w.to(DEV), E4, G.BLOCKWISE, block_size=128, scaling_recipe=recipe)
        qo, so = O.quant_block2d(w, E4)
        assert_quant_equal(q, s, qo, so, "block2d")
        d = dequantize_fp8(q, torch.float32, G.BLOCKWISE, block_size=128, scale_inv=s, scaling_recipe=recipe)
        assert torch.equal(d.cpu(), O.dequant_block2d(qo, so))


def test_blockwise_e5m2_and_tiny_values():
    x = randn(gen(9), 256, 384, scale=1e-6)  # below the 1e-4 amax floor
    for fp8 in (E4, E5):
        r = quantize_fp8_with_trans(x.to(DEV), fp8, G.BLOCKWISE, block_size=128)
        ro = O.quant_block1d_dual(x, fp8)
        assert_quant_equal(r[0], r[1], ro[0], ro[1])
        assert_quant_equal(r[2], r[3], ro[2], ro[3])


@pytest.mark.parametrize(
    "lens",
    [[100, 0, 256, 1, 300], [128, 128], [0, 0, 5], [513], [0], [0, 0], [64] * 40 + [0] * 8 + [700]],
)
@pytest.mark.parametrize("n", [384, 200])
def test_segment_row_col(lens, n):
    gl = torch.tensor(lens, dtype=torch.int64)
    offs = O.group_offs_from_lens(gl)
    m = int(offs[-1]) + 7  # rows past the last group are left untouched
    x = randn(gen(n + len(lens)), m, n)
    offs_dev = group_offs_from_lens(gl.to(DEV))
    assert torch.equal(offs_dev.cpu(), offs)
    r = quant_fp8_blockwise_segment_m_row_col_impl(x.to(DEV), E4, 128, gl.to(DEV), offs_dev)
    ro = O.quant_segment_row_col(x, E4, 128, gl, offs)
    mu, pu = int(offs[-1]), ro[7]
    assert r[1].shape == ro[1].shape and r[3].shape == ro[3].shape and r[2].shape == ro[2].shape
    assert O.bytes_equal(r[0].cpu()[:mu], ro[0][:mu])
    assert O.bytes_equal(r[1].cpu()[:pu], ro[1][:pu])
    assert O.bits_equal_f32(r[2].cpu()[:, :mu].contiguous(), ro[2][:, :mu].contiguous())
    assert O.bits_equal_f32(r[3].cpu()[: pu // 128], ro[3][: pu // 128])
    assert torch.equal(r[4].cpu(), ro[4]) and torch.equal(r[5].cpu(), ro[5])


def test_group_offs_large():
    gl = torch.randint(0, 1000, (1000,), generator=gen(3), dtype=torch.int64)
    assert torch.equal(group_offs_from_lens(gl.to(DEV)).cpu(), O.group_offs_from_lens(gl))


def test_transpose_bytes():
    q = randn(gen(4), 3, 130, 77).to(E4)
    t = transpose_2d_fp8(q.to(DEV))
    assert torch.equal(t.cpu().view(torch.uint8), q.view(torch.uint8).transpose(-1, -2).contiguous())


def test_golden_c1_bytes(golden_dir):
    """The small benchmark configuration against the committed digests."""
    z = np.load(golden_dir / "oracle_c1.npz")
    g0 = gen(0)
    A = torch.randn(256, 1024, generator=g0).to(torch.bfloat16)
    B = (torch.randn(512, 1024, generator=g0) * 0.02).to(torch.bfloat16)

    def sha(t):
        t = t.cpu().contiguous()
        v = {1: torch.uint8, 2: torch.int16, 4: torch.int32}[t.element_size()]
        return hashlib.sha256(t.view(v).numpy().tobytes()).hexdigest()

    dig = [str(d) for d in z["digests"]]
    a_row, a_s_row, a_col, a_s_col = quantize_fp8_with_trans(A.to(DEV), E4, G.BLOCKWISE, block_size=128)
    b_q, b_s = quantize_fp8(B.to(DEV), E4, G.BLOCKWISE, block_size=128, scaling_recipe=ScalingRecipe(use_2d_block=True))
    assert [sha(a_row), sha(a_col), sha(b_q)] == dig[2:5]
    assert np.array_equal(a_s_row.cpu().view(torch.int32).numpy(), z["a_s_row"])
    assert np.array_equal(a_s_col.cpu().view(torch.int32).numpy(), z["a_s_col"])
    assert np.array_equal(b_s.cpu().view(torch.int32).numpy(), z["b_s"])


def test_full_size_properties():
    """Benchmark-size activation (65536 x 7168): size-independent checks -- the row copy of the
    grouped quantiser equals the ungrouped 1x128 quantiser, dequantise(quantise(x)) stays within
    the FP8 step, and quantising a dequantised row copy again is idempotent."""
    m, n, G_ = 65536, 7168, 256
    x = torch.randn(m, n, device=DEV, dtype=torch.bfloat16)
    lens = O.make_counts_softmax(G_, m, gen(0)).to(DEV)
    offs = group_offs_from_lens(lens)
    q_row, q_col, s_row, s_col, vk_lens, vk_offs = quant_fp8_blockwise_segment_m_row_col_impl(x, E4, 128, lens, offs)
    q1, s1 = quantize_fp8(x, E4, G.BLOCKWISE, block_size=128, axis=1)
    assert torch.equal(q_row.view(torch.uint8), q1.view(torch.uint8))
    assert torch.equal(s_row, s1.t())
    d = dequantize_fp8(q1, torch.float32, G.BLOCKWISE, block_size=128, axis=1, scale_inv=s1)
    rel = (d - x.float()).abs().max() / x.float().abs().max()
    assert rel < 0.07  # half an e4m3 step (2^-4) of the block amax
    q2, s2 = quantize_fp8(d, E4, G.BLOCKWISE, block_size=128, axis=1)  # fp32 in: payload is a fixed point
    assert torch.equal(q2.view(torch.uint8), q1.view(torch.uint8))
    torch.testing.assert_close(s2, s1, rtol=1e-6, atol=0)
    assert int(vk_offs[-1]) == int(((lens + 127) // 128 * 128).sum())
    # padded rows are zero bytes
    g = int(torch.nonzero(lens % 128 != 0)[0])
    lo = int(vk_offs[g]) + int(lens[g])
    hi = int(vk_offs[g + 1])
    assert int(q_col[lo:hi].view(torch.uint8).max()) == 0


def test_quantize_traces_as_one_graph():
    """``torch.compile(quantize_fp8, fullgraph=True)`` (reference tests/pytorch/ops/test_quantization.py:43-52):
    the op is an opaque custom op with a fake kernel, so dynamo captures it without a graph break."""
    x = randn(gen(77), 128, 512).to(DEV)
    fn = torch.compile(quantize_fp8, fullgraph=True, backend="eager")
    q, s = fn(x, E4, G.BLOCKWISE, block_size=128, axis=1)
    qo, so = O.quant_block1d(x.cpu(), E4, 1)
    assert_quant_equal(q, s, qo, so)
    q, s = fn(x, E4, G.TENSORWISE)
    assert_quant_equal(q, s, *O.quant_tensorwise(x.cpu(), E4))


def test_blockwise_kernels_match_reference_triton_fixture():
    """The CUDA blockwise quantisers against outputs of the reference's own Triton kernels (captured on
    CPU by Triton's interpreter, tests/golden/make_golden.py): scale bits, layouts, and FP8 bytes
    wherever the interpreter's cast is sound (tests/golden_util.py)."""
    from tests import golden_util as GU

    z = GU.load()
    x = GU.bf16(z["b1_x"])
    xd = x.to(DEV)
    for axis, mode in ((1, "row"), (0, "col")):
        q, s = quantize_fp8(xd, E4, G.BLOCKWISE, block_size=128, axis=axis)
        GU.assert_scales_equal(s, GU.f32(z[f"b1_s_axis{axis}"]), f"1-D axis {axis}")
        GU.assert_payload_matches(q, GU.u8(z[f"b1_q_axis{axis}"]), x, GU.forward_scale(x, mode), f"1-D axis {axis}")
    q_row, s_row, q_col, s_col = quantize_fp8_with_trans(xd, E4, G.BLOCKWISE, block_size=128)
    GU.assert_scales_equal(s_row, GU.f32(z["dual_s_row"]), "dual row")
    GU.assert_scales_equal(s_col, GU.f32(z["dual_s_col"]), "dual col")
    GU.assert_payload_matches(q_row, GU.u8(z["dual_q_row"]), x, GU.forward_scale(x, "row"), "dual row")
    GU.assert_payload_matches(q_col, GU.u8(z["dual_q_col"]), x, GU.forward_scale(x, "col"), "dual col")
    w = GU.bf16(z["w_x"])
    q, s = quantize_fp8(w.to(DEV), E4, G.BLOCKWISE, block_size=128, scaling_recipe=ScalingRecipe(use_2d_block=True))
    GU.assert_scales_equal(s, GU.f32(z["w_s"]), "128x128 weight")
    GU.assert_payload_matches(q, GU.u8(z["w_q"]), w, GU.forward_scale(w, "2d"), "128x128 weight")
    xs = GU.bf16(z["seg_x"])
    lens = torch.from_numpy(z["seg_lens"])
    ref_vk = torch.from_numpy(z["seg_vk_offs"])
    offs_dev = group_offs_from_lens(lens.to(DEV))
    q_row, q_col, s_row, s_col, vk_lens, vk_offs = quant_fp8_blockwise_segment_m_row_col_impl(
        xs.to(DEV), E4, 128, lens.to(DEV), offs_dev)
    assert torch.equal(vk_offs.cpu(), ref_vk)
    mu, pu = int(lens.sum()), int(ref_vk[-1])
    GU.assert_scales_equal(s_row[:, :mu].contiguous(), GU.f32(z["seg_s_row"])[:, :mu].contiguous(), "segment row scales")
    GU.assert_payload_matches(q_row[:mu], GU.u8(z["seg_q_row"])[:mu], xs[:mu], GU.forward_scale(xs[:mu], "row"),
                              "segment row copy")
    xp = GU.padded_segments(xs, lens, ref_vk)
    GU.assert_scales_equal(s_col[: pu // 128], GU.f32(z["seg_s_col"])[: pu // 128].contiguous(), "segment column scales")
    GU.assert_payload_matches(q_col[:pu], GU.u8(z["seg_q_col"])[:pu], xp, GU.forward_scale(xp, "col"),
                              "segment column copy")


def test_segment_row_col_without_block_table_gives_the_same_bytes():
    """The per-block source-row table is an optional workspace: with NULL every tile scans the group
    offsets instead, and all six outputs must be identical."""
    from primus_turbo_b200 import _lib

    gl = torch.tensor([100, 0, 256, 1, 300, 129], dtype=torch.int64)
    m, n = int(gl.sum()) + 5, 384
    x = randn(gen(9), m, n).to(DEV)
    gld = gl.to(DEV)
    offs = group_offs_from_lens(gld)
    with_table = quant_fp8_blockwise_segment_m_row_col_impl(x, E4, 128, gld, offs)
    G_, m_pad = gl.numel(), m + 128 * gl.numel()
    q_row = torch.zeros((m, n), dtype=E4, device=DEV)
    q_col = torch.zeros((m_pad, n), dtype=E4, device=DEV)
    s_row = torch.zeros((3, m), dtype=torch.float32, device=DEV)
    s_col = torch.zeros(((m_pad + 127) // 128, n), dtype=torch.float32, device=DEV)
    vk_lens = torch.zeros(G_, dtype=torch.int64, device=DEV)
    vk_offs = torch.zeros(G_ + 1, dtype=torch.int64, device=DEV)
    _lib.call("ptb_quant_fp8_segment_row_col", x.data_ptr(), _lib.PTB_BF16, m, n, G_, gld.data_ptr(), offs.data_ptr(),
              q_row.data_ptr(), q_col.data_ptr(), s_row.data_ptr(), s_col.data_ptr(), vk_lens.data_ptr(),
              vk_offs.data_ptr(), None, _lib.PTB_E4M3, torch.cuda.current_stream().cuda_stream)
    mu, pu = int(gl.sum()), int(vk_offs[-1])
    assert torch.equal(vk_offs, with_table[5]) and torch.equal(vk_lens, with_table[4])
    assert torch.equal(q_row[:mu].view(torch.uint8), with_table[0][:mu].view(torch.uint8))
    assert torch.equal(q_col[:pu].view(torch.uint8), with_table[1][:pu].view(torch.uint8))
    assert torch.equal(s_row[:, :mu], with_table[2][:, :mu])
    assert torch.equal(s_col[: pu // 128], with_table[3][: pu // 128])
