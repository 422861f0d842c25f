"""CPU: the blockwise part of the oracle against outputs of the reference's own Triton kernels
(primus_turbo/triton/quantization/quant_blockwise.py:22-62 1-D, :65-112 dual, :118-156 weight,
:237-327 grouped segment row + column), captured by tests/golden/make_golden.py with Triton's CPU
interpreter.  Scales must agree bit for bit, layouts position for position (positions the reference
leaves unwritten still hold the generator's sentinels), and FP8 bytes wherever the interpreter's cast
is sound (tests/golden_util.py)."""

import torch

from oracle import fp8_oracle as O
from tests import golden_util as GU

E4 = torch.float8_e4m3fn


def test_block1d_both_axes_and_dual():
    z = GU.load()
    x = GU.bf16(z["b1_x"])
    M, N = x.shape
    for axis, mode in ((1, "row"), (0, "col")):
        q, s = O.quant_block1d(x, E4, axis)
        GU.assert_scales_equal(s, GU.f32(z[f"b1_s_axis{axis}"]), f"1-D axis {axis}")
        GU.assert_payload_matches(q, GU.u8(z[f"b1_q_axis{axis}"]), x, GU.forward_scale(x, mode), f"1-D axis {axis}")
    q_row, s_row, q_col, s_col = O.quant_block1d_dual(x, E4)
    GU.assert_scales_equal(s_row, GU.f32(z["dual_s_row"]), "dual row")
    GU.assert_scales_equal(s_col, GU.f32(z["dual_s_col"]), "dual col")
    GU.assert_payload_matches(q_row, GU.u8(z["dual_q_row"]), x, GU.forward_scale(x, "row"), "dual row")
    GU.assert_payload_matches(q_col, GU.u8(z["dual_q_col"]), x, GU.forward_scale(x, "col"), "dual col")
    # the block scaled down below the amax floor takes scale_inv = 1 / (448 / 1e-4)
    floor_inv = torch.tensor(1.0) / (torch.tensor(448.0) / torch.tensor(1e-4))
    assert float(GU.f32(z["b1_s_axis1"])[5, 0]) == float(floor_inv)


def test_block2d_weight():
    z = GU.load()
    w = GU.bf16(z["w_x"])
    q, s = O.quant_block2d(w, E4)
    GU.assert_scales_equal(s, GU.f32(z["w_s"]), "128x128 weight")
    GU.assert_payload_matches(q, GU.u8(z["w_q"]), w, GU.forward_scale(w, "2d"), "128x128 weight")


def test_segment_row_col_layout_scales_and_bytes():
    z = GU.load()
    x = GU.bf16(z["seg_x"])
    lens = torch.from_numpy(z["seg_lens"])
    offs = O.group_offs_from_lens(lens)
    ref_vk = torch.from_numpy(z["seg_vk_offs"])
    q_row, q_col, s_row, s_col, vk_lens, vk_offs, written, pad_used = O.quant_segment_row_col(x, E4, 128, lens, offs)
    assert torch.equal(vk_offs, ref_vk) and pad_used == int(ref_vk[-1])
    mu, Ms, N = int(offs[-1]), x.shape[0], x.shape[1]
    r_q_row, r_q_col = GU.u8(z["seg_q_row"]), GU.u8(z["seg_q_col"])
    r_s_row, r_s_col = GU.f32(z["seg_s_row"]), GU.f32(z["seg_s_col"])
    assert q_col.shape[0] == Ms + 128 * lens.numel() == r_q_col.shape[0]
    # --- what the reference leaves unwritten: rows past the last group, padded rows past the last segment
    assert bool((r_q_row[mu:] == GU.SENT_Q).all()) and bool((r_s_row[:, mu:] == GU.SENT_S).all())
    assert bool((r_q_col[pad_used:] == GU.SENT_Q).all()) and bool((r_s_col[pad_used // 128 :] == GU.SENT_S).all())
    assert bool(written[:mu].all()) and not bool(written[mu:].any())
    # --- row copy and its [ceil(N/128), M] scales over the used rows
    GU.assert_scales_equal(s_row[:, :mu], r_s_row[:, :mu].contiguous(), "segment row scales")
    GU.assert_payload_matches(q_row[:mu], r_q_row[:mu], x[:mu], GU.forward_scale(x[:mu], "row"), "segment row copy")
    # --- column copy: group-relative 128-row blocks, zero rows up to the next multiple of 128
    xp = GU.padded_segments(x, lens, ref_vk)
    GU.assert_scales_equal(s_col[: pad_used // 128], r_s_col[: pad_used // 128].contiguous(), "segment column scales")
    GU.assert_payload_matches(q_col[:pad_used], r_q_col[:pad_used], xp, GU.forward_scale(xp, "col"), "segment column copy")
    for g, n in enumerate(lens.tolist()):
        lo, hi = int(ref_vk[g]) + n, int(ref_vk[g + 1])
        assert bool((r_q_col[lo:hi] == 0).all()), "padding rows of a segment hold the byte 0x00"
