"""Helpers for the fixtures in tests/golden/ref_blockwise_interp.npz (outputs of the reference's
Triton blockwise quantise kernels run by Triton's CPU interpreter).

Scales in those fixtures are sound bit for bit.  The FP8 payload is sound except where the
interpreter's float-to-e4m3 cast (a numpy emulation, not the GPU's conversion instruction) departs from
round-to-nearest-even: exact ties (it rounds away from zero), values that round up into the next
binade (it returns the binade below) and subnormal results (it truncates).  ``unsound_cast_mask``
marks exactly those positions from the pre-cast value; everything else must match byte for byte.
"""

from pathlib import Path

import numpy as np
import torch

E4 = torch.float8_e4m3fn
SENT_Q, SENT_S = 0x55, -777.0  # sentinels pre-filled by tests/golden/make_golden.py
FIXTURE = Path(__file__).resolve().parent / "golden" / "ref_blockwise_interp.npz"


def load():
    return np.load(FIXTURE)


def bf16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.copy()).view(torch.bfloat16)


def f32(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.copy()).view(torch.float32)


def u8(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.copy())


def forward_scale(x: torch.Tensor, mode: str) -> torch.Tensor:
    """Per-element scale = 448 / max(amax_block, 1e-4) in fp32, for 128-wide blocks along the row
    ('row': 1x128), the column ('col': 128x1) or both ('2d': 128x128).  Written independently of the
    oracle on purpose."""
    xf = x.float()
    M, N = xf.shape[-2:]
    Mp, Np = -(-M // 128) * 128, -(-N // 128) * 128
    pad = xf.new_zeros(*xf.shape[:-2], Mp, Np)
    pad[..., :M, :N] = xf.abs()
    lead = pad.shape[:-2]
    t = pad.reshape(*lead, Mp // 128, 128, Np // 128, 128)
    if mode == "row":
        amax = t.amax(dim=-1, keepdim=True).expand_as(t)
    elif mode == "col":
        amax = t.amax(dim=-3, keepdim=True).expand_as(t)
    else:
        amax = t.amax(dim=(-3, -1), keepdim=True).expand_as(t)
    amax = torch.maximum(amax, torch.tensor(1e-4, dtype=torch.float32))
    scale = torch.tensor(448.0, dtype=torch.float32) / amax
    return scale.reshape(*lead, Mp, Np)[..., :M, :N]


def unsound_cast_mask(x: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """True where the interpreter's cast of v = clamp(x * scale) is known to differ from RNE."""
    v = (x.float() * scale).clamp(-448.0, 448.0)
    av = v.abs().double()
    q = v.to(E4)
    code = (q.view(torch.uint8) & 0x7F).to(torch.int16)
    r = q.float().abs().double()
    up = (code + 1).clamp(max=0x7E).to(torch.uint8).view(E4).float().double()
    dn = (code - 1).clamp(min=0).to(torch.uint8).view(E4).float().double()
    tie = ((r > av) & ((r - av) == (av - dn))) | ((r < av) & ((av - r) == (up - av)))
    binade_top = ((code & 7) == 0) & (r > av) & (code >= 8)
    subnormal = (av < 2.0 ** -6) & (av > 0)
    return tie | binade_top | subnormal


def assert_payload_matches(got_q: torch.Tensor, ref_bytes: torch.Tensor, x: torch.Tensor, scale: torch.Tensor, what: str):
    """FP8 bytes equal wherever the fixture's cast is sound; the skipped share stays small."""
    got = got_q.contiguous().view(torch.uint8).cpu()
    skip = unsound_cast_mask(x, scale)
    assert got.shape == ref_bytes.shape, what
    bad = (got != ref_bytes) & ~skip
    assert int(bad.sum()) == 0, f"{what}: {int(bad.sum())} FP8 bytes differ from the reference kernel's output"
    assert float(skip.float().mean()) < 0.08, f"{what}: too many positions skipped"


def assert_scales_equal(got_s: torch.Tensor, ref_s: torch.Tensor, what: str):
    assert got_s.shape == ref_s.shape, what
    assert torch.equal(got_s.contiguous().cpu().view(torch.int32), ref_s.view(torch.int32)), f"{what}: scale bits differ"


def padded_segments(x: torch.Tensor, lens: torch.Tensor, vk_offs: torch.Tensor) -> torch.Tensor:
    """x's rows laid out the way the segment-padded column copy holds them (missing rows zero)."""
    out = x.new_zeros(int(vk_offs[-1]), x.shape[1])
    lo = 0
    for g, n in enumerate(lens.tolist()):
        p = int(vk_offs[g])
        out[p : p + n] = x[lo : lo + n]
        lo += n
    return out
