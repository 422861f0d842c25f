"""CPU: the oracle against the committed golden fixtures (tests/golden/make_golden.py)."""

import hashlib

import numpy as np
import pytest
import torch

from oracle import fp8_oracle as O

E4, E5 = torch.float8_e4m3fn, torch.float8_e5m2
HP = [torch.float32, torch.bfloat16, torch.float16]
_VIEW = {torch.float32: torch.int32, torch.bfloat16: torch.int16, torch.float16: torch.int16}


def _from_bits(arr: np.ndarray, dtype: torch.dtype) -> torch.Tensor:
    t = torch.from_numpy(arr.copy())
    return t.view(dtype)


def _sha(t: torch.Tensor) -> str:
    t = t.contiguous()
    v = {1: torch.uint8, 2: torch.int16, 4: torch.int32}[t.element_size()]
    return hashlib.sha256(t.view(v).numpy().tobytes()).hexdigest()


def _oracle_scale(amax: torch.Tensor, fmax: float) -> torch.Tensor:
    return torch.tensor(fmax, dtype=torch.float32) / torch.maximum(amax.float(), torch.tensor(1e-12))


def test_tensorwise_matches_reference_torch_ref(golden_dir):
    """Byte equality wherever the reference's torch ref used the same fp32 scale (its
    ``fmax / t`` is reciprocal-then-multiply, so the scale may be one ulp off) and its product was
    formed in fp32; the reference's own tolerances elsewhere."""
    z = np.load(golden_dir / "ref_quant.npz")
    n = int(z["num_tensorwise"])
    assert n >= 12
    exact_seen = 0
    for i in range(n):
        m, k, dti, fi, fp32_product = (int(v) for v in z[f"t{i}_meta"])
        dt, fp8 = HP[dti], (E4, E5)[fi]
        x = _from_bits(z[f"t{i}_x"], dt).reshape(m, k)
        q_ref = _from_bits(z[f"t{i}_q"], fp8).reshape(m, k)
        s_ref = _from_bits(z[f"t{i}_sinv"], torch.float32).reshape(())
        sc_ref = _from_bits(z[f"t{i}_scale"], torch.float32).reshape(())
        q, s = O.quant_tensorwise(x, fp8)
        torch.testing.assert_close(s, s_ref, rtol=3e-7, atol=0)
        same_scale = O.bits_equal_f32(_oracle_scale(x.float().abs().amax(), O.FP8_MAX[fp8]).reshape(()), sc_ref)
        if fp32_product and same_scale:
            assert O.bytes_equal(q, q_ref), f"case {i}: fp8 bytes differ from the reference's torch ref"
            exact_seen += 1
        else:
            tol = 1e-1 * float(x.float().abs().max())
            torch.testing.assert_close(q.float() * s, q_ref.float() * s_ref, rtol=1e-1, atol=tol)
            diff = (q.view(torch.uint8) != q_ref.view(torch.uint8)).float().mean()
            assert diff < 0.05, f"case {i}: {diff:.3f} of the bytes differ"
    assert exact_seen >= 3


def test_rowwise_matches_reference_torch_ref(golden_dir):
    z = np.load(golden_dir / "ref_quant.npz")
    n = int(z["num_rowwise"])
    assert n >= 12
    rows_exact = 0
    for i in range(n):
        meta = [int(v) for v in z[f"r{i}_meta"]]
        axis, dti, nd, shape = meta[0], meta[1], meta[2], meta[3:]
        dt = HP[dti]
        x = _from_bits(z[f"r{i}_x"], dt).reshape(*shape)
        q_ref = _from_bits(z[f"r{i}_q"], E4).reshape(*shape)
        sshape = list(shape)
        sshape[axis] = 1
        s_ref = _from_bits(z[f"r{i}_sinv"], torch.float32).reshape(*sshape)
        sc_ref = _from_bits(z[f"r{i}_scale"], torch.float32).reshape(*sshape)
        q, s = O.quant_rowwise(x, E4, axis)
        torch.testing.assert_close(s, s_ref, rtol=3e-7, atol=0)
        same = _oracle_scale(x.float().abs().amax(dim=axis, keepdim=True), 448.0).view(torch.int32) == sc_ref.view(
            torch.int32
        )
        neq = q.view(torch.uint8) != q_ref.view(torch.uint8)
        # every slice quantised with a bit-identical scale must be byte-identical
        assert not bool((neq & same.expand_as(neq)).any()), f"case {i}"
        assert neq.float().mean() < 0.05
        rows_exact += int(same.sum())
    assert rows_exact > 100


def test_grouped_gemm_ref_fixture(golden_dir):
    """Dequantise-then-matmul of the oracle stays within the reference's SNR gate of the
    reference's own fp32-accumulated grouped matmul on the unquantised operands."""
    z = np.load(golden_dir / "ref_grouped_gemm.npz")
    lens = torch.from_numpy(z["lens"])
    a = _from_bits(z["a"], torch.bfloat16).reshape(int(lens.sum()), 256)
    b = _from_bits(z["b"], torch.bfloat16).reshape(4, -1, 256)
    out_ref = _from_bits(z["out"], torch.bfloat16).reshape(a.shape[0], b.shape[1])
    offs = O.group_offs_from_lens(lens)
    q_row, _, s_row, _, _, _, _, _ = O.quant_segment_row_col(a, E4, 128, lens, offs)
    bq, bs = O.quant_block2d(b, E4)
    out = O.grouped_gemm_blockwise(q_row, s_row, bq, bs, offs, True, torch.bfloat16)
    assert O.snr_db(out_ref, out) > 25.0


def test_oracle_c1_frozen(golden_dir):
    z = np.load(golden_dir / "oracle_c1.npz")
    g0 = torch.Generator().manual_seed(0)
    A = torch.randn(256, 1024, generator=g0).to(torch.bfloat16)
    B = (torch.randn(512, 1024, generator=g0) * 0.02).to(torch.bfloat16)
    dig = [str(d) for d in z["digests"]]
    assert _sha(A) == dig[0] and _sha(B) == dig[1], "seeded inputs changed"
    a_row, a_s_row, a_col, a_s_col = O.quant_block1d_dual(A, E4)
    b_q, b_s = O.quant_block2d(B, E4)
    C = O.gemm_blockwise_nt(a_row, a_s_row, b_q, b_s, torch.bfloat16)
    assert [_sha(a_row), _sha(a_col), _sha(b_q), _sha(C)] == dig[2:]
    assert O.bits_equal_f32(a_s_row, _from_bits(z["a_s_row"], torch.float32).reshape(256, 8))
    assert O.bits_equal_f32(a_s_col, _from_bits(z["a_s_col"], torch.float32).reshape(2, 1024))
    assert O.bits_equal_f32(b_s, _from_bits(z["b_s"], torch.float32).reshape(4, 8))


@pytest.mark.parametrize("shape", [(1, 1), (128, 128), (129, 257), (300, 333)])
def test_oracle_roundtrip_and_shapes(shape):
    g = torch.Generator().manual_seed(7)
    x = torch.randn(*shape, generator=g).to(torch.bfloat16)
    for axis in (0, 1):
        q, s = O.quant_block1d(x, E4, axis)
        assert q.shape == x.shape
        want = (shape[0], O.cdiv(shape[1], 128)) if axis == 1 else (O.cdiv(shape[0], 128), shape[1])
        assert tuple(s.shape) == want
        d = O.dequant_block1d(q, s, axis)
        torch.testing.assert_close(d, x.float(), rtol=1e-1, atol=1e-1)
    q, s = O.quant_block2d(x, E4)
    assert tuple(s.shape) == (O.cdiv(shape[0], 128), O.cdiv(shape[1], 128))
    torch.testing.assert_close(O.dequant_block2d(q, s), x.float(), rtol=1e-1, atol=1e-1)


def test_oracle_scale_formula_is_two_divisions():
    """scale_inv = 1/(448/amax), not amax/448: the two differ in the last bit for many inputs."""
    g = torch.Generator().manual_seed(3)
    amax = torch.rand(4096, generator=g) * 8 + 1e-3
    s = torch.tensor(448.0) / amax
    two_div = torch.tensor(1.0) / s
    one_div = amax / torch.tensor(448.0)
    assert (two_div != one_div).float().mean() > 0.2
    x = amax.reshape(-1, 1).repeat(1, 128).to(torch.float32)
    _, s_inv = O.quant_block1d(x, E4, 1)
    assert O.bits_equal_f32(s_inv.reshape(-1), two_div)


def test_segment_layout():
    lens = torch.tensor([100, 0, 256, 1, 300], dtype=torch.int64)
    offs = O.group_offs_from_lens(lens)
    g = torch.Generator().manual_seed(11)
    x = torch.randn(int(offs[-1]) + 3, 256, generator=g).to(torch.bfloat16)
    q_row, q_col, s_row, s_col, vk_lens, vk_offs, written, pad_used = O.quant_segment_row_col(x, E4, 128, lens, offs)
    assert vk_lens.tolist() == [128, 0, 256, 128, 384] and vk_offs.tolist() == [0, 128, 128, 384, 512, 896]
    assert q_col.shape == (x.shape[0] + 5 * 128, 256) and s_col.shape == (O.cdiv(x.shape[0] + 640, 128), 256)
    assert s_row.shape == (2, x.shape[0]) and pad_used == 896
    # padding rows are zero bytes; group 3 (one row) sits at padded row 384
    assert int(q_col[100:128].view(torch.uint8).max()) == 0
    one_row_q, one_row_s = O.quant_block1d(x[356:357], E4, 0)
    assert O.bytes_equal(q_col[384:385], one_row_q) and O.bits_equal_f32(s_col[3:4], one_row_s)
    # row part equals the ungrouped 1x128 quantisation
    qr, sr = O.quant_block1d(x, E4, 1)
    m = int(offs[-1])
    assert O.bytes_equal(q_row[:m], qr[:m]) and O.bits_equal_f32(s_row[:, :m].contiguous(), sr[:m].t().contiguous())
    assert written.sum() == m
