"""Generate the committed golden fixtures in this folder.  Run from the repository root, in a
checkout that has the reference project mounted (it is only needed here, never at test time):

    python tests/golden/make_golden.py /path/to/reference

Two families of fixtures are written:

* ``ref_*.npz`` -- outputs of the REFERENCE's own torch test references
  (tests/pytorch/ref/quantization_ref.py and tests/pytorch/ref/gemm_ref.py, executed unmodified
  on CPU).  For fp32 inputs (tensorwise) and for every dtype (rowwise, whose scale tensor is
  dimensioned so torch promotes the product to fp32) these are fp32 statements of
  ``q = cast(clamp(x * scale))``.  torch evaluates ``fmax / tensor`` as ``reciprocal(tensor) * fmax``
  (two roundings), so the stored reference scale can differ from the kernels' single IEEE division
  in the last bit; the fixtures therefore keep the reference's scale as well, and the tests demand
  byte equality wherever the two scales agree bit for bit and the reference's tolerance elsewhere.  For
  16-bit tensorwise inputs the reference's torch code multiplies in 16-bit precision (a 0-dim
  fp32 scale does not promote), which its own tests absorb with tolerances; those cases are stored
  with ``exact = 0`` and compared the way the reference compares them.
* ``ref_blockwise_interp.npz`` -- outputs of the REFERENCE's own Triton blockwise quantise kernels
  (primus_turbo/triton/quantization/quant_blockwise.py, imported unmodified and executed on CPU
  tensors by Triton's interpreter, ``TRITON_INTERPRET=1``): 1-D blocks along both axes, the dual
  kernel, the 128x128 weight kernel and the grouped ``segment_m_row_col`` kernel, on shapes with
  partial tiles, empty and one-row groups.  Outputs are pre-filled with sentinels so that positions the
  reference never writes are recorded too.  These pin the layouts (padded segment rows, the
  ``[ceil(N/128), M]`` order of the row scales, padded offsets), every scale bit for bit, and the FP8
  bytes wherever the interpreter's float-to-e4m3 cast is sound: that cast (numpy emulation, not the
  GPU instruction) rounds ties away from zero, mis-rounds values that round up into the next binade
  and truncates subnormals, so the tests skip exactly those positions and demand equality elsewhere.
* ``oracle_c1.npz`` -- the CPU oracle on the small benchmark configuration (A bf16 [256,1024]
  ~N(0,1), B bf16 [512,1024] ~N(0,0.02), seed 0): scales in full, FP8 payloads as SHA-256 digests
  plus their leading bytes, bf16 output digest.  It freezes the oracle and lets the GPU tests check
  the CUDA path against committed bytes.
"""

from __future__ import annotations

import hashlib
import importlib.util
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
sys.path.insert(0, str(REPO))

from oracle import fp8_oracle as O  # noqa: E402

E4, E5 = torch.float8_e4m3fn, torch.float8_e5m2


def _load_reference_refs(ref_root: Path):
    """Import the reference's torch test references with only the enum module stubbed in."""
    from primus_turbo_b200.pytorch.core import low_precision as lp

    for name in ("primus_turbo", "primus_turbo.pytorch", "primus_turbo.pytorch.core"):
        sys.modules.setdefault(name, types.ModuleType(name))
    sys.modules["primus_turbo.pytorch.core.low_precision"] = lp
    mods = {}
    for stem in ("quantization_ref", "gemm_ref"):
        spec = importlib.util.spec_from_file_location(stem, ref_root / "tests" / "pytorch" / "ref" / f"{stem}.py")
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mods[stem] = mod
    return mods, lp


def _bits(t: torch.Tensor) -> np.ndarray:
    t = t.contiguous()
    if t.element_size() == 1:
        return t.view(torch.uint8).numpy()
    if t.element_size() == 2:
        return t.view(torch.int16).numpy()
    return t.view(torch.int32).numpy()


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(_bits(t).tobytes()).hexdigest()


SENT_Q = 0x55  # byte pre-filled into FP8 outputs (positions the reference leaves unwritten keep it)
SENT_S = -777.0  # value pre-filled into scale outputs


def write_blockwise_interp(ref_root: Path) -> None:
    """Run the reference's Triton blockwise quantise kernels on CPU tensors through the interpreter.
    Must run in a process started with TRITON_INTERPRET=1 (main() re-executes itself for this)."""
    import os
    import subprocess

    if os.environ.get("TRITON_INTERPRET") != "1":
        env = dict(os.environ, TRITON_INTERPRET="1")
        subprocess.run([sys.executable, __file__, str(ref_root), "--blockwise-only"], check=True, env=env)
        return
    spec = importlib.util.spec_from_file_location(
        "ref_quant_blockwise", ref_root / "primus_turbo" / "triton" / "quantization" / "quant_blockwise.py")
    qb = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(qb)
    gen = torch.Generator().manual_seed(77)
    out = {}

    def q_buf(*shape):
        return torch.full(shape, SENT_Q, dtype=torch.uint8).view(E4)

    def s_buf(*shape):
        return torch.full(shape, SENT_S, dtype=torch.float32)

    cd = lambda a, b: (a + b - 1) // b  # noqa: E731
    # 1-D blocks, both axes, and the dual kernel: partial tiles in both dimensions
    M, N = 200, 192
    x = torch.randn(M, N, generator=gen).to(torch.bfloat16)
    x[5, :128] *= 1e-6  # a block below the 1e-4 amax floor
    out["b1_x"] = _bits(x)
    for axis in (1, 0):
        q, s = q_buf(M, N), s_buf(*((M, cd(N, 128)) if axis == 1 else (cd(M, 128), N)))
        qb.quant_fp8_blockwise_kernel[(cd(M, 128), cd(N, 128))](x, q, s, M, N, BLOCK_SIZE=128, FP8_MAX=448.0, AXIS=axis)
        out[f"b1_q_axis{axis}"], out[f"b1_s_axis{axis}"] = _bits(q), _bits(s)
    qr, sr, qc, sc = q_buf(M, N), s_buf(M, cd(N, 128)), q_buf(M, N), s_buf(cd(M, 128), N)
    qb.quant_fp8_blockwise_dual_kernel[(cd(M, 128), cd(N, 128))](x, qr, sr, qc, sc, M, N, BLOCK_SIZE=128, FP8_MAX=448.0)
    out["dual_q_row"], out["dual_s_row"], out["dual_q_col"], out["dual_s_col"] = _bits(qr), _bits(sr), _bits(qc), _bits(sc)
    # 128x128 weight blocks, batched
    B, Mw, Nw = 2, 136, 192
    w = (torch.randn(B, Mw, Nw, generator=gen) * 0.02).to(torch.bfloat16)
    q, s = q_buf(B, Mw, Nw), s_buf(B, cd(Mw, 128), cd(Nw, 128))
    qb.quant_fp8_blockwise_for_weight_kernel[(B, cd(Mw, 128), cd(Nw, 128))](w, q, s, Mw, Nw, BLOCK_SIZE=128, FP8_MAX=448.0)
    out["w_x"], out["w_q"], out["w_s"] = _bits(w), _bits(q), _bits(s)
    # grouped segment row + column: empty group, one-row group, lengths around 128, rows past the last group
    lens = torch.tensor([100, 0, 257, 1, 129], dtype=torch.int64)
    offs = O.group_offs_from_lens(lens)
    G, Ms, Ns = lens.numel(), int(offs[-1]) + 6, 192
    xs = torch.randn(Ms, Ns, generator=gen).to(torch.bfloat16)
    vk_lens = ((lens + 127) // 128) * 128  # primus_turbo/pytorch/kernels/quantization/quantization_impl.py:428-430
    vk_offs = torch.zeros(G + 1, dtype=torch.int64)
    vk_offs[1:] = torch.cumsum(vk_lens, 0)
    m_pad = Ms + G * 128
    qr, qc = q_buf(Ms, Ns), q_buf(m_pad, Ns)
    sr, sc = s_buf(cd(Ns, 128), Ms), s_buf(cd(m_pad, 128), Ns)
    qb.quant_fp8_blockwise_segment_m_row_col_kernel[(cd(m_pad, 128), cd(Ns, 128))](
        xs, qr, qc, sr, sc, offs, vk_offs, Ms, Ns, G, BLOCK_SIZE=128, FP8_MAX=448.0)
    out["seg_x"], out["seg_lens"] = _bits(xs), lens.numpy()
    out["seg_q_row"], out["seg_q_col"], out["seg_s_row"], out["seg_s_col"] = _bits(qr), _bits(qc), _bits(sr), _bits(sc)
    out["seg_vk_offs"] = vk_offs.numpy()
    np.savez_compressed(HERE / "ref_blockwise_interp.npz", **out)


def main(ref_root: str) -> None:
    mods, lp = _load_reference_refs(Path(ref_root))
    qref = mods["quantization_ref"]
    G = lp.ScalingGranularity
    gen = torch.Generator().manual_seed(1234)

    # ---- reference torch refs: tensorwise + rowwise --------------------------------------------
    cases = {}
    idx = 0
    for dt_name, dt in (("f32", torch.float32), ("bf16", torch.bfloat16), ("f16", torch.float16)):
        for shape in ((24, 200), (1, 111), (9, 128)):
            for fp8_name, fp8 in (("e4m3", E4), ("e5m2", E5)):
                x = (torch.randn(*shape, generator=gen) * 3.0).to(dt)
                q, sc, sinv = qref.quantize_fp8_ref(x, fp8, G.TENSORWISE)
                cases[f"t{idx}_scale"] = _bits(sc.reshape(1))
                cases[f"t{idx}_x"] = _bits(x)
                cases[f"t{idx}_q"] = _bits(q)
                cases[f"t{idx}_sinv"] = _bits(sinv.reshape(1))
                cases[f"t{idx}_meta"] = np.array([shape[0], shape[1], ["f32", "bf16", "f16"].index(dt_name),
                                                  ["e4m3", "e5m2"].index(fp8_name), 1 if dt == torch.float32 else 0])
                idx += 1
    cases["num_tensorwise"] = np.array(idx)
    ridx = 0
    for dt_name, dt in (("f32", torch.float32), ("bf16", torch.bfloat16), ("f16", torch.float16)):
        for shape in ((24, 200), (3, 10, 96)):
            for axis in range(-len(shape), 0):
                x = (torch.randn(*shape, generator=gen) * 0.5).to(dt)
                q, sc, sinv = qref.quantize_fp8_ref(x, E4, G.ROWWISE, axis=axis)
                cases[f"r{ridx}_scale"] = _bits(sc)
                cases[f"r{ridx}_x"] = _bits(x)
                cases[f"r{ridx}_q"] = _bits(q)
                cases[f"r{ridx}_sinv"] = _bits(sinv)
                cases[f"r{ridx}_meta"] = np.array([axis, ["f32", "bf16", "f16"].index(dt_name), len(shape), *shape])
                ridx += 1
    cases["num_rowwise"] = np.array(ridx)
    np.savez_compressed(HERE / "ref_quant.npz", **cases)

    # ---- reference grouped GEMM ref on dequantised operands (tests/pytorch/ref/gemm_ref.py:13-24)
    gref = mods["gemm_ref"]
    lens = torch.tensor([5, 0, 17, 10], dtype=torch.int64)
    a = torch.randn(int(lens.sum()), 256, generator=gen).to(torch.bfloat16)
    b = (torch.randn(4, 48, 256, generator=gen) * 0.02).to(torch.bfloat16)
    out = gref.grouped_gemm_ref(a, b, lens, trans_b=True)
    np.savez_compressed(HERE / "ref_grouped_gemm.npz", a=_bits(a), b=_bits(b), lens=lens.numpy(), out=_bits(out))

    # ---- reference Triton blockwise kernels under the interpreter --------------------------------
    write_blockwise_interp(Path(ref_root))

    # ---- oracle on the small benchmark configuration ------------------------------------------------
    g0 = torch.Generator().manual_seed(0)
    A = torch.randn(256, 1024, generator=g0).to(torch.bfloat16)
    B = (torch.randn(512, 1024, generator=g0) * 0.02).to(torch.bfloat16)
    a_row, a_s_row, a_col, a_s_col = O.quant_block1d_dual(A, E4)
    b_q, b_s = O.quant_block2d(B, E4)
    C = O.gemm_blockwise_nt(a_row, a_s_row, b_q, b_s, torch.bfloat16)
    np.savez_compressed(
        HERE / "oracle_c1.npz",
        a_s_row=_bits(a_s_row), a_s_col=_bits(a_s_col), b_s=_bits(b_s),
        a_row_head=_bits(a_row).reshape(-1)[:4096], a_col_head=_bits(a_col).reshape(-1)[:4096],
        b_q_head=_bits(b_q).reshape(-1)[:4096], c_head=_bits(C).reshape(-1)[:4096],
        digests=np.array([sha(A), sha(B), sha(a_row), sha(a_col), sha(b_q), sha(C)]),
    )
    print("wrote", sorted(p.name for p in HERE.glob("*.npz")))


if __name__ == "__main__":
    if len(sys.argv) == 3 and sys.argv[2] == "--blockwise-only":
        write_blockwise_interp(Path(sys.argv[1]))
    elif len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/reference")
    else:
        main(sys.argv[1])
