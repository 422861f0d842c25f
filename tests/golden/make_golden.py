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
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/reference")
    main(sys.argv[1])
