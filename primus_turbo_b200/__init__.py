"""B200-native FP8 quantize / GEMM / grouped-GEMM behind the Primus-Turbo ops surface.

``primus_turbo_b200.pytorch`` mirrors ``primus_turbo.pytorch`` for the FP8 hot path;
``install_as_primus_turbo()`` registers it under the reference's import name.
"""

__version__ = "0.1.0"


def install_as_primus_turbo() -> None:
    """Make ``import primus_turbo.pytorch`` resolve to this package (drop-in use)."""
    import importlib
    import sys

    pt = importlib.import_module("primus_turbo_b200.pytorch")
    root = sys.modules[__name__]
    sys.modules.setdefault("primus_turbo", root)
    sys.modules.setdefault("primus_turbo.pytorch", pt)
    for name, mod in list(sys.modules.items()):
        if name.startswith("primus_turbo_b200.pytorch."):
            sys.modules.setdefault("primus_turbo" + name[len("primus_turbo_b200") :], mod)
