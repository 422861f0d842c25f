from .linear_fp8 import Float8Linear

__all__ = ["Float8Linear"]
