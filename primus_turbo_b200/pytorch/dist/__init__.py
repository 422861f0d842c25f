from .fp8_alltoall import FP8AllToAll  # noqa: F401

__all__ = ["FP8AllToAll"]
