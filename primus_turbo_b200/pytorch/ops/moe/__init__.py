from .permutation import token_permute, token_unpermute  # noqa: F401

__all__ = ["token_permute", "token_unpermute"]
