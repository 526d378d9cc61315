"""B200-native triangle self-attention: a drop-in for ``trifast.triangle_attention``."""

from .torch import triangle_attention  # noqa: F401

__all__ = ["triangle_attention"]
