"""B200-native triangle self-attention: a drop-in for ``trifast.triangle_attention``."""

from .torch import triangle_attention, triangle_attention_ending_node  # noqa: F401

__all__ = ["triangle_attention", "triangle_attention_ending_node"]
