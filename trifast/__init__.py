"""Drop-in name: ``import trifast`` resolves to the B200-native implementation.

Same public surface as latkins/trifast (``src/trifast/__init__.py:1-3``):
``trifast.triangle_attention`` plus ``trifast.utils.gen_tensors`` and
``trifast.torch.triangle_attention``.
"""

from trifast_b200 import triangle_attention  # noqa: F401

__all__ = ["triangle_attention"]
