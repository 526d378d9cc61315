"""``trifast.torch`` of the reference (``src/trifast/torch.py``), served by trifast_b200."""

from trifast_b200.torch import (_triangle_attention, triangle_attention,  # noqa: F401
                                triangle_attention_bwd)
