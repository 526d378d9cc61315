"""``trifast.utils`` of the reference (``src/trifast/utils.py``), served by trifast_b200."""

from trifast_b200.utils import (clone_and_clear_grad, disable_tf32, enable_tf32,  # noqa: F401
                                gen_tensors)
