"""Input generator and small helpers, behaviour-compatible with the reference's
``src/trifast/utils.py`` (``gen_tensors`` :5-33, ``clone_and_clear_grad`` :36-44,
``disable_tf32`` / ``enable_tf32`` :47-88).
"""

from __future__ import annotations

import contextlib
from functools import wraps

import torch


def gen_tensors(n, d, h, use_mask, device, dtype, batch=1, std=1.0):
    """Seed-driven q, k, v, bias and mask.

    Draw order (q, k, v, bias, then mask) and distributions match the reference
    generator, so a given ``torch.manual_seed`` yields the same tensors: q, k, v
    ~ N(0, std) of shape (batch, h, n, n, d), bias ~ N(0, std) of shape
    (batch, h, n, n), all leaf tensors requiring grad; mask is Bernoulli(0.5)
    bool of shape (batch, n, n) (True = key masked out) or all-False when
    ``use_mask`` is false.
    """
    def draw(*shape):
        return torch.normal(0, std, shape, device=device, dtype=dtype, requires_grad=True)

    q = draw(batch, h, n, n, d)
    k = draw(batch, h, n, n, d)
    v = draw(batch, h, n, n, d)
    b = draw(batch, h, n, n)
    if use_mask:
        m = torch.randint(0, 2, (batch, n, n), device=device, dtype=torch.bool)
    else:
        m = torch.zeros((batch, n, n), device=device, dtype=torch.bool)
    return q, k, v, b, m


def clone_and_clear_grad(*tensors):
    """Return clones of the tensors' gradients and reset them to None."""
    out = []
    for t in tensors:
        out.append(None if t.grad is None else t.grad.clone())
        t.grad = None
    return tuple(out)


@contextlib.contextmanager
def _tf32(flag):
    saved = (torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32)
    torch.backends.cuda.matmul.allow_tf32 = flag
    torch.backends.cudnn.allow_tf32 = flag
    try:
        yield
    finally:
        torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32 = saved


def disable_tf32(fn):
    """Decorator: run ``fn`` with TF32 matmuls off, restoring the flags after."""
    @wraps(fn)
    def inner(*a, **kw):
        with _tf32(False):
            return fn(*a, **kw)
    return inner


def enable_tf32(fn):
    """Decorator: run ``fn`` with TF32 matmuls on, restoring the flags after."""
    @wraps(fn)
    def inner(*a, **kw):
        with _tf32(True):
            return fn(*a, **kw)
    return inner
