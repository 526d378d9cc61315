"""Operator boundary: custom ops + autograd for triangle self-attention.

Mirrors the reference's ``src/trifast/torch.py``: a forward op returning
``(o, lse)`` (``_triangle_attention``, :17-65), a backward op returning
``(dq, dk, dv, db, dmask)`` (``triangle_attention_bwd``, :68-182), autograd glue
(:185-217) and the public ``triangle_attention`` (:220-228).  The ops live in the
``trifast_b200`` namespace so the reference can be imported beside them.  All
compute happens in the CUDA library behind the C ABI (``_lib.py``); this module
only checks arguments, allocates outputs and passes pointers and strides.
"""

from __future__ import annotations

import ctypes as C

import torch

from . import _lib


def _row_vector_ok(t: torch.Tensor) -> bool:
    """Strides the kernels accept for (b, h, i, j, d): d contiguous, every other
    stride a multiple of 16 bytes, base 16-byte aligned."""
    if t.stride(-1) != 1 or t.data_ptr() % 16:
        return False
    es = t.element_size()
    # a stride of 0 (an expanded dimension) cannot be described to TMA
    return all((s > 0 or n == 1) and (s * es) % 16 == 0 for s, n in zip(t.stride()[:-1], t.shape[:-1])) \
        and t.stride(-2) >= t.shape[-1]


def _dense(t: torch.Tensor) -> torch.Tensor:
    """A contiguous tensor with the canonical strides.  ``contiguous()`` alone keeps whatever
    strides the extent-1 dimensions came with (PyTorch ignores them), but the C side reads
    every stride."""
    t = t.contiguous()
    want, acc = [], 1
    for n in reversed(t.shape):
        want.append(acc)
        acc *= max(n, 1)
    want = tuple(reversed(want))
    return t if t.stride() == want else t.as_strided(t.shape, want)


def _prep5(t):
    return t if _row_vector_ok(t) else _dense(t)


def _prep4(t):
    return t if (t.stride(-1) == 1 and all(s >= 0 for s in t.stride())
                 and t.stride(-2) >= t.shape[-1]) else _dense(t)


def _prep_mask(m):
    if m.dtype != torch.bool:
        raise TypeError("mask must be a bool tensor (True = key masked out)")
    if m.stride(-1) != 1 or m.stride(-2) < m.shape[-1]:
        m = _dense(m)
    return m.view(torch.uint8)


def _check_inputs(q, k, v, b, mask):
    if q.dim() != 5:
        raise ValueError(f"q must be (batch, heads, rows, n, d); got {tuple(q.shape)}")
    bs, h, n_rows, n, d = q.shape
    if k.shape != q.shape or v.shape != q.shape:
        raise ValueError("q, k and v must have the same shape")
    if tuple(b.shape) != (bs, h, n, n):
        raise ValueError(f"bias must be {(bs, h, n, n)}; got {tuple(b.shape)}")
    if tuple(mask.shape) != (bs, n_rows, n):
        raise ValueError(f"mask must be {(bs, n_rows, n)}; got {tuple(mask.shape)}")
    if not (q.dtype == k.dtype == v.dtype == b.dtype):
        raise TypeError("q, k, v and bias must share one dtype")
    for name, t in (("k", k), ("v", v), ("bias", b), ("mask", mask)):
        if t.device != q.device:
            raise ValueError(f"{name} is on {t.device} but q is on {q.device}: every tensor "
                             "must live on the same CUDA device")
    if not q.is_cuda:
        raise RuntimeError("trifast_b200 runs on CUDA devices only (there is no CPU path)")
    return bs, h, n_rows, n, d


def _check_saved(do, q, o, l):
    """The backward's extra arguments: dO and o like q, lse fp32 (b, h, rows, n)."""
    bs, h, n_rows, n, d = q.shape
    for name, t in (("do", do), ("o", o)):
        if tuple(t.shape) != tuple(q.shape) or t.dtype != q.dtype:
            raise ValueError(f"{name} must be {tuple(q.shape)} {q.dtype}; got {tuple(t.shape)} {t.dtype}")
        if t.device != q.device:
            raise ValueError(f"{name} is on {t.device} but q is on {q.device}")
    if tuple(l.shape) != (bs, h, n_rows, n) or l.dtype != torch.float32:
        raise ValueError(f"lse must be float32 {(bs, h, n_rows, n)}; got {l.dtype} {tuple(l.shape)}")
    if l.device != q.device:
        raise ValueError(f"lse is on {l.device} but q is on {q.device}")


def _stream(t):
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


@torch.library.custom_op("trifast_b200::triangle_attention", mutates_args=(), device_types="cuda")
def _triangle_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, b: torch.Tensor,
                        mask: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    bs, h, n_rows, n, d = _check_inputs(q, k, v, b, mask)
    lib = _lib.load()
    _lib.raise_if_device_gave_up(q.device)
    q, k, v, b = _prep5(q), _prep5(k), _prep5(v), _prep4(b)
    m8 = _prep_mask(mask)
    o = torch.empty((bs, h, n_rows, n, d), dtype=q.dtype, device=q.device)
    lse = torch.empty((bs, h, n_rows, n), dtype=torch.float32, device=q.device)
    shp = _lib.make_shape(bs, h, n, n_rows, d, q.dtype)
    ws_bytes = lib.trifast_forward_workspace_bytes(C.byref(shp))   # 0 on the CUDA-core plan
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device) if ws_bytes else None
    with torch.cuda.device(q.device):
        rc = lib.trifast_forward(C.byref(shp), C.byref(_lib.t5(q)), C.byref(_lib.t5(k)),
                                 C.byref(_lib.t5(v)), C.byref(_lib.t4(b)),
                                 C.byref(_lib.mask_view(m8)), C.byref(_lib.t5(o)),
                                 C.c_void_p(lse.data_ptr()),
                                 C.c_void_p(ws.data_ptr() if ws is not None else None),
                                 C.c_size_t(ws_bytes), _stream(q))
    _lib.check(rc, "trifast_forward")
    _lib.snapshot_status(q.device, _stream(q))
    return o, lse


@_triangle_attention.register_fake
def _(q, k, v, b, mask):
    bs, h, n_rows, n, d = q.shape
    return (q.new_empty((bs, h, n_rows, n, d)),
            q.new_empty((bs, h, n_rows, n), dtype=torch.float32))


@torch.library.custom_op("trifast_b200::triangle_attention_backward", mutates_args=(),
                         device_types="cuda")
def triangle_attention_bwd(do: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                           b: torch.Tensor, o: torch.Tensor, l: torch.Tensor, mask: torch.Tensor
                           ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
                                      torch.Tensor]:
    bs, h, n_rows, n, d = _check_inputs(q, k, v, b, mask)
    _check_saved(do, q, o, l)
    lib = _lib.load()
    _lib.raise_if_device_gave_up(q.device)
    do, q, k, v, o, b = _prep5(do), _prep5(q), _prep5(k), _prep5(v), _prep5(o), _prep4(b)
    m8 = _prep_mask(mask)
    l = l.contiguous()
    dq, dk, dv = (torch.empty((bs, h, n_rows, n, d), dtype=q.dtype, device=q.device)
                  for _ in range(3))
    db = torch.empty((bs, h, n, n), dtype=q.dtype, device=q.device)
    dmask = torch.zeros_like(mask)   # mask has no gradient; the reference returns zeros too
    shp = _lib.make_shape(bs, h, n, n_rows, d, q.dtype)
    ws_bytes = lib.trifast_backward_workspace_bytes(C.byref(shp))
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
    with torch.cuda.device(q.device):
        rc = lib.trifast_backward(
            C.byref(shp), C.byref(_lib.t5(do)), C.byref(_lib.t5(q)), C.byref(_lib.t5(k)),
            C.byref(_lib.t5(v)), C.byref(_lib.t4(b)), C.byref(_lib.mask_view(m8)),
            C.byref(_lib.t5(o)), C.c_void_p(l.data_ptr()), C.byref(_lib.t5(dq)),
            C.byref(_lib.t5(dk)), C.byref(_lib.t5(dv)), C.byref(_lib.t4(db)),
            C.c_void_p(ws.data_ptr()), C.c_size_t(ws_bytes), _stream(q))
    _lib.check(rc, "trifast_backward")
    _lib.snapshot_status(q.device, _stream(q))
    return dq, dk, dv, db, dmask


@triangle_attention_bwd.register_fake
def _(do, q, k, v, b, o, l, mask):
    return (torch.empty_like(q, memory_format=torch.contiguous_format),
            torch.empty_like(k, memory_format=torch.contiguous_format),
            torch.empty_like(v, memory_format=torch.contiguous_format),
            torch.empty_like(b, memory_format=torch.contiguous_format),
            torch.empty_like(mask, memory_format=torch.contiguous_format))


def _setup_context(ctx, inputs, output):
    q, k, v, b, mask = inputs
    o, l = output
    ctx.save_for_backward(q, k, v, b, mask, o, l)


def _backward(ctx, do, _dlse):
    q, k, v, b, mask, o, l = ctx.saved_tensors
    dq, dk, dv, db, _ = triangle_attention_bwd(do, q, k, v, b, o, l, mask)
    return dq, dk, dv, db, None


_triangle_attention.register_autograd(_backward, setup_context=_setup_context)


def triangle_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, b: torch.Tensor,
                       mask: torch.Tensor) -> torch.Tensor:
    """Fused triangle self-attention (around the starting node).

    q, k, v: (*batch, heads, n, n, d); b (pair bias): (*batch, heads, n, n), shared
    by all rows; mask: (*batch, n, n) bool, True = key masked out for that row.
    ``*batch`` is any number of leading dimensions, including none (the reference
    takes exactly one, src/trifast/torch.py:29 notes the rest as to do); they are
    folded into one batch dimension for the kernels.  Returns o with the shape and
    dtype of q.  Differentiable in q, k, v and b.
    """
    if q.dim() == 5:
        o, _ = _triangle_attention(q, k, v, b, mask)
        return o
    if q.dim() < 4:
        raise ValueError(f"q must be (*batch, heads, n, n, d); got {tuple(q.shape)}")
    lead = q.shape[:-4]
    if k.shape != q.shape or v.shape != q.shape or b.shape[:-3] != lead or mask.shape[:-2] != lead:
        raise ValueError("q, k, v, bias and mask must share their leading batch dimensions")
    fold = lambda t, keep: t.reshape((-1,) + tuple(t.shape[-keep:]))
    o, _ = _triangle_attention(fold(q, 4), fold(k, 4), fold(v, 4), fold(b, 3), fold(mask, 2))
    return o.reshape(q.shape)


def triangle_attention_ending_node(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                                   b: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """Triangle self-attention around the ending node:

        o[i, j] = sum_k softmax_k(q[i, j] . k[k, j] / sqrt(d) + b[k, i] + mask[k, j]) v[k, j]

    (keys run along the first pair index).  It is the starting-node operator on the
    pair-transposed problem, o = T(triangle_attention(T(q), T(k), T(v), b^T, mask^T)), with T
    the swap of the two pair dimensions; the transposed q, k, v are read through their
    strides, nothing is copied but the small bias and mask.  The reference lists this
    variant as planned (README.md:104 there); shapes and dtypes as in triangle_attention.
    """
    t = lambda x: x.transpose(-3, -2)
    o = triangle_attention(t(q), t(k), t(v), b.transpose(-1, -2), mask.transpose(-1, -2))
    return t(o)
