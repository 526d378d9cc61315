"""Row-sharded triangle attention over the GPUs of one box.

Pair rows i are independent in the forward and in dq, dk, dv; only the bias
gradient db sums over rows.  Rank r therefore holds a contiguous block of rows
of q, k, v, mask (and produces the same rows of o, dq, dk, dv), the pair bias is
replicated, and the single exchange of the whole step is one all-reduce of the
fp32 db partial, issued as soon as the db kernels finish and overlapped with
the dq/dk/dv kernels.  The reference (latkins/trifast) is single-GPU; this layer
has no counterpart there.

The compute steps come from a ``kernels`` object so that the host logic
(sharding, ordering, the all-reduce) can be exercised with CPU tensors under
the ``gloo`` backend; the default is the CUDA library.
"""

from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import _lib
from .torch import (_check_inputs, _check_saved, _prep4, _prep5, _prep_mask, _stream,
                    _triangle_attention)


def shard_rows(n: int, rank: int, world: int) -> slice:
    """Contiguous, balanced row block of ``rank``: the first ``n % world`` ranks
    hold one row more."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, rem = divmod(n, world)
    start = rank * base + min(rank, rem)
    return slice(start, start + base + (1 if rank < rem else 0))


class CudaKernels:
    """The three backward steps and the forward, through the C ABI."""

    def forward(self, q, k, v, b, mask):
        return _triangle_attention(q, k, v, b, mask)

    def __init__(self, share_gpu: bool = False):
        # under a process group the all-reduce of db runs beside the dq/dk/dv kernels:
        # they then leave a few SMs free for it (TRIFAST_FLAG_SHARE_GPU)
        self.flags = _lib.flags_choice() | (_lib.FLAG_SHARE_GPU if share_gpu else 0)

    def _common(self, do, q, k, v, b, mask):
        bs, h, n_rows, n, d = _check_inputs(q, k, v, b, mask)
        shp = _lib.make_shape(bs, h, n, n_rows, d, q.dtype, flags=self.flags)
        t = [_prep5(x) for x in (do, q, k, v)]
        return shp, t, _prep4(b), _prep_mask(mask), (bs, h, n_rows, n, d)

    def backward_db(self, do, q, k, v, b, mask, o, lse):
        """Returns (db_f32 partial over the local rows, workspace holding delta)."""
        lib = _lib.load()
        _check_saved(do, q, o, lse)
        _lib.raise_if_device_gave_up(q.device)
        shp, (do, q, k, v), b, m8, (bs, h, n_rows, n, d) = self._common(do, q, k, v, b, mask)
        o, lse = _prep5(o), lse.contiguous()
        nbytes = lib.trifast_backward_workspace_bytes(C.byref(shp))
        ws = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
        db_f32 = torch.empty((bs, h, n, n), dtype=torch.float32, device=q.device)
        with torch.cuda.device(q.device):
            rc = lib.trifast_backward_db(
                C.byref(shp), C.byref(_lib.t5(do)), C.byref(_lib.t5(q)), C.byref(_lib.t5(k)),
                C.byref(_lib.t5(v)), C.byref(_lib.t4(b)), C.byref(_lib.mask_view(m8)),
                C.byref(_lib.t5(o)), C.c_void_p(lse.data_ptr()), C.c_void_p(db_f32.data_ptr()),
                C.c_void_p(ws.data_ptr()), C.c_size_t(nbytes), _stream(q))
        _lib.check(rc, "trifast_backward_db")
        return db_f32, ws

    def backward_dqkv(self, do, q, k, v, b, mask, lse, ws):
        lib = _lib.load()
        shp, (do, q, k, v), b, m8, (bs, h, n_rows, n, d) = self._common(do, q, k, v, b, mask)
        lse = lse.contiguous()
        dq, dk, dv = (torch.empty((bs, h, n_rows, n, d), dtype=q.dtype, device=q.device)
                      for _ in range(3))
        with torch.cuda.device(q.device):
            rc = lib.trifast_backward_dqkv(
                C.byref(shp), C.byref(_lib.t5(do)), C.byref(_lib.t5(q)), C.byref(_lib.t5(k)),
                C.byref(_lib.t5(v)), C.byref(_lib.t4(b)), C.byref(_lib.mask_view(m8)),
                C.c_void_p(lse.data_ptr()), C.byref(_lib.t5(dq)), C.byref(_lib.t5(dk)),
                C.byref(_lib.t5(dv)), C.c_void_p(ws.data_ptr()), C.c_size_t(ws.numel()),
                _stream(q))
        _lib.check(rc, "trifast_backward_dqkv")
        _lib.snapshot_status(q.device, _stream(q))
        return dq, dk, dv

    def db_finalize(self, db_f32, dtype):
        lib = _lib.load()
        bs, h, n, _ = db_f32.shape
        db = torch.empty((bs, h, n, n), dtype=dtype, device=db_f32.device)
        shp = _lib.make_shape(bs, h, n, n, 32, dtype)   # d is irrelevant to the cast
        with torch.cuda.device(db_f32.device):
            rc = lib.trifast_db_finalize(C.byref(shp), C.c_void_p(db_f32.data_ptr()),
                                         C.byref(_lib.t4(db)), _stream(db_f32))
        _lib.check(rc, "trifast_db_finalize")
        return db


class _RowSharded(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, b, mask, group, kernels):
        o, lse = kernels.forward(q, k, v, b, mask)
        ctx.save_for_backward(q, k, v, b, mask, o, lse)
        ctx.group, ctx.kernels = group, kernels
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, b, mask, o, lse = ctx.saved_tensors
        kern, group = ctx.kernels, ctx.group
        db_f32, ws = kern.backward_db(do, q, k, v, b, mask, o, lse)
        work = None
        if dist.is_initialized() and dist.get_world_size(group) > 1:
            # Enqueued behind the db kernels; runs beside the dq/dk/dv kernels below.
            work = dist.all_reduce(db_f32, op=dist.ReduceOp.SUM, group=group, async_op=True)
        dq, dk, dv = kern.backward_dqkv(do, q, k, v, b, mask, lse, ws)
        if work is not None:
            work.wait()
        db = kern.db_finalize(db_f32, b.dtype)
        return dq, dk, dv, db, None, None, None


def triangle_attention_row_sharded(q, k, v, b, mask, group=None, kernels=None):
    """Triangle attention on this rank's block of pair rows.

    q, k, v: (batch, heads, local_rows, n, d); b: (batch, heads, n, n), the same on
    every rank; mask: (batch, local_rows, n).  Returns o for the local rows.  In
    the backward, b.grad is the bias gradient summed over all ranks' rows.
    """
    if kernels is None:
        kernels = CudaKernels(share_gpu=dist.is_initialized() and dist.get_world_size(group) > 1)
    return _RowSharded.apply(q, k, v, b, mask, group, kernels)
