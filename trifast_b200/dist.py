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

    def __init__(self, share_gpu: bool = False, free_sms: int = 0):
        # under a process group the all-reduce of db runs beside the dq/dk/dv kernels:
        # they then leave a few SMs free for it (TRIFAST_FLAG_SHARE_GPU; free_sms = 0: the
        # library's 8, which suits a collective of up to 8 CTAs)
        self.flags = _lib.flags_choice() | (_lib.share_gpu_flags(free_sms) if share_gpu else 0)

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


class PushReducer:
    """The db exchange without a collective library: every rank pushes slices of its fp32
    partial into the other ranks' memory with plain stores and adds what it received in rank
    order (``trifast_db_push_reduce`` of the C ABI, csrc/db_push_reduce.cu).

    Holds, per process group and db size, one symmetric allocation (staging area, result
    buffer, flag words; mapped into every rank of the box through
    ``torch.distributed._symmetric_memory``), a side stream and the call counter that all
    ranks advance together.  ``reduce(partial)`` enqueues the exchange on the side stream
    behind the work already enqueued on the current stream and returns the local result
    tensor; ``join()`` makes the current stream wait for it.
    """

    _FLAG_FLOATS = 64          # 16 flag words per rank, padded

    def __init__(self, count: int, device: torch.device, group=None, ctas: int = 4):
        import torch.distributed._symmetric_memory as symm
        self.ctas = ctas      # CTAs of the exchange kernel: each wants a free SM, all at once
        self.lib = _lib.load()
        self.group = dist.group.WORLD if group is None else group
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world > 8:
            raise ValueError("the push reduce serves the GPUs of one box (world <= 8)")
        self.count, self.device = count, torch.device(device)
        self.staging_floats = int(self.lib.trifast_db_push_reduce_staging_floats(count, self.world))
        result_floats = (count + 3) // 4 * 4
        total = self.staging_floats + result_floats + self._FLAG_FLOATS
        self.buf = symm.empty(total, dtype=torch.float32, device=self.device)
        self.buf.zero_()
        torch.cuda.synchronize(self.device)
        self.handle = symm.rendezvous(self.buf, self.group)
        dist.barrier(self.group)                     # every rank's flags are zero before any push
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self._staging = [p for p in ptrs]
        self._result = [p + 4 * self.staging_floats for p in ptrs]
        self._flags = [p + 4 * (self.staging_floats + result_floats) for p in ptrs]
        self.result = self.buf[self.staging_floats:self.staging_floats + count]
        self.counters = torch.zeros(2, dtype=torch.int32, device=self.device)
        self.stream = torch.cuda.Stream(device=self.device)
        self.epoch = 0

    def reduce(self, partial: torch.Tensor) -> torch.Tensor:
        assert partial.dtype == torch.float32 and partial.is_contiguous() and partial.numel() == self.count
        self.epoch += 1
        a = _lib.PushReduce()
        a.rank, a.world, a.ctas, a.epoch, a.count = self.rank, self.world, self.ctas, self.epoch, self.count
        a.partial, a.counters = partial.data_ptr(), self.counters.data_ptr()
        for r in range(self.world):
            a.staging[r], a.result[r], a.flags[r] = self._staging[r], self._result[r], self._flags[r]
        self.stream.wait_stream(torch.cuda.current_stream(self.device))
        partial.record_stream(self.stream)
        with torch.cuda.device(self.device):
            rc = self.lib.trifast_db_push_reduce(C.byref(a), C.c_void_p(self.stream.cuda_stream))
        _lib.check(rc, "trifast_db_push_reduce")
        return self.result

    def join(self) -> None:
        torch.cuda.current_stream(self.device).wait_stream(self.stream)


_push_reducers: dict = {}


def _push_reducer(count, device, group) -> PushReducer:
    key = (count, torch.device(device).index, id(group))
    if key not in _push_reducers:
        _push_reducers[key] = PushReducer(count, device, group)
    return _push_reducers[key]


class _RowSharded(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, b, mask, group, kernels, db_reduce="nccl"):
        o, lse = kernels.forward(q, k, v, b, mask)
        ctx.save_for_backward(q, k, v, b, mask, o, lse)
        ctx.group, ctx.kernels, ctx.db_reduce = group, kernels, db_reduce
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, b, mask, o, lse = ctx.saved_tensors
        kern, group = ctx.kernels, ctx.group
        db_f32, ws = kern.backward_db(do, q, k, v, b, mask, o, lse)
        work = reducer = None
        if dist.is_initialized() and dist.get_world_size(group) > 1:
            # Enqueued behind the db kernels; runs beside the dq/dk/dv kernels below.
            if ctx.db_reduce == "push":
                reducer = _push_reducer(db_f32.numel(), db_f32.device, group)
                db_f32 = reducer.reduce(db_f32).view(db_f32.shape)
            else:
                work = dist.all_reduce(db_f32, op=dist.ReduceOp.SUM, group=group, async_op=True)
        dq, dk, dv = kern.backward_dqkv(do, q, k, v, b, mask, lse, ws)
        if work is not None:
            work.wait()
        if reducer is not None:
            reducer.join()
        db = kern.db_finalize(db_f32, b.dtype)
        return dq, dk, dv, db, None, None, None, None


def triangle_attention_row_sharded(q, k, v, b, mask, group=None, kernels=None, db_reduce="nccl"):
    """Triangle attention on this rank's block of pair rows.

    q, k, v: (batch, heads, local_rows, n, d); b: (batch, heads, n, n), the same on
    every rank; mask: (batch, local_rows, n).  Returns o for the local rows.  In
    the backward, b.grad is the bias gradient summed over all ranks' rows: by an NCCL
    all-reduce (``db_reduce="nccl"``) or by the library's own peer-store exchange
    (``"push"``: the ranks of one box, summation in rank order).
    """
    if db_reduce not in ("nccl", "push"):
        raise ValueError("db_reduce must be 'nccl' or 'push'")
    if kernels is None:
        kernels = CudaKernels(share_gpu=dist.is_initialized() and dist.get_world_size(group) > 1)
    return _RowSharded.apply(q, k, v, b, mask, group, kernels, db_reduce)
