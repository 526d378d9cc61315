"""Forward + backward for pair tensors that live in pinned host memory.

Pair rows are independent in o, dq, dk and dv, and db is a sum over rows, so a
step over host-resident q, k, v, dO can run as a pipeline over blocks of rows:
block c + 1 is copied to the GPU and block c - 1 is copied back while block c
is computed.  Host-to-device copies, kernels and device-to-host copies run on
three streams; PCIe carries both directions at once, so a step takes about as
long as the larger of the two transfers instead of their sum plus the compute.
The device holds ``slots`` blocks at a time, so n is not limited by HBM either.

The reference (latkins/trifast, src/trifast/torch.py:220-228) takes device
tensors only; this layer has no counterpart there.  All compute goes through
the same C-ABI entry points as ``trifast_b200.triangle_attention``.
"""

from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
import torch.distributed as dist

from . import _lib

_NAMES_IN = ("q", "k", "v", "do")
_NAMES_OUT = ("o", "dq", "dk", "dv")


def _check_host5(name, t, shape, dtype):
    if t.is_cuda or not t.is_pinned():
        raise ValueError(f"{name} must be a pinned host tensor (torch.Tensor.pin_memory)")
    if tuple(t.shape) != shape or t.dtype != dtype:
        raise ValueError(f"{name} must be {shape} {dtype}; got {tuple(t.shape)} {t.dtype}")
    _, _, rows, n, d = shape
    if t.stride(4) != 1 or t.stride(3) != d or (rows > 1 and t.stride(2) != n * d):
        raise ValueError(f"{name}: the (rows, n, d) block of every (batch, head) must be contiguous")


def block_bounds(rows: int, chunk: int) -> list:
    """Row boundaries of the blocks a step is streamed in: blocks of ``chunk`` rows, but the
    first and the last two are a quarter and a half of that.  The first block's copy in and
    the last block's copy out have nothing to overlap with, so they are kept short; the blocks
    in between keep the transfers long enough for the full PCIe rate."""
    if rows <= 2 * chunk or chunk < 8:
        edges = list(range(0, rows, chunk)) + [rows]
        return edges
    q, h = chunk // 4, chunk // 2
    head = [0, q, q + h]
    tail_start = rows - (q + h)
    edges = head[:]
    r = head[-1]
    while r + chunk <= tail_start:
        r += chunk
        edges.append(r)
    if r < tail_start:                       # what does not fill a whole block
        edges.append(tail_start)
    edges += [rows - q, rows]
    return edges


class HostPipeline:
    """Preallocated device buffers and streams for one problem shape.

    ``rows`` is the number of pair rows this process works on (all n of them on
    one GPU, its shard under ``group``); ``chunk_rows`` of them travel and are
    computed at a time.
    """

    def __init__(self, batch: int, heads: int, n: int, d: int, dtype: torch.dtype,
                 device: torch.device, rows: Optional[int] = None, chunk_rows: int = 64,
                 slots: int = 3, backward: bool = True, ramp: bool = True):
        if slots < 2:
            raise ValueError("at least two slots are needed to overlap copies with compute")
        self.lib = _lib.load()
        self.batch, self.heads, self.n, self.d, self.dtype = batch, heads, n, d, dtype
        self.rows = n if rows is None else rows
        self.chunk = max(1, min(chunk_rows, self.rows))
        self.slots, self.backward = slots, backward
        self.ramp = ramp          # short first and last blocks (see block_bounds)
        self.device = torch.device(device)
        es = torch.empty((), dtype=dtype).element_size()
        blk = batch * heads * self.chunk * n * d
        dev = self.device
        names = _NAMES_IN + _NAMES_OUT if backward else ("q", "k", "v", "o")
        self._flat = {nm: [torch.empty(blk, dtype=dtype, device=dev) for _ in range(slots)]
                      for nm in names}
        self._mask = [torch.empty(batch * self.chunk * n, dtype=torch.uint8, device=dev)
                      for _ in range(slots)]
        self._lse = [torch.empty(batch * heads * self.chunk * n, dtype=torch.float32, device=dev)
                     for _ in range(slots)]
        self.bias = torch.empty((batch, heads, n, n), dtype=dtype, device=dev)
        full = _lib.make_shape(batch, heads, n, self.chunk, d, dtype)
        self._fws_bytes = self.lib.trifast_forward_workspace_bytes(C.byref(full))
        self._fws = torch.empty(max(self._fws_bytes, 1), dtype=torch.uint8, device=dev)
        if backward:
            self._ws_bytes = self.lib.trifast_backward_workspace_bytes(C.byref(full))
            self._ws = torch.empty(self._ws_bytes, dtype=torch.uint8, device=dev)
            self.db_part = torch.empty((batch, heads, n, n), dtype=torch.float32, device=dev)
            self.db_f32 = torch.empty((batch, heads, n, n), dtype=torch.float32, device=dev)
            self.db = torch.empty((batch, heads, n, n), dtype=dtype, device=dev)
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(device=dev) for _ in range(3))
        self.bytes_per_elem = es
        self.kernel_launches = 0      # of the last run()

    # -- views of the slot buffers for a block of r rows (always dense)
    def _v5(self, name, slot, r):
        return self._flat[name][slot][: self.batch * self.heads * r * self.n * self.d].view(
            self.batch, self.heads, r, self.n, self.d)

    def _vmask(self, slot, r):
        return self._mask[slot][: self.batch * r * self.n].view(self.batch, r, self.n)

    def _vlse(self, slot, r):
        return self._lse[slot][: self.batch * self.heads * r * self.n]

    def _copy_rows(self, dst5, src5, r0, r1, to_host, stream):
        """Rows r0:r1 of every (batch, head) between a host tensor and a slot buffer: one 2-D
        transfer per batch entry (a block per head; all of them in one when the batch entries
        are evenly spaced too), enqueued on ``stream``."""
        host, devt = (dst5, src5) if to_host else (src5, dst5)
        es = host.element_size()
        block = (r1 - r0) * self.n * self.d * es
        even = self.batch == 1 or host.stride(0) == self.heads * host.stride(1)
        groups = [(0, self.batch * self.heads)] if even else \
            [(b, self.heads) for b in range(self.batch)]
        for first, count in groups:
            b0 = first if not even else 0
            hp = host[b0, 0, r0].data_ptr()
            dp = devt[b0, 0].data_ptr()
            rc = self.lib.trifast_copy_blocks(
                C.c_void_p(hp if to_host else dp), C.c_size_t(host.stride(1) * es if to_host else block),
                C.c_void_p(dp if to_host else hp), C.c_size_t(block if to_host else host.stride(1) * es),
                C.c_size_t(block), C.c_size_t(count), C.c_int(1 if to_host else 0),
                C.c_void_p(stream.cuda_stream))
            _lib.check(rc, "trifast_copy_blocks")

    def run(self, q, k, v, bias, mask, do=None, out=None, group=None):
        """q, k, v (and do): pinned (batch, heads, rows, n, d); bias: pinned
        (batch, heads, n, n); mask: pinned bool (batch, rows, n).  ``out`` is a dict
        of pinned result tensors ``o`` (and ``dq, dk, dv, db``), allocated when
        absent.  Everything is enqueued; the calling stream waits for the last
        copy, so ``torch.cuda.current_stream().synchronize()`` (or an event on it)
        marks the results complete.  Under ``group`` the db of all ranks' rows is
        summed before it is copied back.
        """
        B, H, R, n, d = self.batch, self.heads, self.rows, self.n, self.d
        bwd = self.backward
        if bwd and do is None:
            raise ValueError("this pipeline was built with backward=True: pass do")
        shape5 = (B, H, R, n, d)
        for nm, t in (("q", q), ("k", k), ("v", v)) + ((("do", do),) if bwd else ()):
            _check_host5(nm, t, shape5, self.dtype)
        if tuple(bias.shape) != (B, H, n, n) or bias.dtype != self.dtype or not bias.is_pinned() \
                or not bias.is_contiguous():
            raise ValueError("bias must be a pinned, contiguous (batch, heads, n, n) host tensor")
        if tuple(mask.shape) != (B, R, n) or mask.dtype != torch.bool or not mask.is_pinned() \
                or not mask.is_contiguous():
            raise ValueError("mask must be a pinned, contiguous bool (batch, rows, n) host tensor")
        m8 = mask.view(torch.uint8)
        if out is None:
            out = {}
        for nm in (_NAMES_OUT if bwd else ("o",)):
            if nm not in out:
                out[nm] = torch.empty(shape5, dtype=self.dtype).pin_memory()
            _check_host5(nm, out[nm], shape5, self.dtype)
        if bwd and "db" not in out:
            out["db"] = torch.empty((B, H, n, n), dtype=self.dtype).pin_memory()
        src = dict(q=q, k=k, v=v, do=do)

        lib, L = self.lib, _lib
        L.raise_if_device_gave_up(self.device)
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_stream(cur)
        run_stream = C.c_void_p(self.s_run.cuda_stream)
        bounds = block_bounds(R, self.chunk) if self.ramp else list(range(0, R, self.chunk)) + [R]
        nchunks = len(bounds) - 1
        ev_in = [None] * nchunks
        ev_run = [None] * nchunks
        ev_out = [None] * nchunks
        launches = 0

        with torch.cuda.device(self.device):
            with torch.cuda.stream(self.s_in):
                self.bias.copy_(bias, non_blocking=True)
            ab = L.t4(self.bias)
            for c in range(nchunks):
                slot = c % self.slots
                r0, r1 = bounds[c], bounds[c + 1]
                r = r1 - r0
                # ---- host -> device
                with torch.cuda.stream(self.s_in):
                    if c >= self.slots:
                        self.s_in.wait_event(ev_run[c - self.slots])   # inputs of the slot consumed
                    for nm in (_NAMES_IN if bwd else ("q", "k", "v")):
                        self._copy_rows(self._v5(nm, slot, r), src[nm], r0, r1, False, self.s_in)
                    for b in range(B):
                        self._vmask(slot, r)[b].copy_(m8[b, r0:r1], non_blocking=True)
                    ev_in[c] = self.s_in.record_event()
                # ---- kernels
                with torch.cuda.stream(self.s_run):
                    self.s_run.wait_event(ev_in[c])
                    if c >= self.slots:
                        self.s_run.wait_event(ev_out[c - self.slots])  # results of the slot copied out
                    shp = L.make_shape(B, H, n, r, d, self.dtype)
                    a = {nm: L.t5(self._v5(nm, slot, r)) for nm in self._flat}
                    am = L.mask_view(self._vmask(slot, r))
                    lse = C.c_void_p(self._vlse(slot, r).data_ptr())
                    rc = lib.trifast_forward(C.byref(shp), C.byref(a["q"]), C.byref(a["k"]),
                                             C.byref(a["v"]), C.byref(ab), C.byref(am),
                                             C.byref(a["o"]), lse,
                                             C.c_void_p(self._fws.data_ptr()),
                                             C.c_size_t(self._fws_bytes), run_stream)
                    L.check(rc, "trifast_forward")
                    plan = L.pick_plan(B, H, n, r, d, self.dtype)
                    tc = plan["kernel"] == L.KERNEL_TCGEN05
                    launches += 1 + (2 if self._fws_bytes else 0)
                    if bwd:
                        part = self.db_f32 if c == 0 else self.db_part
                        ws, wsb = C.c_void_p(self._ws.data_ptr()), C.c_size_t(self._ws_bytes)
                        rc = lib.trifast_backward_db(
                            C.byref(shp), C.byref(a["do"]), C.byref(a["q"]), C.byref(a["k"]),
                            C.byref(a["v"]), C.byref(ab), C.byref(am), C.byref(a["o"]), lse,
                            C.c_void_p(part.data_ptr()), ws, wsb, run_stream)
                        L.check(rc, "trifast_backward_db")
                        if c > 0:
                            self.db_f32.add_(self.db_part)
                        rc = lib.trifast_backward_dqkv(
                            C.byref(shp), C.byref(a["do"]), C.byref(a["q"]), C.byref(a["k"]),
                            C.byref(a["v"]), C.byref(ab), C.byref(am), lse, C.byref(a["dq"]),
                            C.byref(a["dk"]), C.byref(a["dv"]), ws, wsb, run_stream)
                        L.check(rc, "trifast_backward_dqkv")
                        # row flags, bias copies, delta, db (+ split reduce), dq, dk/dv
                        launches += 1 + (1 if tc else 0) + (1 if tc and n % 8 else 0) + 2 + \
                            (1 if plan["db_row_splits"] > 1 else 0) + 2
                    ev_run[c] = self.s_run.record_event()
                # ---- device -> host
                with torch.cuda.stream(self.s_out):
                    self.s_out.wait_event(ev_run[c])
                    for nm in (_NAMES_OUT if bwd else ("o",)):
                        self._copy_rows(out[nm], self._v5(nm, slot, r), r0, r1, True, self.s_out)
                    ev_out[c] = self.s_out.record_event()
            if bwd:
                with torch.cuda.stream(self.s_run):
                    if group is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
                        dist.all_reduce(self.db_f32, op=dist.ReduceOp.SUM, group=group)
                    shp = L.make_shape(B, H, n, n, d, self.dtype)
                    rc = lib.trifast_db_finalize(C.byref(shp), C.c_void_p(self.db_f32.data_ptr()),
                                                 C.byref(L.t4(self.db)), run_stream)
                    L.check(rc, "trifast_db_finalize")
                    launches += 1
                    ev_db = self.s_run.record_event()
                with torch.cuda.stream(self.s_out):
                    self.s_out.wait_event(ev_db)
                    out["db"].copy_(self.db, non_blocking=True)
        cur.wait_stream(self.s_out)
        cur.wait_stream(self.s_run)
        cur.wait_stream(self.s_in)
        L.snapshot_status(self.device, C.c_void_p(cur.cuda_stream))
        self.kernel_launches = launches
        return out


def triangle_attention_host(q, k, v, bias, mask, do=None, device=None, chunk_rows: int = 64,
                            out=None):
    """One-shot form of :class:`HostPipeline` on a single GPU: pinned host tensors
    in, pinned host tensors out (``{"o": ...}`` or, with ``do``, also ``dq, dk, dv,
    db``).  Blocks until the results are in host memory."""
    B, H, R, n, d = q.shape
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    pipe = HostPipeline(B, H, n, d, q.dtype, device, rows=R, chunk_rows=chunk_rows,
                        backward=do is not None)
    res = pipe.run(q, k, v, bias, mask, do=do, out=out)
    torch.cuda.current_stream(device).synchronize()
    return res
