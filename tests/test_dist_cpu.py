"""World-size-2 (and 3) ``gloo`` runs of the row-sharded wrapper on CPU tensors.
The compute steps are provided by the oracle here; what is under test is the
host logic: sharding, the db all-reduce, and that every rank ends with the same
full bias gradient."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import triangle_oracle as orc
from trifast_b200.dist import shard_rows, triangle_attention_row_sharded


class OracleKernels:
    def forward(self, q, k, v, b, mask):
        o, lse = orc.forward(q, k, v, b, mask, torch.float64)
        return o.to(q.dtype), lse.float()

    def backward_db(self, do, q, k, v, b, mask, o, lse):
        g = orc.backward(do, q, k, v, b, mask, torch.float64)
        return g[3].float().contiguous(), g

    def backward_dqkv(self, do, q, k, v, b, mask, lse, ws):
        return tuple(t.to(q.dtype) for t in ws[:3])

    def db_finalize(self, db_f32, dtype):
        return db_f32.to(dtype)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n, fail_rank, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        h, d = 2, 16
        q, k, v = (torch.randn(1, h, n, n, d) for _ in range(3))
        b = torch.randn(1, h, n, n)
        mask = torch.rand(1, n, n) < 0.3
        do = torch.randn(1, h, n, n, d)
        rows = shard_rows(n, rank, world)
        ql, kl, vl = (t[:, :, rows].clone().requires_grad_(True) for t in (q, k, v))
        bl = b.clone().requires_grad_(True)
        if rank == fail_rank:
            raise RuntimeError("injected host failure before the step")
        o = triangle_attention_row_sharded(ql, kl, vl, bl, mask[:, rows], kernels=OracleKernels())
        o.backward(do[:, :, rows])
        ref_o, _ = orc.forward(q, k, v, b, mask, torch.float64)
        ref = orc.backward(do, q, k, v, b, mask, torch.float64)
        errs = [float((o.double() - ref_o[:, :, rows]).abs().max()),
                float((ql.grad.double() - ref[0][:, :, rows]).abs().max()),
                float((kl.grad.double() - ref[1][:, :, rows]).abs().max()),
                float((vl.grad.double() - ref[2][:, :, rows]).abs().max()),
                float((bl.grad.double() - ref[3]).abs().max())]
        out.put((rank, errs))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n", [(2, 24), (3, 23)])
def test_row_sharded_matches_whole_problem(world, n):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n, -1, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = [out.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for rank, errs in results:
        assert max(errs) < 1e-5, (rank, errs)


def test_shard_rows_partition():
    for n in (1, 7, 128, 1023, 1024):
        for world in (1, 2, 3, 8):
            cover = []
            for r in range(world):
                s = shard_rows(n, r, world)
                cover += list(range(s.start, s.stop))
            assert cover == list(range(n))
            sizes = [shard_rows(n, r, world).stop - shard_rows(n, r, world).start
                     for r in range(world)]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_rows(8, 2, 2)


def test_rank_failure_surfaces_on_host():
    """A rank that raises before the step makes its process exit non-zero; the
    surviving rank's all-reduce ends with an error instead of hanging (gloo
    notices the closed connection)."""
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, 16, 1, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    assert all(p.exitcode is not None for p in procs), "a rank hung"
    assert procs[1].exitcode != 0
    assert procs[0].exitcode != 0     # its collective failed rather than completing
