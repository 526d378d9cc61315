"""Two-GPU check of the row-sharded path over NCCL: each rank runs its block of
pair rows through the CUDA kernels, db is all-reduced inside the backward, and
the result must equal the single-GPU run of the whole problem.  Skipped when
fewer than two GPUs are visible."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n, dtype, out, db_reduce="nccl"):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    try:
        from trifast_b200 import triangle_attention
        from trifast_b200.dist import shard_rows, triangle_attention_row_sharded
        g = torch.Generator().manual_seed(0)
        h, d = 2, 32
        mk = lambda *s: (torch.randn(*s, generator=g) * 0.5).to(dtype)
        q, k, v, do = (mk(1, h, n, n, d) for _ in range(4))
        b = mk(1, h, n, n)
        m = torch.rand(1, n, n, generator=g) < 0.3
        dev = torch.device("cuda", rank)
        rows = shard_rows(n, rank, world)
        ql, kl, vl = (t[:, :, rows].contiguous().to(dev).requires_grad_(True) for t in (q, k, v))
        bl = b.to(dev).requires_grad_(True)
        o = triangle_attention_row_sharded(ql, kl, vl, bl, m[:, rows].to(dev), db_reduce=db_reduce)
        o.backward(do[:, :, rows].to(dev))
        torch.cuda.synchronize()
        if db_reduce == "push":
            # a second and third step through the same symmetric buffers (epochs 2, 3), and
            # the NCCL path on the same inputs: two ranks add two numbers, so the sums agree
            # bit for bit
            first = bl.grad.clone()
            for _ in range(2):
                ql.grad = kl.grad = vl.grad = bl.grad = None
                o2 = triangle_attention_row_sharded(ql, kl, vl, bl, m[:, rows].to(dev), db_reduce="push")
                o2.backward(do[:, :, rows].to(dev))
                torch.cuda.synchronize()
                assert torch.equal(bl.grad, first), "push reduce is not reproducible across calls"
            ql.grad = kl.grad = vl.grad = bl.grad = None
            o3 = triangle_attention_row_sharded(ql, kl, vl, bl, m[:, rows].to(dev), db_reduce="nccl")
            o3.backward(do[:, :, rows].to(dev))
            torch.cuda.synchronize()
            assert torch.equal(bl.grad, first), "push reduce and NCCL all-reduce disagree"
            from trifast_b200 import _lib
            import ctypes
            assert _lib.load().trifast_check_device_status(
                ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)) == 0
        # whole problem on this rank's GPU
        qw, kw, vw, bw = (t.to(dev).requires_grad_(True) for t in (q, k, v, b))
        ow = triangle_attention(qw, kw, vw, bw, m.to(dev))
        ow.backward(do.to(dev))
        torch.cuda.synchronize()
        same = [torch.equal(o, ow[:, :, rows]), torch.equal(ql.grad, qw.grad[:, :, rows]),
                torch.equal(kl.grad, kw.grad[:, :, rows]), torch.equal(vl.grad, vw.grad[:, :, rows])]
        db_err = float((bl.grad.float() - bw.grad.float()).abs().max() /
                       bw.grad.float().abs().max())
        # the same shard through the host-resident pipeline (pinned host tensors, db summed
        # over the ranks inside run())
        from trifast_b200.host import HostPipeline
        pin = lambda t: t.contiguous().pin_memory()
        pipe = HostPipeline(1, h, n, d, dtype, dev, rows=rows.stop - rows.start, chunk_rows=24)
        res = pipe.run(pin(q[:, :, rows]), pin(k[:, :, rows]), pin(v[:, :, rows]), pin(b),
                       pin(m[:, rows]), do=pin(do[:, :, rows]), group=dist.group.WORLD)
        torch.cuda.synchronize()
        same.append(torch.equal(res["o"], ow[:, :, rows].cpu()))
        same.append(torch.equal(res["dk"], kw.grad[:, :, rows].cpu()))
        host_db_err = float((res["db"].float() - bw.grad.float().cpu()).abs().max() /
                            bw.grad.float().abs().max())
        out.put((rank, same, max(db_err, host_db_err)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n,dtype,db_reduce", [(136, torch.bfloat16, "nccl"), (72, torch.float32, "nccl"),
                                               (200, torch.bfloat16, "push"), (75, torch.float32, "push")])
def test_two_gpu_row_shards_match_single_gpu(n, dtype, db_reduce):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, n, dtype, out, db_reduce)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=300) for _ in range(2)]
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    tol = 1e-5 if dtype == torch.float32 else 2e-2   # db: fp32 partial sums, one rounding
    for rank, same, db_err in results:
        assert all(same), (rank, same)        # rows are independent: bit-identical
        assert db_err < tol, (rank, db_err)
