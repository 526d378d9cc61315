"""Host-resident pipeline (trifast_b200/host.py) against the device-resident operator."""

import pytest
import torch

from trifast_b200 import triangle_attention
from trifast_b200.host import HostPipeline, triangle_attention_host
from trifast_b200.utils import gen_tensors

pytestmark = pytest.mark.gpu


def _inputs(n, h, d, dtype, seed=0, bs=1):
    torch.manual_seed(seed)
    q, k, v, b, m = gen_tensors(n, d, h, True, "cpu", torch.float32, batch=bs)
    m[:, 3] = True                                    # one fully masked row
    do = torch.randn(q.shape)
    host = [t.detach().to(dtype).contiguous().pin_memory() for t in (q, k, v, b)]
    return host + [m.contiguous().pin_memory(), do.to(dtype).contiguous().pin_memory()]


def _device_reference(q, k, v, b, m, do):
    dev = [t.cuda().requires_grad_(True) for t in (q, k, v, b)]
    o = triangle_attention(*dev, m.cuda())
    o.backward(do.cuda())
    return [o.detach().cpu()] + [t.grad.cpu() for t in dev]


@pytest.mark.parametrize("n,h,d,dtype,chunk", [
    (160, 2, 32, torch.bfloat16, 48),      # ragged last block, tensor-core kernels
    (131, 2, 64, torch.float16, 40),       # n % 8 != 0: forward workspace in use
    (72, 2, 32, torch.float32, 16),        # CUDA-core kernels, more blocks than slots
])
def test_pipeline_matches_device_operator(n, h, d, dtype, chunk):
    q, k, v, b, m, do = _inputs(n, h, d, dtype)
    ref = _device_reference(q, k, v, b, m, do)
    out = triangle_attention_host(q, k, v, b, m, do=do, chunk_rows=chunk)
    # rows are independent: o, dq, dk, dv are the same bits whatever the blocking
    for name, r in zip(("o", "dq", "dk", "dv"), ref):
        assert torch.equal(out[name], r), name
    # db sums the blocks' fp32 partials in a different order than one launch does
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    err = (out["db"].double() - ref[4].double()).abs().max() / ref[4].double().abs().max()
    assert float(err) < tol


def test_pipeline_reuse_and_forward_only():
    n, h, d = 136, 2, 32
    q, k, v, b, m, do = _inputs(n, h, d, torch.bfloat16, seed=4)
    ref = _device_reference(q, k, v, b, m, do)
    pipe = HostPipeline(1, h, n, d, torch.bfloat16, torch.device("cuda", 0), chunk_rows=32, slots=2)
    out = None
    for _ in range(2):                               # same buffers, two steps in a row
        out = pipe.run(q, k, v, b, m, do=do, out=out)
        torch.cuda.synchronize()
        assert torch.equal(out["o"], ref[0]) and torch.equal(out["dk"], ref[2])
    assert pipe.kernel_launches > 0
    fwd = triangle_attention_host(q, k, v, b, m, chunk_rows=64)
    assert set(fwd) == {"o"} and torch.equal(fwd["o"], ref[0])


def test_rejects_pageable_and_strided_host_tensors():
    n, h, d = 32, 1, 32
    q, k, v, b, m, do = _inputs(n, h, d, torch.float32)
    with pytest.raises(ValueError, match="pinned"):
        triangle_attention_host(q.clone(), k, v, b, m)
    wide = torch.zeros(1, h, n, n, 2 * d).pin_memory()[..., :d]      # row pitch 2 * d
    with pytest.raises(ValueError, match="contiguous"):
        triangle_attention_host(wide, k, v, b, m)
