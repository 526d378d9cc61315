"""The allocation-free backward entry point, ``trifast_backward_static_scratch``.

Some hosts of this library cannot call cudaMalloc when the backward runs (the
GPU's memory already belongs to their own pool, or their callback is not
allowed to allocate), so they cannot supply the workspace ``trifast_backward``
asks for.  This entry point keeps that workspace in a fixed array inside the
library.  The test calls it through the C ABI with caller-owned inputs and
outputs only, twice in a row with different problems (the array is shared and
keeps the previous call's contents), and requires the same dq, dk, dv, db as
the regular entry point given a caller workspace.

Collected last on purpose: a failure here cannot hide the other tests from a
run that stops at the first failure.
"""

import ctypes as C

import pytest
import torch

from trifast_b200 import _lib


def _problem(n, h, d, dtype, seed, dev):
    g = torch.Generator().manual_seed(seed)
    mk = lambda *s: (torch.randn(*s, generator=g) * 0.5).to(dtype).to(dev)
    q, k, v, do = (mk(1, h, n, n, d) for _ in range(4))
    b = mk(1, h, n, n)
    m = (torch.rand(1, n, n, generator=g) < 0.3).to(dev)
    m[0, 1] = True                                  # one fully masked row
    return q, k, v, b, m, do


def _backward(entry, q, k, v, b, m, do, o, lse, workspace):
    lib = _lib.load()
    bs, h, rows, n, d = q.shape
    shp = _lib.make_shape(bs, h, n, rows, d, q.dtype)
    dq, dk, dv, db = (torch.full_like(t, float("nan")) for t in (q, k, v, b))
    m8 = m.view(torch.uint8)
    args = [C.byref(shp), C.byref(_lib.t5(do)), C.byref(_lib.t5(q)), C.byref(_lib.t5(k)),
            C.byref(_lib.t5(v)), C.byref(_lib.t4(b)), C.byref(_lib.mask_view(m8)),
            C.byref(_lib.t5(o)), C.c_void_p(lse.data_ptr()), C.byref(_lib.t5(dq)),
            C.byref(_lib.t5(dk)), C.byref(_lib.t5(dv)), C.byref(_lib.t4(db))]
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    if workspace:
        nbytes = lib.trifast_backward_workspace_bytes(C.byref(shp))
        ws = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
        rc = lib.trifast_backward(*args, C.c_void_p(ws.data_ptr()), C.c_size_t(nbytes), stream)
    else:
        rc = getattr(lib, entry)(*args, stream)
    _lib.check(rc, entry)
    torch.cuda.synchronize()
    return dq, dk, dv, db


@pytest.mark.gpu
def test_static_scratch_backward_matches_regular_backward_twice():
    from trifast_b200.torch import _triangle_attention
    dev = "cuda"
    lib = _lib.load()
    # two calls in a row, different sizes and dtypes, the larger one first so the
    # second call runs over leftovers of the first
    for n, h, d, dtype, seed in [(160, 2, 32, torch.bfloat16, 1), (72, 3, 16, torch.float32, 2)]:
        q, k, v, b, m, do = _problem(n, h, d, dtype, seed, dev)
        o, lse = _triangle_attention(q, k, v, b, m)
        want = _backward("trifast_backward", q, k, v, b, m, do, o, lse, workspace=True)
        got = _backward("trifast_backward_static_scratch", q, k, v, b, m, do, o, lse,
                        workspace=False)
        for name, a, w in zip(("dq", "dk", "dv", "db"), got, want):
            assert not torch.isnan(a.float()).any(), name
            # same kernels, same order of operations: the tolerance of the fp32
            # contract (1e-4 relative) is met with room to spare
            err = float((a.double() - w.double()).abs().max() / w.double().abs().max())
            assert err <= 1e-4, (n, name, err)


def test_static_scratch_rejects_problems_beyond_its_capacity():
    """Validation happens before any device work, so this needs no GPU."""
    lib = _lib.load()
    shp = _lib.make_shape(1, 4, 1024, 1024, 32, torch.bfloat16)
    assert lib.trifast_backward_workspace_bytes(C.byref(shp)) > _lib.STATIC_SCRATCH_BYTES
    null5, null4 = _lib.T5(), _lib.T4()
    rc = lib.trifast_backward_static_scratch(
        C.byref(shp), C.byref(null5), C.byref(null5), C.byref(null5), C.byref(null5),
        C.byref(null4), C.byref(_lib.Mask()), C.byref(null5), None, C.byref(null5),
        C.byref(null5), C.byref(null5), C.byref(null4), None)
    assert rc == -12
    assert "maximum" in _lib.status_str(rc)
    bad = _lib.Shape(1, 4, 64, 64, 48, 1, 0, 0)
    assert lib.trifast_backward_static_scratch(
        C.byref(bad), C.byref(null5), C.byref(null5), C.byref(null5), C.byref(null5),
        C.byref(null4), C.byref(_lib.Mask()), C.byref(null5), None, C.byref(null5),
        C.byref(null5), C.byref(null5), C.byref(null4), None) == -3
