"""Head dim 128: the forward runs on its own tensor-core kernel (csrc/tc_fwd_d128.cu: two
128-query tiles of one pair row per CTA, P written over S in TMEM), the backward on the CUDA
cores.  Forward against the fp64 oracle and against the CUDA-core forward; the whole op with
autograd against the oracle."""

import pytest
import torch

from oracle import triangle_oracle as orc
from tests.helpers import DTYPE_EPS, abi_forward, assert_direction, assert_within_pt_error, max_abs
from trifast_b200 import _lib, triangle_attention

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True)
def device_status_is_clean():
    yield
    import ctypes
    rc = _lib.load().trifast_check_device_status(
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, _lib.status_str(rc)


def _inputs(n, h, rows, dtype, mask, seed=0, std=1.0):
    g = torch.Generator().manual_seed(seed)
    d = 128
    q, k, v = ((torch.randn(1, h, rows, n, d, generator=g) * std * d ** -0.25).to(dtype) for _ in range(3))
    b = (torch.randn(1, h, n, n, generator=g) * std).to(dtype)
    keys = torch.arange(n)
    if mask == "none":
        m = torch.zeros(1, rows, n, dtype=torch.bool)
    elif mask == "random":
        m = torch.rand(1, rows, n, generator=g) < 0.4
        m[0, min(2, rows - 1)] = True                       # a fully masked row
    elif mask == "padding":
        nv = int(0.8 * n)
        m = ((torch.arange(rows)[:, None] >= max(1, rows - 2)) | (keys[None, :] >= nv))[None]
    else:                                                   # dropped head / tail tiles, row by row
        m = torch.zeros(1, rows, n, dtype=torch.bool)
        for i in range(rows):
            if i % 3 == 0:
                m[0, i] = keys < min(n - 1, 128 + 5 * i)
            elif i % 3 == 1:
                m[0, i] = keys >= max(1, n - 130 - i)
    return q, k, v, b, m.contiguous()


def _forward(args, kernel):
    q, k, v, b, m = (t.to(DEV) for t in args)
    o = torch.full_like(q, float("nan"))
    lse = torch.full(q.shape[:4], float("nan"), dtype=torch.float32, device=DEV)
    abi_forward(q, k, v, b, m, o, lse, kernel=kernel)
    torch.cuda.synchronize()
    return o.float().cpu(), lse.cpu()


SHAPES = [  # (n, h, rows, dtype, mask)
    (128, 1, None, torch.bfloat16, "none"),        # one tile: slot 1 has no tile of its own
    (256, 2, None, torch.float16, "random"),       # one pair of tiles
    (333, 2, 40, torch.bfloat16, "random"),        # ragged n, odd number of tiles (3)
    (96, 2, None, torch.bfloat16, "padding"),      # a partly filled tile
    (640, 1, 24, torch.bfloat16, "ranges"),        # live key-tile ranges differ row by row
    (1024, 2, 20, torch.float16, "padding"),       # the long row: 4 tile pairs x 8 key tiles
    (1000, 1, 300, torch.bfloat16, "none"),        # more items than CTAs: several items per CTA
]


@pytest.mark.parametrize("n,h,rows,dtype,mask", SHAPES)
def test_forward_on_tensor_cores(n, h, rows, dtype, mask):
    rows = rows or n
    args = _inputs(n, h, rows, dtype, mask)
    plan = _lib.pick_plan(1, h, n, rows, 128, dtype)
    assert plan["fwd_kernel"] == _lib.KERNEL_TCGEN05 and plan["kernel"] == _lib.KERNEL_SIMT
    o, lse = _forward(args, None)
    o_simt, lse_simt = _forward(args, _lib.KERNEL_SIMT)
    q, k, v, b, m = args
    f = [t.float() for t in (q, k, v, b)]
    ref, lref, _ = orc.forward_backward_chunked(f[0], f[1], f[2], f[3], m, rows_per_chunk=8,
                                                acc_dtype=torch.float64)
    pt = orc.attention_reference_port(q, k, v, b, m).float()
    assert torch.isfinite(o).all() and torch.isfinite(lse).all()
    assert_within_pt_error(o, pt, ref, DTYPE_EPS[dtype], f"d=128 n={n} o")
    assert_direction(o, pt, ref, f"d=128 n={n} o")
    assert max_abs(o, o_simt) <= 3 * (max_abs(o_simt, ref) + DTYPE_EPS[dtype])
    full = m.all(dim=-1)[:, None, :, None].expand_as(lse)      # fully masked rows carry the sentinel
    assert torch.equal(lse[full], lse_simt[full])
    assert float((lse[~full] - lref.float()[~full]).abs().max()) <= 2e-3 * max(1.0, float(lref.abs().max()))


def test_forward_is_deterministic_and_ignores_masked_values():
    args = list(_inputs(300, 2, 30, torch.bfloat16, "random", seed=5))
    o1, l1 = _forward(args, None)
    o2, l2 = _forward(args, None)
    assert torch.equal(o1, o2) and torch.equal(l1, l2)
    q, k, v, b, m = args
    partial = ~m.all(dim=-1)
    sel = (m & partial[..., None])[:, None, :, :, None].expand_as(k)
    k2, v2 = k.clone(), v.clone()
    k2[sel] = 7.0
    v2[sel] = -9.0
    o3, _ = _forward([q, k2, v2, b, m], None)
    assert torch.equal(o1, o3)


def test_whole_op_with_autograd():
    """Forward on tensor cores, backward on CUDA cores, through the public op."""
    n, h, dtype = 160, 2, torch.bfloat16
    q, k, v, b, m = _inputs(n, h, n, dtype, "random", seed=9)
    do = torch.randn(1, h, n, n, 128, generator=torch.Generator().manual_seed(1)).to(dtype)
    qq, kk, vv, bb = (t.detach().to(DEV).requires_grad_(True) for t in (q, k, v, b))
    o = triangle_attention(qq, kk, vv, bb, m.to(DEV))
    o.backward(do.to(DEV))
    torch.cuda.synchronize()
    got = tuple(t.detach().float().cpu() for t in (o, qq.grad, kk.grad, vv.grad, bb.grad))
    ref_o, _ = orc.forward(q, k, v, b, m, torch.float64)
    ref = (ref_o,) + orc.backward(do, q, k, v, b, m, torch.float64)
    q2, k2, v2, b2 = (t.detach().clone().requires_grad_(True) for t in (q, k, v, b))
    o2 = orc.attention_reference_port(q2, k2, v2, b2, m)
    o2.backward(do)
    pt = tuple(t.detach().float() for t in (o2, q2.grad, k2.grad, v2.grad, b2.grad))
    for nm, x, r_, p in zip(("o", "dq", "dk", "dv", "db"), got, ref, pt):
        assert_within_pt_error(x, p, r_, DTYPE_EPS[dtype], f"d=128 op {nm}")


def test_tensor_core_family_cannot_be_forced_onto_the_backward():
    import ctypes as C
    shp = _lib.make_shape(1, 2, 256, 256, 128, torch.bfloat16, _lib.KERNEL_TCGEN05)
    plan = _lib.Plan()
    assert _lib.load().trifast_pick_plan(C.byref(shp), C.byref(plan)) == 0
    assert plan.fwd_kernel == _lib.KERNEL_TCGEN05 and plan.kernel == _lib.KERNEL_SIMT
