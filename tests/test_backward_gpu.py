"""GPU tier, backward in depth: the one-pass dq/dk/dv kernel against the two-kernel
path, db determinism, gradients of the large configured workloads on row samples,
strided inputs on the tensor-core path, memory around the outputs, and the
device-timeout path.  Every call goes through the C ABI (directly or through the
public operator)."""

import ctypes as C

import os

import pytest
import torch

from oracle import triangle_oracle as orc
from tests.helpers import (DTYPE_EPS, abi_backward, abi_forward, assert_direction, max_abs,
                           assert_within_pt_error, rel_err)
from trifast_b200 import _lib, triangle_attention
from trifast_b200.configs import WORKLOADS, make_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda"
NAMES = ("o", "dq", "dk", "dv", "db")


@pytest.fixture(autouse=True)
def device_status_is_clean():
    """No kernel may have given up on one of its bounded waits during a test."""
    yield
    rc = _lib.load().trifast_check_device_status(
        C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, _lib.status_str(rc)


def _inputs(n, h, d, dtype, mask, rows=None, seed=0, bias_std=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    rows = rows or n
    q, k, v = ((torch.randn(1, h, rows, n, d, generator=g) * d ** -0.5).to(dtype) for _ in range(3))
    b = (torch.randn(1, h, n, n, generator=g) * bias_std).to(dtype)
    do = torch.randn(1, h, rows, n, d, generator=g).to(dtype)
    if mask == "none":
        m = torch.zeros(1, rows, n, dtype=torch.bool)
    elif mask == "random":
        m = torch.rand(1, rows, n, generator=g) < 0.3
        m[0, min(3, rows - 1)] = True                      # one fully masked row as well
    else:                                                  # padding in rows and keys
        nv = int(0.85 * n)
        m = ((torch.arange(rows)[:, None] >= min(nv, rows - 2)) | (torch.arange(n)[None, :] >= nv))[None]
    return q, k, v, b, m.contiguous(), do


def _run_abi(args, flags=0, kernel=None):
    q, k, v, b, m, do = (t.to(DEV) for t in args)
    o = torch.empty_like(q)
    lse = torch.empty(q.shape[:4], dtype=torch.float32, device=DEV)
    abi_forward(q, k, v, b, m, o, lse, kernel=kernel)
    dq, dk, dv = (torch.full_like(q, float("nan")) for _ in range(3))
    db = torch.full_like(b, float("nan"))
    abi_backward(do, q, k, v, b, m, o, lse, dq, dk, dv, db, kernel=kernel, flags=flags)
    torch.cuda.synchronize()
    return o, dq, dk, dv, db


FUSED_SHAPES = [  # (n, h, d, dtype, mask, rows): every shape the one-pass kernel serves differs
    (128, 1, 32, torch.bfloat16, "none", None),       # a single key tile, two query steps
    (192, 2, 32, torch.float16, "random", None),      # odd number of 64-query steps
    (333, 2, 32, torch.bfloat16, "random", None),     # ragged n (padded bias copy)
    (512, 4, 32, torch.bfloat16, "padding", None),    # fully masked rows, dropped key tiles
    (200, 2, 64, torch.bfloat16, "random", None),     # head dim 64
    (384, 1, 64, torch.float16, "padding", None),     # largest n for head dim 64
    (1000, 2, 32, torch.bfloat16, "random", 40),      # a row shard of a long problem
    (1024, 1, 32, torch.bfloat16, "none", 150),       # all eight dQ tiles, > 1 item per CTA
    (1100, 1, 32, torch.bfloat16, "random", 20),      # two query chunks (8 + 1 tiles): dK / dV partials
    (2048, 1, 32, torch.bfloat16, "padding", 24),     # two full chunks, fully masked rows
    (512, 1, 64, torch.float16, "random", 16),        # head dim 64: chunks of three tiles (3 + 1)
    (1001, 1, 64, torch.bfloat16, "padding", 12),     # three chunks (3 + 3 + 2), ragged n
    (2500, 1, 32, torch.bfloat16, "random", 170),     # three chunks, more items than CTAs
    (141, 2, 32, torch.float16, "random", 1),         # a single pair row of a ragged problem
]


@pytest.mark.parametrize("n,h,d,dtype,mask,rows", FUSED_SHAPES)
def test_one_pass_backward_equals_two_kernel_backward(n, h, d, dtype, mask, rows):
    """dq, dk, dv of the one-pass kernel are bit-identical to those of the dq and dk/dv
    kernels: both round P and dS to 16 bits at the same points and accumulate in the
    same order.  Any difference is an indexing or synchronisation error."""
    args = _inputs(n, h, d, dtype, mask, rows, seed=n)
    plan = _lib.pick_plan(1, h, n, rows or n, d, dtype)
    assert plan["bwd_fused"] == 1, "shape is meant to exercise the one-pass kernel"
    fused = _run_abi(args, flags=0)
    split = _run_abi(args, flags=_lib.FLAG_SPLIT_BWD)
    for name, a, b in zip(NAMES, fused, split):
        assert not torch.isnan(a.float()).any(), f"{name}: output not fully written"
        if plan["bwd_chunks"] > 1 and name in ("dk", "dv"):
            # a row walked in query chunks sums dK / dV per chunk and adds the fp32 partials:
            # another summation order than one accumulation over all queries, so the
            # 16-bit results may differ in the last place of a few elements
            err = float((a.float() - b.float()).abs().max())
            assert err <= 2.0 ** -7 * float(b.float().abs().max()), f"{name}: {err:.3e}"
            assert float((a != b).float().mean()) < 0.02, name
        else:
            assert torch.equal(a, b), f"{name}: one-pass and two-kernel results differ"


def test_one_pass_backward_is_run_to_run_deterministic():
    args = _inputs(640, 2, 32, torch.bfloat16, "random", 70, seed=5)
    a, b = _run_abi(args), _run_abi(args)
    for name, x, y in zip(NAMES, a, b):
        assert torch.equal(x, y), name


@pytest.mark.parametrize("n,h,rows", [(384, 2, None), (256, 4, 100), (1024, 1, 64)])
def test_db_is_bitwise_reproducible_and_matches_the_cuda_core_db(n, h, rows):
    """db is a fixed-order sum (one CTA per tile and row split, splits added in order):
    repeated runs agree bit for bit, over many tiles and splits, and the tensor-core
    result agrees with the CUDA-core kernel's to bf16 rounding of the sum."""
    args = _inputs(n, h, 32, torch.bfloat16, "random", rows, seed=11)
    plan = _lib.pick_plan(1, h, n, rows or n, 32, torch.bfloat16)
    assert plan["db_row_splits"] > 1
    first = _run_abi(args)[4]
    for _ in range(4):
        assert torch.equal(_run_abi(args)[4], first)
    simt = _run_abi(args, kernel=_lib.KERNEL_SIMT)[4]
    assert rel_err(first.float(), simt.float()) < 2e-2


def _sample_rows(w, count=32):
    """Rows for a sampled check: the first ones, the rows around the end of the valid
    range (last valid row, first padded = fully masked rows) and the very last row."""
    n = w.n
    if w.mask.startswith("padding"):
        nv = int(float(w.mask.split(":")[1]) * n)
        rows = list(range(0, count // 2 - 1)) + list(range(nv - count // 4, nv + count // 4)) + [n - 1]
    else:
        rows = list(range(0, count - 8)) + list(range(n - 8, n))
    return torch.tensor(sorted(set(rows)))


@pytest.mark.parametrize("name", ["c4_n1024_h8_d64_fwd", "c5_n2048_pad", "metric_n1024"])
def test_large_workloads_gradients_on_a_row_sample(name):
    """o, dq, dk, dv and the db partial of >= 32 sampled pair rows of the large workloads,
    against the fp64 oracle under the reference's rule: error <= 3 * (error of PyTorch in
    the same dtype + eps), plus its direction rules.  The sample holds padded (fully
    masked) rows and the last valid row where the workload has padding.  Rows are
    independent, so a row subset is a complete problem (db = the subset's partial)."""
    w = WORKLOADS[name]
    q, k, v, b, m, do = make_inputs(w, seed=1337)
    rows = _sample_rows(w)
    assert len(rows) >= 32
    q, k, v, do = (t[:, :, rows].contiguous() for t in (q, k, v, do))
    m = m[:, rows].contiguous()
    got = tuple(t.float().cpu() for t in _run_abi((q, k, v, b, m, do), kernel=_lib.KERNEL_TCGEN05))
    f = [t.float() for t in (q, k, v, b)]
    o, _, grads = orc.forward_backward_chunked(f[0], f[1], f[2], f[3], m, do=do.float(),
                                               rows_per_chunk=4, acc_dtype=torch.float64)
    ref = (o,) + grads
    # PyTorch in the workload's dtype, in row chunks (db adds up over chunks)
    parts = []
    for r in range(0, len(rows), 8):
        s = slice(r, r + 8)
        qq, kk, vv, bb = (t.detach().clone().requires_grad_(True) for t in (q[:, :, s], k[:, :, s], v[:, :, s], b))
        oo = orc.attention_reference_port(qq, kk, vv, bb, m[:, s])
        oo.backward(do[:, :, s])
        parts.append(tuple(t.detach().float() for t in (oo, qq.grad, kk.grad, vv.grad, bb.grad)))
    pt = tuple(torch.cat([p[x] for p in parts], dim=2) for x in range(4)) + (sum(p[4] for p in parts),)
    for nm, g, r, p in zip(NAMES, got, ref, pt):
        assert_within_pt_error(g, p, r, DTYPE_EPS[w.dtype], f"{name} {nm}")
        assert_direction(g, p, r, f"{name} {nm}")


def test_strided_projection_layout_on_the_tensor_core_path():
    """q, k, v as (b, n, n, h, d) projections permuted to (b, h, n, n, d) and a bias whose
    rows have a pitch larger than n: the TMA maps are built from the user strides, nothing
    is copied, and the results equal those of dense copies bit for bit."""
    torch.manual_seed(2)
    n, h, d = 256, 2, 32
    base = [(torch.randn(1, n, n, h, d) * d ** -0.5).to(torch.bfloat16).to(DEV) for _ in range(4)]
    q, k, v, do = (t.permute(0, 3, 1, 2, 4) for t in base)
    assert not q.is_contiguous()
    big = torch.randn(1, h, n, n + 24).to(torch.bfloat16).to(DEV)
    b = big[..., :n]
    m = (torch.rand(1, n, n) < 0.2).to(DEV)
    from trifast_b200.torch import _prep4, _prep5
    assert _prep5(q) is q and _prep4(b) is b, "layout must be consumed as it is"

    def run(q, k, v, b, do):
        q, k, v, b = (t.detach().requires_grad_(True) for t in (q, k, v, b))
        o = triangle_attention(q, k, v, b, m)
        o.backward(do)
        return o, q.grad, k.grad, v.grad, b.grad

    a = run(q, k, v, b, do)
    c = run(q.contiguous(), k.contiguous(), v.contiguous(), b.contiguous(), do.contiguous())
    for name, x, y in zip(NAMES, a, c):
        assert torch.equal(x, y), name
    ref_o, _ = orc.forward(*(t.float().cpu() for t in (q, k, v, b)), m.cpu(), torch.float32)
    assert rel_err(a[0].float().cpu(), ref_o) < 2e-2


@pytest.mark.parametrize("n,h,d,dtype", [(203, 2, 32, torch.bfloat16), (136, 1, 64, torch.float16),
                                          (1001, 1, 32, torch.bfloat16)])
def test_nothing_is_written_outside_the_outputs(n, h, d, dtype):
    """Ragged n on the tensor-core path: o, dq, dk, dv live in buffers whose rows have a
    pitch of d + 8 elements and which are surrounded by guard areas, lse and db sit between
    guards; after forward and backward every guard element and every element of the row
    padding still holds its fill pattern, and every output element has been written."""
    rows = min(n, 48)
    q, k, v, b, m, do = (t.to(DEV) for t in _inputs(n, h, d, dtype, "random", rows, seed=3))
    fill = -7.0
    guard = 4096

    def padded5():
        flat = torch.full((guard + h * rows * n * (d + 8) + guard,), fill, dtype=dtype, device=DEV)
        view = flat[guard:guard + h * rows * n * (d + 8)].view(1, h, rows, n, d + 8)[..., :d]
        return flat, view

    def guarded(shape, dt):
        numel = 1
        for s in shape:
            numel *= s
        flat = torch.full((guard + numel + guard,), fill, dtype=dt, device=DEV)
        return flat, flat[guard:guard + numel].view(shape)

    bufs = {nm: padded5() for nm in ("o", "dq", "dk", "dv")}
    lse_flat, lse = guarded((1, h, rows, n), torch.float32)
    db_flat, db = guarded((1, h, n, n), dtype)
    abi_forward(q, k, v, b, m, bufs["o"][1], lse, kernel=_lib.KERNEL_TCGEN05)
    abi_backward(do, q, k, v, b, m, bufs["o"][1], lse, bufs["dq"][1], bufs["dk"][1], bufs["dv"][1],
                 db, kernel=_lib.KERNEL_TCGEN05)
    torch.cuda.synchronize()
    for nm, (flat, view) in bufs.items():
        assert bool((flat[:guard] == fill).all()) and bool((flat[-guard:] == fill).all()), nm
        body = flat[guard:-guard].view(1, h, rows, n, d + 8)
        assert bool((body[..., d:] == fill).all()), f"{nm}: row padding overwritten"
        assert torch.isfinite(view.float()).all(), nm
    for nm, flat in (("lse", lse_flat), ("db", db_flat)):
        assert bool((flat[:guard] == fill).all()) and bool((flat[-guard:] == fill).all()), nm
    # every output element was written: a second run into differently filled buffers agrees
    bufs2 = {nm: padded5() for nm in ("o", "dq", "dk", "dv")}
    for flat, _ in bufs2.values():
        flat.fill_(3.0)
    lse2 = torch.full_like(lse, 5.0)
    db2 = torch.full_like(db, 5.0)
    abi_forward(q, k, v, b, m, bufs2["o"][1], lse2, kernel=_lib.KERNEL_TCGEN05)
    abi_backward(do, q, k, v, b, m, bufs2["o"][1], lse2, bufs2["dq"][1], bufs2["dk"][1],
                 bufs2["dv"][1], db2, kernel=_lib.KERNEL_TCGEN05)
    torch.cuda.synchronize()
    for nm in bufs:
        assert torch.equal(bufs[nm][1], bufs2[nm][1]), f"{nm}: some element keeps its fill value"
    assert torch.equal(lse, lse2) and torch.equal(db, db2)


def test_a_wait_that_runs_out_becomes_an_exception_and_clears():
    """Failure detection without a fault: a test-only kernel waits, with the bounded wait
    all kernels use, on a barrier nobody arrives on; after 200 microseconds the wait gives
    up and sets the device status word.  Kernels launched while the word is set exit at
    once, so the next operator call must raise instead of returning unwritten memory; the
    call after that works again."""
    lib = _lib.load()
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    args = [t.to(DEV) for t in _inputs(128, 1, 32, torch.bfloat16, "none", 8)]
    q, k, v, b, m, do = args
    good = triangle_attention(q, k, v, b, m)
    torch.cuda.synchronize()
    assert lib.trifast_debug_wait_probe(200, st) == 0
    torch.cuda.synchronize()                      # the probe returned by itself
    # a call made now still runs (its kernels exit early); it leaves the snapshot behind
    triangle_attention(q, k, v, b, m)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="bounded wait"):
        triangle_attention(q, k, v, b, m)
    # the raise read and cleared the status
    assert lib.trifast_check_device_status(st) == 0
    again = triangle_attention(q, k, v, b, m)
    torch.cuda.synchronize()
    assert torch.equal(again, good)


def test_check_device_status_reports_the_probe():
    lib = _lib.load()
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.trifast_debug_wait_probe(50, st) == 0
    assert lib.trifast_check_device_status(st) == -11     # synchronises, reports, clears
    assert lib.trifast_check_device_status(st) == 0
    _lib._status_word(torch.device(DEV)).zero_()


@pytest.mark.parametrize("n,h,d,dtype", [(40, 2, 32, torch.float32), (136, 2, 32, torch.bfloat16)])
def test_ending_node_variant(n, h, d, dtype):
    """The pair-transposed operator against a direct statement of the ending-node formula,
    forward and (through autograd on that statement) backward."""
    from trifast_b200 import triangle_attention_ending_node
    torch.manual_seed(4)
    q, k, v = ((torch.randn(1, h, n, n, d) * d ** -0.5).to(dtype) for _ in range(3))
    b = torch.randn(1, h, n, n).to(dtype)
    m = torch.rand(1, n, n) < 0.25
    m[:, torch.arange(n), torch.arange(n)] = False
    do = torch.randn(1, h, n, n, d).to(dtype)
    ref_in = [t.double().requires_grad_(True) for t in (q, k, v, b)]
    ref_o = orc.forward_ending_node(*ref_in, m, torch.float64)
    ref_o.backward(do.double())
    got_in = [t.to(DEV).requires_grad_(True) for t in (q, k, v, b)]
    o = triangle_attention_ending_node(*got_in, m.to(DEV))
    o.backward(do.to(DEV))
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    for name, g, r in zip(NAMES, [o] + [t.grad for t in got_in], [ref_o] + [t.grad for t in ref_in]):
        assert rel_err(g.detach().float().cpu(), r.detach()) < tol, name


def test_leading_batch_dimensions():
    """Any number of leading batch dimensions, including none, gives the rows of the
    five-dimensional call."""
    torch.manual_seed(6)
    n, h, d = 48, 2, 32
    q, k, v = (torch.randn(2, 3, h, n, n, d, device=DEV, dtype=torch.bfloat16) for _ in range(3))
    b = torch.randn(2, 3, h, n, n, device=DEV, dtype=torch.bfloat16)
    m = torch.rand(2, 3, n, n, device=DEV) < 0.3
    o = triangle_attention(q, k, v, b, m)
    assert o.shape == q.shape
    flat = triangle_attention(q.flatten(0, 1), k.flatten(0, 1), v.flatten(0, 1), b.flatten(0, 1),
                              m.flatten(0, 1))
    assert torch.equal(o.flatten(0, 1), flat)
    single = triangle_attention(q[1, 2], k[1, 2], v[1, 2], b[1, 2], m[1, 2])
    assert single.shape == q.shape[2:] and torch.equal(single, o[1, 2])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("n", [128, 256])
def test_error_is_within_the_triton_kernels_own_error(dtype, n):
    """The bound the reference's kernels set themselves: tests/golden/triton_reference_b200.json
    holds the maximum absolute error of the unmodified Triton kernels against the fp64 oracle,
    measured on a B200 by baseline/triton_ref.py (same seed, same draws as here: h = 4, d = 32,
    std 1, Bernoulli(0.5) mask with the diagonal kept, dO ~ N(0, 1)).  Every output and
    gradient of this implementation must be at least as close to the oracle."""
    import json
    import os
    from tests.helpers import GOLDEN_DIR
    with open(os.path.join(GOLDEN_DIR, "triton_reference_b200.json")) as f:
        bound = json.load(f)["max_abs_err_vs_fp64_oracle"][f"{str(dtype).replace('torch.', '')}_n{n}"]
    torch.manual_seed(1337)
    h, d = 4, 32
    q, k, v = (torch.randn(1, h, n, n, d) for _ in range(3))
    b = torch.randn(1, h, n, n)
    m = torch.randint(0, 2, (1, n, n), dtype=torch.bool)
    m[:, torch.arange(n), torch.arange(n)] = False
    do = torch.randn(1, h, n, n, d)
    lo = [t.to(dtype) for t in (q, k, v, b, do)]
    ref_o, _ = orc.forward(*(t.float() for t in lo[:4]), m, torch.float64)
    ref_g = orc.backward(lo[4].float(), *(t.float() for t in lo[:4]), m, torch.float64)
    g = [t.to(DEV).requires_grad_(True) for t in lo[:4]]
    o = triangle_attention(g[0], g[1], g[2], g[3], m.to(DEV))
    o.backward(lo[4].to(DEV))
    torch.cuda.synchronize()
    for name, x, r in zip(NAMES, [o] + [t.grad for t in g], (ref_o,) + tuple(ref_g)):
        err = float((x.detach().double().cpu() - r.double()).abs().max())
        assert err <= bound[name], f"{name}: max abs err {err:.3e} > Triton kernel's {bound[name]:.3e}"


def _fuzz_cases(count=24, seed=2024):
    """Seeded random problems on the tensor-core path: ragged and aligned n up to 700, the three
    head dims and both 16-bit dtypes, row shards, and five mask patterns."""
    g = torch.Generator().manual_seed(seed)
    r = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=g))
    cases = []
    for idx in range(count):
        d = (16, 32, 64)[r(0, 2)]
        n = r(128, 700 if d <= 32 else 520)
        if r(0, 3) == 0:
            n = (n // 64) * 64                      # aligned now and then
        rows = n if r(0, 2) == 0 else r(1, min(n, 40))
        cases.append((idx, n, r(1, 3), d, (torch.bfloat16, torch.float16)[r(0, 1)],
                      ("none", "random", "padding", "sparse", "blocks")[r(0, 4)], min(rows, 48)))
    return cases


@pytest.mark.parametrize("idx,n,h,d,dtype,mask,rows",
                         _fuzz_cases(int(os.environ.get("TRIFAST_B200_FUZZ_DRAWS", "24"))))
def test_random_problems_against_the_oracle(idx, n, h, d, dtype, mask, rows):
    """o, dq, dk, dv, db of randomly drawn problems against the fp64 oracle (3 x (pt + eps) rule
    of the reference), plus exact zeros of dk, dv at dropped keys of partially masked rows."""
    g = torch.Generator().manual_seed(1000 + idx)
    q, k, v = ((torch.randn(1, h, rows, n, d, generator=g) * d ** -0.5).to(dtype) for _ in range(3))
    b = torch.randn(1, h, n, n, generator=g).to(dtype)
    do = torch.randn(1, h, rows, n, d, generator=g).to(dtype)
    if mask == "none":
        m = torch.zeros(1, rows, n, dtype=torch.bool)
    elif mask == "random":
        m = torch.rand(1, rows, n, generator=g) < 0.4
    elif mask == "padding":
        nv = int(0.7 * n)
        m = ((torch.arange(rows)[:, None] >= max(1, rows - 3)) | (torch.arange(n)[None, :] >= nv))[None]
    elif mask == "sparse":                              # almost everything dropped
        m = torch.rand(1, rows, n, generator=g) < 0.97
    else:                                               # whole 128-key tiles dropped on some rows
        m = torch.zeros(1, rows, n, dtype=torch.bool)
        m[0, ::2, 128:256] = True
        m[0, 1::3, : min(n, 128)] = True
    m = m.contiguous()
    got = tuple(t.float().cpu() for t in _run_abi((q, k, v, b, m, do), kernel=_lib.KERNEL_TCGEN05))
    f = [t.float() for t in (q, k, v, b)]
    o, _, grads = orc.forward_backward_chunked(f[0], f[1], f[2], f[3], m, do=do.float(),
                                               rows_per_chunk=8, acc_dtype=torch.float64)
    qq, kk, vv, bb = (t.detach().clone().requires_grad_(True) for t in (q, k, v, b))
    oo = orc.attention_reference_port(qq, kk, vv, bb, m)
    oo.backward(do)
    pt = tuple(t.detach().float() for t in (oo, qq.grad, kk.grad, vv.grad, bb.grad))
    tag = f"fuzz {idx}: n={n} h={h} d={d} {dtype} mask={mask} rows={rows}"
    for nm, x, r_, p in zip(NAMES, got, (o,) + grads, pt):
        assert_within_pt_error(x, p, r_, DTYPE_EPS[dtype], f"{tag} {nm}")
    partial = ~m.all(dim=-1)
    sel = (m & partial[..., None])[:, None, :, :, None].expand_as(got[2])
    if sel.any():
        assert float(got[2][sel].abs().max()) == 0.0 and float(got[3][sel].abs().max()) == 0.0, tag


HEAD_DIM_16_SHAPES = [  # (n, h, rows, dtype, mask)
    (128, 1, None, torch.bfloat16, "none"),
    (333, 2, None, torch.float16, "random"),
    (512, 2, 40, torch.bfloat16, "padding"),
    (1024, 1, 24, torch.bfloat16, "random"),     # all eight dQ tiles of one pass
    (1300, 1, 12, torch.float16, "padding"),     # two query chunks
]


@pytest.mark.parametrize("n,h,rows,dtype,mask", HEAD_DIM_16_SHAPES)
def test_head_dim_16_on_tensor_cores(n, h, rows, dtype, mask):
    """d = 16 (32-byte rows, 32-byte swizzle, 16-column accumulators): forward and backward on
    the tensor-core kernels against the fp64 oracle and against the CUDA-core kernels."""
    args = _inputs(n, h, 16, dtype, mask, rows)
    assert _lib.pick_plan(1, h, n, args[0].shape[2], 16, dtype)["kernel"] == _lib.KERNEL_TCGEN05
    got = tuple(t.float().cpu() for t in _run_abi(args, kernel=_lib.KERNEL_TCGEN05))
    simt = tuple(t.float().cpu() for t in _run_abi(args, kernel=_lib.KERNEL_SIMT))
    q, k, v, b, m, do = args
    f = [t.float() for t in (q, k, v, b)]
    o, _, grads = orc.forward_backward_chunked(f[0], f[1], f[2], f[3], m, do=do.float(),
                                               rows_per_chunk=8, acc_dtype=torch.float64)
    qq, kk, vv, bb = (t.detach().clone().requires_grad_(True) for t in (q, k, v, b))
    oo = orc.attention_reference_port(qq, kk, vv, bb, m)
    oo.backward(do)
    pt = tuple(t.detach().float() for t in (oo, qq.grad, kk.grad, vv.grad, bb.grad))
    for nm, x, y, r_, p in zip(NAMES, got, simt, (o,) + grads, pt):
        assert torch.isfinite(x).all(), nm
        assert_within_pt_error(x, p, r_, DTYPE_EPS[dtype], f"d=16 n={n} {nm}")
        assert_direction(x, p, r_, f"d=16 n={n} {nm}")
        assert max_abs(x, y) <= 3 * (max_abs(y, r_) + DTYPE_EPS[dtype]), f"d=16 n={n} {nm} vs CUDA cores"


@pytest.mark.parametrize("d,dtype", [(32, torch.bfloat16), (64, torch.float16), (16, torch.bfloat16)])
def test_key_tiles_without_an_open_key_are_skipped_exactly(d, dtype):
    """Rows whose open keys sit in a sub-range of the 128-key tiles (dropped head, dropped tail,
    both, a single open key, nothing dropped, everything dropped) next to each other: the
    kernels walk only each row's live tiles.  Outputs must equal the oracle, dk / dv must be
    exactly zero at every dropped key (walked or not), and where a two-kernel backward exists
    (it walks every tile) dq, dk, dv must agree with it bit for bit."""
    n, h, rows = 640, 2, 24                       # five key tiles
    q, k, v, b, _, do = _inputs(n, h, d, dtype, "none", rows, seed=11)
    m = torch.zeros(1, rows, n, dtype=torch.bool)
    keys = torch.arange(n)
    for i in range(rows):
        kind = i % 6
        if kind == 0:
            m[0, i] = keys < 128 + 7 * i                     # head dropped: first live tile 1
        elif kind == 1:
            m[0, i] = keys >= 300 - i                        # tail dropped: live tiles 0..2
        elif kind == 2:
            m[0, i] = (keys < 256) | (keys >= 384)           # only tile 2 live
        elif kind == 3:
            m[0, i] = keys != (77 * i) % n                   # a single open key
        elif kind == 4:
            m[0, i] = False
        else:
            m[0, i] = True                                   # fully masked: all n keys, uniform
    m = m.contiguous()
    args = (q, k, v, b, m, do)
    got = tuple(t.float().cpu() for t in _run_abi(args, kernel=_lib.KERNEL_TCGEN05))
    f = [t.float() for t in (q, k, v, b)]
    o, _, grads = orc.forward_backward_chunked(f[0], f[1], f[2], f[3], m, do=do.float(),
                                               rows_per_chunk=8, acc_dtype=torch.float64)
    qq, kk, vv, bb = (t.detach().clone().requires_grad_(True) for t in (q, k, v, b))
    oo = orc.attention_reference_port(qq, kk, vv, bb, m)
    oo.backward(do)
    pt = tuple(t.detach().float() for t in (oo, qq.grad, kk.grad, vv.grad, bb.grad))
    for nm, x, r_, p in zip(NAMES, got, (o,) + grads, pt):
        assert torch.isfinite(x).all(), nm
        assert_within_pt_error(x, p, r_, DTYPE_EPS[dtype], f"live tiles d={d} {nm}")
    partial = ~m.all(dim=-1)
    sel = (m & partial[..., None])[:, None, :, :, None].expand_as(got[2])
    assert float(got[2][sel].abs().max()) == 0.0 and float(got[3][sel].abs().max()) == 0.0
    if d != 16:
        split = tuple(t.float().cpu() for t in _run_abi(args, kernel=_lib.KERNEL_TCGEN05,
                                                        flags=_lib.FLAG_SPLIT_BWD))
        # (a row walked in several query chunks sums dK / dV in another order: o and dq only)
        one_pass = _lib.pick_plan(1, h, n, rows, d, dtype)["bwd_chunks"] == 1
        for nm, x, y in zip(NAMES[:4], got[:4], split[:4]):
            if one_pass or nm in ("o", "dq"):
                assert torch.equal(x, y), f"{nm}: the walk over live tiles differs from the walk over all"
