"""GPU tier: the CUDA path (through the public op, i.e. through the C ABI) against
the CPU oracle and the reference-generated golden vectors.

Tolerances
* fp32: max|x - ref| / max|ref| <= 1e-4 against the fp64 oracle, for o, dq, dk, dv, db.
* bf16 / fp16: the reference's own rule (tests/utils.py:31-36 there): kernel error
  <= 3 * (error of PyTorch run in the same dtype + eps), eps = 1e-3, plus its
  direction rules (cosine > 0.99, >= 0.99 * PyTorch's, projection within 0.01).
* masked keys: exactly zero weight (bitwise-identical outputs when masked k/v change).
"""

import os

import pytest
import torch

from oracle import triangle_oracle as orc
from tests.helpers import (DTYPE_EPS, FP32_REL_TOL, assert_direction, assert_within_pt_error,
                           golden_cases, load_golden, max_abs, rel_err)
from trifast_b200 import triangle_attention
from trifast_b200.configs import WORKLOADS, Workload, make_inputs
from trifast_b200.utils import gen_tensors

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True)
def device_status_is_clean():
    """No kernel may have given up on one of its bounded waits during a test."""
    yield
    import ctypes
    from trifast_b200 import _lib
    rc = _lib.load().trifast_check_device_status(
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, _lib.status_str(rc)

NAMES = ("o", "dq", "dk", "dv", "db")


def run_kernel(q, k, v, b, m, do):
    q, k, v, b = (t.detach().to(DEV).requires_grad_(True) for t in (q, k, v, b))
    o = triangle_attention(q, k, v, b, m.to(DEV))
    o.backward(do.to(DEV))
    torch.cuda.synchronize()
    return tuple(t.detach().float().cpu() for t in (o, q.grad, k.grad, v.grad, b.grad))


def run_oracle64(q, k, v, b, m, do):
    o, _ = orc.forward(q, k, v, b, m, torch.float64)
    return (o,) + orc.backward(do, q, k, v, b, m, torch.float64)


def run_pt(q, k, v, b, m, do):
    """PyTorch in the inputs' dtype on the CPU (the error bar of the relative rule)."""
    q, k, v, b = (t.detach().clone().requires_grad_(True) for t in (q, k, v, b))
    o = orc.attention_reference_port(q, k, v, b, m)
    o.backward(do)
    return tuple(t.detach().float() for t in (o, q.grad, k.grad, v.grad, b.grad))


def check(dtype, got, ref, pt, tag):
    for name, g, r, p in zip(NAMES, got, ref, pt if pt is not None else ref):
        if dtype == torch.float32:
            e = rel_err(g, r)
            assert e <= FP32_REL_TOL, f"{tag} {name}: rel err {e:.3e} > {FP32_REL_TOL}"
        else:
            assert_within_pt_error(g, p, r, DTYPE_EPS[dtype], f"{tag} {name}")
            assert_direction(g, p, r, f"{tag} {name}")


@pytest.mark.parametrize("case", golden_cases())
def test_golden_vectors(case):
    t, dtype = load_golden(case)
    args = tuple(t[x].to(dtype) for x in ("q", "k", "v", "bias")) + (t["mask"], t["do"].to(dtype))
    got = run_kernel(*args)
    stored = tuple(t[x] for x in NAMES)
    if dtype == torch.float32:
        check(dtype, got, stored, None, case)      # the reference's own fp32 results
    else:
        ref = run_oracle64(*args)
        check(dtype, got, ref, stored, case)       # stored = the reference run in bf16


def seeded(n, h, d, dtype, use_mask, bs, std, seed=1337):
    torch.manual_seed(seed)
    q, k, v, b, m = gen_tensors(n, d, h, use_mask, "cpu", torch.float32, batch=bs, std=std)
    do = torch.randn(q.shape)
    return tuple(t.detach().to(dtype) for t in (q, k, v, b)) + (m, do.to(dtype))


SHAPES = [(16, 1, 16), (32, 1, 32), (64, 1, 64), (16, 4, 128), (191, 4, 32)] + \
         [(n, 4, 32) for n in (17, 31, 33, 63, 65, 96, 100, 127, 128, 129, 136, 160, 199)] + \
         [(128, 2, 64), (144, 2, 64), (256, 2, 32), (264, 1, 32), (257, 2, 32), (333, 1, 64)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("use_mask", [True, False])
@pytest.mark.parametrize("n,h,d", SHAPES)
def test_values_and_directions(n, h, d, dtype, use_mask):
    """The reference's test_values / test_vectors matrix (tests/unit/test_trifast.py:26-149),
    thinned in n, with random dO instead of ones."""
    bs, std = (2, 2.0) if n % 2 else (1, 1.0)
    args = seeded(n, h, d, dtype, use_mask, bs, std)
    got = run_kernel(*args)
    ref = run_oracle64(*args)
    pt = None if dtype == torch.float32 else run_pt(*args)
    check(dtype, got, ref, pt, f"n={n} h={h} d={d} {dtype} mask={use_mask}")


@pytest.mark.parametrize("name", ["c1_cpu_plumbing", "c2_n256", "c3_n512_pad"])
def test_named_workloads(name):
    w = WORKLOADS[name]
    args = make_inputs(w, seed=1337)
    got = run_kernel(*args)
    q, k, v, b, m, do = args
    o, lse, grads = orc.forward_backward_chunked(q, k, v, b, m, do=do, rows_per_chunk=16,
                                                 acc_dtype=torch.float64)
    ref = (o,) + grads
    pt = None
    if w.dtype != torch.float32:
        # same-dtype PyTorch error bar, row-chunked (rows are independent; db adds up)
        parts = [run_pt(q[:, :, r:r + 32], k[:, :, r:r + 32], v[:, :, r:r + 32], b,
                        m[:, r:r + 32], do[:, :, r:r + 32]) for r in range(0, w.n, 32)]
        pt = tuple(torch.cat([p[x] for p in parts], dim=2) for x in range(4)) + \
            (sum(p[4] for p in parts),)
    check(w.dtype, got, ref, pt, name)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n", [48, 131, 256])
def test_masked_keys_have_exactly_zero_weight(dtype, n):
    q, k, v, b, m, do = seeded(n, 2, 32, dtype, True, 1, 1.0, seed=5)
    m[0, 3] = True                                     # one fully masked row as well
    partial = ~m.all(dim=-1)
    sel = (m & partial[..., None])[:, None, :, :, None].expand_as(v)
    v2, k2 = v.clone(), k.clone()
    v2[sel] = 77.0
    k2[sel] = -55.0
    a = run_kernel(q, k, v, b, m, do)
    c = run_kernel(q, k2, v2, b, m, do)
    assert torch.equal(a[0], c[0]), "o changed when masked k/v changed"
    # masked keys of partially masked rows receive exactly zero dk, dv
    assert float(a[2][sel].abs().max()) == 0.0 and float(a[3][sel].abs().max()) == 0.0
    # the fully masked row is the mean of v
    mean_v = v[0, :, 3].float().mean(dim=1)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert float((a[0][0, :, 3] - mean_v[:, None, :]).abs().max()) < tol


@pytest.mark.parametrize("n", [136, 203])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_row_shards_match_whole_problem(dtype, n):
    """Rows are independent: running rows [r0, r1) alone gives the same o, dq, dk, dv,
    bit for bit, and the shard db partials add up to the whole db."""
    q, k, v, b, m, do = seeded(n, 2, 32, dtype, True, 1, 1.0, seed=9)
    whole = run_kernel(q, k, v, b, m, do)
    db = 0
    for r in (slice(0, 50), slice(50, n)):
        part = run_kernel(q[:, :, r], k[:, :, r], v[:, :, r], b, m[:, r], do[:, :, r])
        for x in range(4):
            assert torch.equal(part[x], whole[x][:, :, r]), NAMES[x]
        db = db + part[4].double()
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert rel_err(db, whole[4].double()) < tol


def test_run_to_run_determinism():
    args = seeded(160, 2, 32, torch.bfloat16, True, 1, 1.0)
    a, c = run_kernel(*args), run_kernel(*args)
    for x, y, name in zip(a, c, NAMES):
        assert torch.equal(x, y), name


def test_non_contiguous_inputs():
    """(b, n, n, h, d) projections permuted to (b, h, n, n, d) are consumed through strides."""
    torch.manual_seed(3)
    n, h, d = 40, 2, 32
    base = [torch.randn(1, n, n, h, d) for _ in range(3)]
    q, k, v = (t.permute(0, 3, 1, 2, 4) for t in base)
    b = torch.randn(1, n, n, h).permute(0, 3, 1, 2)
    m = torch.rand(1, n, n) < 0.3
    do = torch.randn(1, h, n, n, d)
    got = run_kernel(q, k, v, b, m, do)
    ref = run_oracle64(q, k, v, b, m, do)
    check(torch.float32, got, ref, None, "permuted")


def test_full_size_properties():
    """Metric shape (n = 1024, h = 4, d = 32, bf16): properties that need no CPU oracle.
    * with v = 1 everywhere every output is exactly 1 (weights sum to one);
    * the forward is linear in v;
    * a second run reproduces the first bit for bit;
    * a 32-row sample of the output matches the oracle."""
    w = WORKLOADS["metric_n1024"]
    q, k, v, b, m, do = make_inputs(w, seed=1, device=DEV)
    o1 = triangle_attention(q, k, v, b, m)
    ones = triangle_attention(q, k, torch.ones_like(v), b, m)
    assert float((ones.float() - 1).abs().max()) <= 2 ** -7
    v2 = torch.randn_like(v) * 0.2
    lin = triangle_attention(q, k, (v.float() + v2.float()).to(v.dtype), b, m).float()
    sep = o1.float() + triangle_attention(q, k, v2, b, m).float()
    assert float((lin - sep).abs().max()) < 3e-2
    assert torch.equal(o1, triangle_attention(q, k, v, b, m))
    rows = slice(500, 532)
    ref, _ = orc.forward(q[:, :, rows].cpu(), k[:, :, rows].cpu(), v[:, :, rows].cpu(), b.cpu(),
                         m[:, rows].cpu(), torch.float32)
    assert rel_err(o1[:, :, rows].float().cpu(), ref) < 2e-2


@pytest.mark.parametrize("name", ["metric_n1024"])
def test_full_size_against_chunked_oracle(name):
    """The headline shape, forward and backward, against the fp32 CPU oracle run in
    row chunks (rows are independent; db accumulates over chunks).  bf16 bound:
    max|x - ref| / max|ref| <= 2e-2 for o, dq, dk, dv and <= 3e-2 for db, i.e. a few
    bf16 roundings of the largest value (the same-dtype PyTorch error on smaller
    problems of this family is 1e-2 .. 9e-2)."""
    w = WORKLOADS[name]
    q, k, v, b, m, do = make_inputs(w, seed=1337, device=DEV)
    got = run_kernel(q, k, v, b, m, do)
    cpu = [t.float().cpu() for t in (q, k, v, b)] + [m.cpu(), do.float().cpu()]
    o, lse, grads = orc.forward_backward_chunked(cpu[0], cpu[1], cpu[2], cpu[3], cpu[4], do=cpu[5],
                                                 rows_per_chunk=8, acc_dtype=torch.float32)
    for nm, g, r, tol in zip(NAMES, got, (o,) + grads, (2e-2, 2e-2, 2e-2, 2e-2, 3e-2)):
        e = rel_err(g, r)
        assert e <= tol, f"{name} {nm}: rel err {e:.3e} > {tol}"


_EXTRA_TC_SHAPES = {
    # head dim 64 with the backward, at the largest n of the table and with a ragged n
    "n2048_h2_d64_bwd": Workload("n2048_h2_d64_bwd", 2048, 2, 64, torch.float16, "random:0.2"),
    "n1001_h2_d64_bwd": Workload("n1001_h2_d64_bwd", 1001, 2, 64, torch.bfloat16, "padding:0.9"),
    "n4096_h1_d32_bwd": Workload("n4096_h1_d32_bwd", 4096, 1, 32, torch.bfloat16, "none"),
}


@pytest.mark.parametrize("name", ["c2_n256", "c3_n512_pad", "c4_n1024_h8_d64_fwd", "c5_n2048_pad",
                                  "metric_n1024"] + sorted(_EXTRA_TC_SHAPES))
def test_configured_workloads_run_on_tensor_cores(name, monkeypatch):
    """With the kernel choice forced to tcgen05 an unsupported problem is an error instead
    of a silent fall-back to the CUDA-core kernels: every 16-bit workload of the table must
    pass (a few pair rows are enough: the tile plan depends on n, h, d and the dtype)."""
    monkeypatch.setenv("TRIFAST_B200_KERNEL", "tcgen05")
    w = WORKLOADS.get(name) or _EXTRA_TC_SHAPES[name]
    q, k, v, b, m, do = make_inputs(w, seed=3, device=DEV, sample_rows=6)
    got = run_kernel(q, k, v, b, m, do) if w.backward else None
    if got is None:
        o = triangle_attention(q, k, v, b, m)
        torch.cuda.synchronize()
        got = (o.float().cpu(),)
    cpu = [t.float().cpu() for t in (q, k, v, b)]
    ref, _ = orc.forward(cpu[0], cpu[1], cpu[2], cpu[3], m.cpu(), torch.float32)
    assert rel_err(got[0], ref) < 2e-2


def test_opcheck():
    """torch.library.opcheck on the forward op (tests/unit/test_trifast_opcheck.py:7-13)."""
    from torch.library import opcheck
    from trifast_b200.torch import _triangle_attention
    for n, d, h in [(16, 16, 1), (128, 32, 4), (136, 64, 1)]:
        q, k, v, b, m = gen_tensors(n, d, h, True, DEV, dtype=torch.bfloat16)
        opcheck(_triangle_attention, (q, k, v, b, m), raise_exception=True)


def test_torch_compile_fullgraph():
    q, k, v, b, m = gen_tensors(64, 32, 2, True, DEV, dtype=torch.bfloat16)
    fn = torch.compile(triangle_attention, fullgraph=True)
    o = fn(q, k, v, b, m)
    assert torch.equal(o, triangle_attention(q, k, v, b, m))
    o.sum().backward()
    assert q.grad is not None and b.grad is not None


def test_weight_updates():
    """Five Adam steps through a toy projection module change every parameter
    (tests/unit/test_trifast.py:152-211 of the reference, in the canonical layout)."""
    torch.manual_seed(0)
    n, h, d = 32, 2, 32

    class Toy(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.q, self.k, self.v = (torch.nn.Linear(d, h * d) for _ in range(3))
            self.b = torch.nn.Linear(d, h)

        def forward(self, x, mask):
            split = lambda t: t.unflatten(-1, (h, d)).permute(0, 3, 1, 2, 4)
            return triangle_attention(split(self.q(x)), split(self.k(x)), split(self.v(x)),
                                      self.b(x).permute(0, 3, 1, 2), mask)

    model = Toy().to(DEV, torch.bfloat16)
    opt = torch.optim.Adam(model.parameters(), lr=1e-3)
    x = torch.randn(1, n, n, d, device=DEV, dtype=torch.bfloat16)
    mask = torch.zeros(1, n, n, dtype=torch.bool, device=DEV)
    before = {k: p.clone() for k, p in model.named_parameters()}
    for _ in range(5):
        out = model(x, mask)
        loss = torch.nn.functional.mse_loss(out, torch.randn_like(out) * 4)
        opt.zero_grad()
        loss.backward()
        opt.step()
    for k, p in model.named_parameters():
        assert not torch.equal(before[k], p), f"parameter {k} did not update"


def _random_square_cases(count=32, seed=77):
    g = torch.Generator().manual_seed(seed)
    r = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=g))
    cases = []
    for idx in range(count):
        d = (16, 32, 64, 128)[r(0, 3)]
        n = r(1, 260) if r(0, 3) else r(1, 24)
        cases.append((idx, n, r(1, 4), d, r(1, 2), (torch.float32, torch.bfloat16, torch.float16)[r(0, 2)],
                      ("none", "random", "head", "tail", "sparse")[r(0, 4)], ("dense", "permuted")[r(0, 1)],
                      (0.5, 1.0, 2.0)[r(0, 2)]))
    return cases


@pytest.mark.parametrize("idx,n,h,d,bs,dtype,mask,layout,std",
                         _random_square_cases(int(os.environ.get("TRIFAST_B200_FUZZ_DRAWS", "32"))))
def test_random_square_problems_through_the_public_op(idx, n, h, d, bs, dtype, mask, layout, std):
    """Seeded random whole problems through `triangle_attention` + autograd (every kernel family:
    n < 64, d = 128 and fp32 on CUDA cores, the rest on tensor cores), batch 1-2, dense or
    permuted-projection layouts, masks that drop the head or the tail of the keys, input scale
    0.5-2 (flat to peaked softmax), against the fp64 oracle."""
    g = torch.Generator().manual_seed(5000 + idx)
    if layout == "dense":
        q, k, v = (torch.randn(bs, h, n, n, d, generator=g) * std for _ in range(3))
        b = torch.randn(bs, h, n, n, generator=g) * std
    else:
        q, k, v = ((torch.randn(bs, n, n, h, d, generator=g) * std).permute(0, 3, 1, 2, 4) for _ in range(3))
        b = (torch.randn(bs, n, n, h, generator=g) * std).permute(0, 3, 1, 2)
    q, k, v, b = (t.to(dtype) for t in (q, k, v, b))
    do = torch.randn(bs, h, n, n, d, generator=g).to(dtype)
    keys = torch.arange(n)
    if mask == "none":
        m = torch.zeros(bs, n, n, dtype=torch.bool)
    elif mask == "random":
        m = torch.rand(bs, n, n, generator=g) < 0.5
    elif mask == "head":                               # the first keys dropped, row by row differently
        cut = torch.randint(0, n + 1, (bs, n, 1), generator=g)
        m = keys[None, None, :] < cut
    elif mask == "tail":
        cut = torch.randint(0, n + 1, (bs, n, 1), generator=g)
        m = keys[None, None, :] >= cut
    else:
        m = torch.rand(bs, n, n, generator=g) < 0.95
    m = m.contiguous()
    got = run_kernel(q, k, v, b, m, do)
    ref = run_oracle64(q, k, v, b, m, do)
    tag = f"draw {idx}: n={n} h={h} d={d} bs={bs} {dtype} mask={mask} {layout} std={std}"
    if dtype == torch.float32:
        for name, x, r_ in zip(NAMES, got, ref):
            assert torch.isfinite(x).all(), f"{tag} {name}: not finite"
            # (floor on the scale: with one open key per row dq, dk and db are zero in exact
            # arithmetic and fp32 leaves the rounding of dP - delta, two sums of d products
            # of size ~sqrt(d) each)
            e = max_abs(x, r_) / max(float(r_.abs().max()), 1e-2 * d ** 0.5)
            assert e <= FP32_REL_TOL, f"{tag} {name}: rel err {e:.3e}"
    else:
        pt = run_pt(q, k, v, b, m, do)
        for name, x, r_, p in zip(NAMES, got, ref, pt):
            assert torch.isfinite(x).all(), f"{tag} {name}: not finite"
            assert_within_pt_error(x, p, r_, DTYPE_EPS[dtype], f"{tag} {name}")


@pytest.mark.parametrize("n,d,dtype", [(192, 32, torch.bfloat16), (96, 128, torch.float16), (40, 32, torch.float32)])
def test_step_can_be_captured_in_a_cuda_graph(n, d, dtype):
    """Forward + backward through the public op inside a CUDA graph (tensor-core kernels, the
    head-dim-128 pair and the CUDA-core kernels): nothing in the library allocates device
    memory, synchronises or calls anything a capture forbids once the first call on the device
    has been made.  The replay, on new input values, must equal the eager result bit for bit."""
    h = 2
    g0 = torch.Generator().manual_seed(21)
    draw = lambda *s: torch.randn(*s, generator=g0)
    stat = [(draw(1, h, n, n, d) * d ** -0.5).to(dtype).to(DEV) for _ in range(3)]
    stat.append(draw(1, h, n, n).to(dtype).to(DEV))
    q, k, v, b = (t.requires_grad_(True) for t in stat)
    m = (torch.rand(1, n, n, generator=g0) < 0.3).to(DEV)
    do = draw(1, h, n, n, d).to(dtype).to(DEV)

    def step():
        o = triangle_attention(q, k, v, b, m)
        return (o,) + torch.autograd.grad(o, (q, k, v, b), do)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            step()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = step()
    # new values in the captured buffers
    with torch.no_grad():
        for t in (q, k, v):
            t.copy_((draw(1, h, n, n, d) * d ** -0.5).to(dtype))
        b.copy_(draw(1, h, n, n).to(dtype))
        do.copy_(draw(1, h, n, n, d).to(dtype))
        m.copy_(torch.rand(1, n, n, generator=g0) < 0.5)
    graph.replay()
    torch.cuda.synchronize()
    replayed = [t.clone() for t in outs]
    eager = step()
    torch.cuda.synchronize()
    for name, x, y in zip(NAMES, replayed, eager):
        assert torch.isfinite(x.float()).all(), name
        assert torch.equal(x, y), f"{name}: graph replay differs from the eager step"
