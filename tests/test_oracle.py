"""Pins the CPU oracle against vectors produced by the reference's own
``attention_reference`` + autograd (tests/golden/*.npz), and checks its internal
consistency.  No GPU needed."""

import pytest
import torch

from oracle import triangle_oracle as orc
from tests.helpers import golden_cases, load_golden, rel_err, max_abs


@pytest.mark.parametrize("case", golden_cases())
def test_explicit_formulas_match_reference_vectors(case):
    t, dtype = load_golden(case)
    o, lse = orc.forward(t["q"], t["k"], t["v"], t["bias"], t["mask"], torch.float64)
    dq, dk, dv, db = orc.backward(t["do"], t["q"], t["k"], t["v"], t["bias"], t["mask"],
                                  torch.float64)
    # fp32 vectors: the reference ran in fp32, the oracle in fp64 -> 1e-5 relative.
    # bf16 vectors: the reference rounded every intermediate to bf16.
    tol = 2e-5 if dtype == torch.float32 else 6e-2
    for name, got in (("o", o), ("dq", dq), ("dk", dk), ("dv", dv), ("db", db)):
        assert rel_err(got, t[name]) < tol, (case, name, rel_err(got, t[name]))


@pytest.mark.parametrize("case", golden_cases())
def test_port_reproduces_reference_vectors(case):
    """The autograd-capable port, run in the case's dtype, equals the stored
    reference results to rounding noise (bit-identical op sequence is not
    required: einsum vs matmul may differ in summation order)."""
    t, dtype = load_golden(case)
    q, k, v, b = (t[x].to(dtype).requires_grad_(True) for x in ("q", "k", "v", "bias"))
    o = orc.attention_reference_port(q, k, v, b, t["mask"])
    o.backward(t["do"].to(dtype))
    tol = 1e-5 if dtype == torch.float32 else 4e-2
    for name, got in (("o", o), ("dq", q.grad), ("dk", k.grad), ("dv", v.grad), ("db", b.grad)):
        assert rel_err(got.detach().float(), t[name]) < tol, (case, name)


def test_fully_masked_rows_are_uniform():
    """Rows whose keys are all masked get weights 1/n (the finite sentinel absorbs
    the logits), so o is the mean of v over all keys."""
    t, _ = load_golden("n24_padrows_fp32")
    o, lse = orc.forward(t["q"], t["k"], t["v"], t["bias"], t["mask"])
    full = t["mask"].all(dim=-1)                      # (b, i)
    assert full.any()
    i = int(full[0].nonzero()[0])
    mean_v = t["v"][0, :, i].mean(dim=1, keepdim=True).expand(-1, t["v"].shape[3], -1)
    assert max_abs(o[0, :, i], mean_v) < 1e-6
    assert max_abs(o[0, :, i], t["o"][0, :, i]) < 1e-6


def test_masked_keys_have_zero_weight():
    t, _ = load_golden("ragged17_randmask_fp32")
    o1, _ = orc.forward(t["q"], t["k"], t["v"], t["bias"], t["mask"])
    v2 = t["v"].clone()
    k2 = t["k"].clone()
    m = t["mask"][:, None, :, :, None].expand_as(v2)
    partial = ~t["mask"].all(dim=-1)[:, None, :, None, None]
    sel = m & partial
    v2[sel] += 100.0
    k2[sel] -= 50.0
    o2, _ = orc.forward(t["q"], k2, v2, t["bias"], t["mask"])
    rows = partial.expand_as(o1)
    assert torch.equal(o1[rows], o2[rows])


def test_chunked_equals_whole():
    t, _ = load_golden("n32_h4_d32_drop10_fp32")
    args = (t["q"], t["k"], t["v"], t["bias"], t["mask"])
    o, lse = orc.forward(*args)
    g = orc.backward(t["do"], *args)
    oc, lc, gc = orc.forward_backward_chunked(*args, do=t["do"], rows_per_chunk=5)
    assert torch.equal(o, oc) and torch.equal(lse, lc)
    for a, b in zip(g[:3], gc[:3]):
        assert torch.equal(a, b)
    assert rel_err(gc[3], g[3]) < 1e-5


def test_row_shards_sum_to_full_db():
    t, _ = load_golden("n32_h4_d32_drop10_fp32")
    full = orc.backward(t["do"], t["q"], t["k"], t["v"], t["bias"], t["mask"], torch.float64)
    db = 0
    for r in (slice(0, 11), slice(11, 32)):
        part = orc.backward(t["do"][:, :, r], t["q"][:, :, r], t["k"][:, :, r], t["v"][:, :, r],
                            t["bias"], t["mask"][:, r], torch.float64)
        db = db + part[3]
        assert max_abs(part[0], full[0][:, :, r]) < 1e-12
    assert max_abs(db, full[3]) < 1e-10


def test_work_accounting():
    assert orc.flops_forward(1, 4, 1024, 32) == pytest.approx(5.498e11, rel=1e-3)
    assert orc.flops_forward(1, 4, 1024, 32) + orc.flops_backward(1, 4, 1024, 32) == \
        pytest.approx(1.924e12, rel=1e-3)
    assert orc.hbm_bytes_forward(1, 4, 1024, 32, 2) == pytest.approx(1100e6, rel=2e-2)
    assert orc.hbm_bytes_backward(1, 4, 1024, 32, 2) == pytest.approx(2182e6, rel=2e-2)


@pytest.mark.parametrize("case,n,h,d,batch,std,use_mask,seed", [
    ("ragged17_randmask_fp32", 17, 2, 16, 2, 1.0, True, 1337),
    ("n19_d128_randmask_fp32", 19, 1, 128, 1, 1.0, True, 5),
    ("n25_d64_std2_nomask_fp32", 25, 1, 64, 1, 2.0, False, 11),
])
def test_gen_tensors_reproduces_the_reference_generator(case, n, h, d, batch, std, use_mask, seed):
    """The fixtures hold what the reference's own gen_tensors drew after
    torch.manual_seed(seed) (tests/golden/make_golden.py); this package's generator
    must draw the same bits: same order (q, k, v, bias, mask), same distributions."""
    from tests.helpers import load_golden
    from trifast_b200.utils import gen_tensors
    t, _ = load_golden(case)
    torch.manual_seed(seed)
    q, k, v, b, m = gen_tensors(n, d, h, use_mask, "cpu", dtype=torch.float32, batch=batch, std=std)
    do = torch.randn(q.shape)                        # the fixture's next draw
    for name, got in (("q", q), ("k", k), ("v", v), ("bias", b), ("do", do)):
        assert torch.equal(got.detach(), t[name]), name
    assert torch.equal(m, t["mask"])
    assert all(x.requires_grad and x.is_leaf for x in (q, k, v, b))
