"""Shared helpers of the parity tests (CPU and GPU tiers)."""

import glob
import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# eps of the reference's relative rule, per dtype (tests/unit/test_trifast.py:19-23
# of the reference).
DTYPE_EPS = {torch.float16: 1e-3, torch.bfloat16: 1e-3, torch.float32: 1e-4}
# fp32 contract: max-abs error relative to the largest reference magnitude.
FP32_REL_TOL = 1e-4


def golden_cases():
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN_DIR, "*.npz")))


def load_golden(name):
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    dtype = getattr(torch, str(z["dtype"]))
    t = {k: torch.from_numpy(z[k]) for k in z.files if k != "dtype"}
    return t, dtype


def rel_err(x, ref):
    """max|x - ref| / max|ref| in fp64 (the denominator floored at 1e-6: a reference that
    is zero throughout, such as dq for n = 1, is compared absolutely)."""
    x, ref = x.double(), ref.double()
    return float((x - ref).abs().max() / ref.abs().max().clamp_min(1e-6))


def max_abs(x, ref):
    return float((x.double() - ref.double()).abs().max())


def cosine(a, b):
    a, b = a.double().flatten(), b.double().flatten()
    return float(torch.dot(a, b) / (a.norm() * b.norm() + 1e-30))


def assert_within_pt_error(kernel, pt, ref, eps, what):
    """The reference's value rule: kernel error <= 3 * (same-dtype PyTorch error + eps)
    (tests/utils.py:31-36 of the reference)."""
    a = max_abs(kernel, ref)
    b = max_abs(pt, ref) + eps
    assert a <= 3 * b, f"{what}: kernel err {a:.3e} > 3 * (pt err + eps) = {3 * b:.3e}"


def assert_direction(kernel, pt, ref, what):
    """The reference's direction rules (tests/utils.py:56-83, test_trifast.py:73-89)."""
    ck, cp = cosine(kernel, ref), cosine(pt, ref)
    assert ck > 0.99, f"{what}: cosine(kernel, ref) = {ck:.4f}"
    assert ck >= 0.99 * cp, f"{what}: cosine(kernel, ref) {ck:.4f} < 0.99 * {cp:.4f}"
    rr = float(torch.dot(ref.double().flatten(), ref.double().flatten()))
    sk = float(torch.dot(kernel.double().flatten(), ref.double().flatten())) / rr
    sp = float(torch.dot(pt.double().flatten(), ref.double().flatten())) / rr
    assert sk - sp >= -0.01, f"{what}: projection {sk:.4f} vs pt {sp:.4f}"


# ---------------------------------------------------------------------------
# Direct calls through the C ABI with caller-owned outputs (GPU tests that need to
# look at the memory around the outputs, or to force a kernel choice per call).
# ---------------------------------------------------------------------------
def abi_forward(q, k, v, bias, mask, o, lse, kernel=None, flags=0):
    import ctypes as C
    from trifast_b200 import _lib
    lib = _lib.load()
    bs, h, rows, n, d = q.shape
    shp = _lib.make_shape(bs, h, n, rows, d, q.dtype, kernel, flags)
    wsb = lib.trifast_forward_workspace_bytes(C.byref(shp))
    ws = torch.empty(max(wsb, 1), dtype=torch.uint8, device=q.device)
    m8 = mask.view(torch.uint8)
    rc = lib.trifast_forward(C.byref(shp), C.byref(_lib.t5(q)), C.byref(_lib.t5(k)),
                             C.byref(_lib.t5(v)), C.byref(_lib.t4(bias)), C.byref(_lib.mask_view(m8)),
                             C.byref(_lib.t5(o)), C.c_void_p(lse.data_ptr()),
                             C.c_void_p(ws.data_ptr()), C.c_size_t(wsb),
                             C.c_void_p(torch.cuda.current_stream().cuda_stream))
    _lib.check(rc, "trifast_forward")


def abi_backward(do, q, k, v, bias, mask, o, lse, dq, dk, dv, db, kernel=None, flags=0):
    import ctypes as C
    from trifast_b200 import _lib
    lib = _lib.load()
    bs, h, rows, n, d = q.shape
    shp = _lib.make_shape(bs, h, n, rows, d, q.dtype, kernel, flags)
    wsb = lib.trifast_backward_workspace_bytes(C.byref(shp))
    ws = torch.empty(wsb, dtype=torch.uint8, device=q.device)
    m8 = mask.view(torch.uint8)
    rc = lib.trifast_backward(
        C.byref(shp), C.byref(_lib.t5(do)), C.byref(_lib.t5(q)), C.byref(_lib.t5(k)),
        C.byref(_lib.t5(v)), C.byref(_lib.t4(bias)), C.byref(_lib.mask_view(m8)),
        C.byref(_lib.t5(o)), C.c_void_p(lse.data_ptr()), C.byref(_lib.t5(dq)),
        C.byref(_lib.t5(dk)), C.byref(_lib.t5(dv)), C.byref(_lib.t4(db)),
        C.c_void_p(ws.data_ptr()), C.c_size_t(wsb),
        C.c_void_p(torch.cuda.current_stream().cuda_stream))
    _lib.check(rc, "trifast_backward")
