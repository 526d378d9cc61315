"""ctypes binding of ``libtrifast_b200.so`` (declarations: include/trifast_b200.h).

The library is the only compute path: if it is missing or fails to load, calls
raise instead of falling back to anything else.
"""

from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtrifast_b200.so")

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
KERNEL_AUTO, KERNEL_SIMT, KERNEL_TCGEN05 = 0, 1, 2
FLAG_SPLIT_BWD, FLAG_SHARE_GPU = 1, 2   # trifast_flags of the header


def share_gpu_flags(free_sms: int = 0) -> int:
    """TRIFAST_FLAG_SHARE_GPU with the number of SMs to leave free (0: the library's 8)."""
    if not 0 <= free_sms <= 255:
        raise ValueError("free_sms must be 0..255")
    return FLAG_SHARE_GPU | (free_sms << 8)
STATIC_SCRATCH_BYTES = 16 << 20   # TRIFAST_STATIC_SCRATCH_BYTES of the header
_KERNEL_ENV = {"": 0, "auto": 0, "simt": 1, "tcgen05": 2}


class Shape(C.Structure):
    _fields_ = [(n, C.c_int32) for n in
                ("batch", "heads", "n", "n_rows", "d", "dtype", "kernel", "flags")]


class T5(C.Structure):
    _fields_ = [("data", C.c_void_p), ("stride", C.c_int64 * 4)]


class T4(C.Structure):
    _fields_ = [("data", C.c_void_p), ("stride", C.c_int64 * 3)]


class Mask(C.Structure):
    _fields_ = [("data", C.c_void_p), ("stride", C.c_int64 * 2)]


class PushReduce(C.Structure):
    _fields_ = [("rank", C.c_int32), ("world", C.c_int32), ("ctas", C.c_int32), ("epoch", C.c_uint32),
                ("count", C.c_int64), ("partial", C.c_void_p), ("counters", C.c_void_p),
                ("staging", C.c_void_p * 8), ("result", C.c_void_p * 8), ("flags", C.c_void_p * 8)]


class Plan(C.Structure):
    _fields_ = [("kernel", C.c_int32), ("block_j", C.c_int32), ("block_k", C.c_int32),
                ("rows_per_cta", C.c_int32), ("stages", C.c_int32), ("db_row_splits", C.c_int32),
                ("bwd_fused", C.c_int32), ("bwd_chunks", C.c_int32), ("fwd_kernel", C.c_int32)]


# name -> (restype, argtypes); one entry per declaration in include/trifast_b200.h
_P = C.POINTER
SIGNATURES = {
    "trifast_version": (C.c_int, []),
    "trifast_status_str": (C.c_char_p, [C.c_int]),
    "trifast_last_cuda_error": (C.c_char_p, []),
    "trifast_copy_blocks": (C.c_int, [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_size_t,
                                      C.c_size_t, C.c_int, C.c_void_p]),
    "trifast_pick_plan": (C.c_int, [_P(Shape), _P(Plan)]),
    "trifast_backward_workspace_bytes": (C.c_size_t, [_P(Shape)]),
    "trifast_forward_workspace_bytes": (C.c_size_t, [_P(Shape)]),
    "trifast_forward": (C.c_int, [_P(Shape), _P(T5), _P(T5), _P(T5), _P(T4), _P(Mask), _P(T5),
                                  C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "trifast_backward": (C.c_int, [_P(Shape), _P(T5), _P(T5), _P(T5), _P(T5), _P(T4), _P(Mask),
                                   _P(T5), C.c_void_p, _P(T5), _P(T5), _P(T5), _P(T4),
                                   C.c_void_p, C.c_size_t, C.c_void_p]),
    "trifast_backward_db": (C.c_int, [_P(Shape), _P(T5), _P(T5), _P(T5), _P(T5), _P(T4), _P(Mask),
                                      _P(T5), C.c_void_p, C.c_void_p,
                                      C.c_void_p, C.c_size_t, C.c_void_p]),
    "trifast_backward_dqkv": (C.c_int, [_P(Shape), _P(T5), _P(T5), _P(T5), _P(T5), _P(T4),
                                        _P(Mask), C.c_void_p, _P(T5), _P(T5), _P(T5),
                                        C.c_void_p, C.c_size_t, C.c_void_p]),
    "trifast_db_finalize": (C.c_int, [_P(Shape), C.c_void_p, _P(T4), C.c_void_p]),
    "trifast_check_device_status": (C.c_int, [C.c_void_p]),
    "trifast_snapshot_device_status": (C.c_int, [C.c_void_p, C.c_void_p]),
    "trifast_db_push_reduce": (C.c_int, [_P(PushReduce), C.c_void_p]),
    "trifast_db_push_reduce_staging_floats": (C.c_size_t, [C.c_int64, C.c_int32]),
    "trifast_debug_wait_probe": (C.c_int, [C.c_uint32, C.c_void_p]),
    "trifast_backward_static_scratch": (C.c_int, [_P(Shape), _P(T5), _P(T5), _P(T5), _P(T5), _P(T4),
                                                  _P(Mask), _P(T5), C.c_void_p, _P(T5), _P(T5),
                                                  _P(T5), _P(T4), C.c_void_p]),
}

_lib = None


def load() -> C.CDLL:
    """Load the library once; raise with build instructions if it is absent."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} not found: build it with `python -m trifast_b200.build` "
                "(needs nvcc; there is no fallback path)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def status_str(rc: int) -> str:
    return load().trifast_status_str(rc).decode()


def check(rc: int, what: str) -> None:
    if rc != 0:
        detail = f", {load().trifast_last_cuda_error().decode()}" if rc == -9 else ""   # TRIFAST_ERR_LAUNCH
        raise RuntimeError(f"{what}: {status_str(rc)} (status {rc}{detail})")


# Per-device pinned host word that mirrors the device status word (see
# trifast_snapshot_device_status in the header): the library copies the status
# into it after every operator call, and the next call looks at it first.
_status_words: dict = {}


def _status_word(device) -> torch.Tensor:
    idx = torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    w = _status_words.get(idx)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32).pin_memory()
        _status_words[idx] = w
    return w


def raise_if_device_gave_up(device) -> None:
    """First thing in every operator call.  If an earlier kernel on this device gave
    up on one of its bounded waits, its outputs (and those of every launch since) were
    never written: read and clear the status and raise, instead of returning
    uninitialised memory.  Costs one host-memory read when nothing is wrong."""
    w = _status_word(device)
    if int(w[0]) == 0:
        return
    w.zero_()
    with torch.cuda.device(device):
        load().trifast_check_device_status(
            C.c_void_p(torch.cuda.current_stream(device).cuda_stream))
    raise RuntimeError(
        "trifast_b200: " + status_str(-11) + " in an earlier call on this device; the results "
        "of that call and of the calls after it are invalid (status cleared, retry is possible)")


def snapshot_status(device, stream: C.c_void_p) -> None:
    """Last thing in every operator call: enqueue the copy of the status word."""
    with torch.cuda.device(device):
        check(load().trifast_snapshot_device_status(C.c_void_p(_status_word(device).data_ptr()),
                                                    stream), "trifast_snapshot_device_status")


def kernel_choice() -> int:
    """Debug override of the tile heuristic: TRIFAST_B200_KERNEL=simt|tcgen05|auto."""
    return _KERNEL_ENV[os.environ.get("TRIFAST_B200_KERNEL", "").lower()]


def flags_choice() -> int:
    """Debug override: TRIFAST_B200_FLAGS=<int>, an OR of the header's trifast_flags."""
    return int(os.environ.get("TRIFAST_B200_FLAGS", "0") or 0)


def make_shape(batch, heads, n, n_rows, d, dtype, kernel=None, flags=None) -> Shape:
    if dtype not in DTYPE_CODE:
        raise TypeError(f"unsupported dtype {dtype}; expected float32, bfloat16 or float16")
    return Shape(batch, heads, n, n_rows, d, DTYPE_CODE[dtype],
                 kernel_choice() if kernel is None else kernel,
                 flags_choice() if flags is None else flags)


def t5(t: torch.Tensor) -> T5:
    assert t.dim() == 5 and t.stride(4) == 1
    return T5(t.data_ptr(), (C.c_int64 * 4)(*t.stride()[:4]))


def t4(t: torch.Tensor) -> T4:
    assert t.dim() == 4 and t.stride(3) == 1
    return T4(t.data_ptr(), (C.c_int64 * 3)(*t.stride()[:3]))


def mask_view(m: torch.Tensor) -> Mask:
    assert m.dim() == 3 and m.stride(2) == 1 and m.element_size() == 1
    return Mask(m.data_ptr(), (C.c_int64 * 2)(*m.stride()[:2]))


def pick_plan(batch, heads, n, n_rows, d, dtype, kernel=KERNEL_AUTO) -> dict:
    """Host-only: the tile plan the heuristic chooses for a problem."""
    plan = Plan()
    shp = make_shape(batch, heads, n, n_rows, d, dtype, kernel)
    check(load().trifast_pick_plan(C.byref(shp), C.byref(plan)), "trifast_pick_plan")
    return {f: getattr(plan, f) for f, _ in Plan._fields_ if f != "reserved"}
