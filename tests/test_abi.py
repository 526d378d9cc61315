"""CPU tier: the C-ABI library loads, exports every symbol the header declares,
validates arguments before touching a device, and the tile heuristic is a pure
host function."""

import ctypes as C
import os
import re

import pytest
import torch

from trifast_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "trifast_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(trifast_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    lib = _lib.load()
    names = header_symbols()
    assert len(names) >= 10
    for name in names:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert set(_lib.SIGNATURES) == set(names)


def test_version_and_status_strings():
    lib = _lib.load()
    assert lib.trifast_version() >= 100
    assert _lib.status_str(0) == "ok"
    for rc in range(-12, 0):
        assert _lib.status_str(rc) != "unknown status"
    assert _lib.status_str(-99) == "unknown status"


@pytest.mark.parametrize("n,h,d,dtype,kernel", [
    (1024, 4, 32, torch.bfloat16, _lib.KERNEL_TCGEN05),
    (2048, 4, 32, torch.bfloat16, _lib.KERNEL_TCGEN05),
    (1024, 8, 64, torch.float16, _lib.KERNEL_TCGEN05),
    (256, 4, 32, torch.bfloat16, _lib.KERNEL_TCGEN05),
    (32, 4, 32, torch.float32, _lib.KERNEL_SIMT),     # fp32 always on CUDA cores
    (1024, 4, 32, torch.float32, _lib.KERNEL_SIMT),
    (191, 4, 32, torch.bfloat16, _lib.KERNEL_TCGEN05),  # ragged n: padded bias copy in the workspace
    (100, 4, 32, torch.bfloat16, _lib.KERNEL_TCGEN05),  # one tile, partly filled
    (64, 1, 64, torch.bfloat16, _lib.KERNEL_TCGEN05),   # smallest n on tensor cores
    (63, 1, 64, torch.bfloat16, _lib.KERNEL_SIMT),      # a tile less than a quarter full
    (256, 4, 128, torch.bfloat16, _lib.KERNEL_SIMT),
    (256, 4, 16, torch.float16, _lib.KERNEL_TCGEN05),  # 32-byte rows
    (48, 4, 16, torch.float16, _lib.KERNEL_SIMT),
])
def test_heuristic_table(n, h, d, dtype, kernel):
    plan = _lib.pick_plan(1, h, n, n, d, dtype)
    assert plan["kernel"] == kernel
    assert plan["db_row_splits"] >= 1
    if kernel == _lib.KERNEL_TCGEN05:
        assert (plan["block_j"], plan["block_k"]) == (128, 128)


def test_forward_workspace_sizes():
    """Tensor-core plan: the live key-tile range of every row (4 bytes per row, 256-byte
    granules); ragged n adds the padded bias copy, packed masks and row flags.  CUDA-core
    plan: none."""
    lib = _lib.load()
    size = lambda n, dtype=torch.bfloat16: lib.trifast_forward_workspace_bytes(
        C.byref(_lib.make_shape(1, 4, n, n, 32, dtype)))
    assert size(1024) == 4096 and size(1000) == 4096          # 4 bytes x 1000 rows -> 4096
    assert size(1001) > 4 * 1001 * 1008 * 2 and size(191) > 4 * 191 * 192 * 2   # + bias copy
    assert size(48) == 0                                      # below a quarter tile: CUDA cores
    assert size(1001, torch.float32) == 0


def test_heuristic_rejects_impossible_forced_kernel():
    shp = _lib.make_shape(1, 4, 48, 48, 32, torch.bfloat16, _lib.KERNEL_TCGEN05)
    plan = _lib.Plan()
    assert _lib.load().trifast_pick_plan(C.byref(shp), C.byref(plan)) == -10


def test_db_splits_cover_small_problems():
    assert _lib.pick_plan(1, 1, 64, 64, 32, torch.float32)["db_row_splits"] > 1
    assert _lib.pick_plan(1, 4, 1024, 1024, 32, torch.float32)["db_row_splits"] == 1


@pytest.mark.parametrize("kw,rc", [
    (dict(n=0), -2), (dict(n_rows=65), -2), (dict(d=48), -3), (dict(dtype=7), -4),
    (dict(batch=0), -2), (dict(kernel=9), -10),
])
def test_shape_validation(kw, rc):
    f = dict(batch=1, heads=2, n=64, n_rows=64, d=32, dtype=1, kernel=0, flags=0)
    f.update(kw)
    shp = _lib.Shape(**f)
    plan = _lib.Plan()
    assert _lib.load().trifast_pick_plan(C.byref(shp), C.byref(plan)) == rc
    assert _lib.load().trifast_backward_workspace_bytes(C.byref(shp)) == 0


def _fake5(ptr=0x1000, stride=(64 * 64 * 32 * 2, 64 * 64 * 32, 64 * 32, 32)):
    return _lib.T5(ptr, (C.c_int64 * 4)(*stride))


def test_forward_argument_validation_needs_no_device():
    lib = _lib.load()
    shp = _lib.make_shape(1, 2, 64, 64, 32, torch.bfloat16, 0)
    t, bias = _fake5(), _lib.T4(0x1000, (C.c_int64 * 3)(2 * 64 * 64, 64 * 64, 64))
    mask = _lib.Mask(0x1000, (C.c_int64 * 2)(64 * 64, 64))
    lse = C.c_void_p(0x1000)

    def call(q=t, k=t, v=t, b=bias, m=mask, o=t, l=lse):
        return lib.trifast_forward(C.byref(shp), C.byref(q), C.byref(k), C.byref(v), C.byref(b),
                                   C.byref(m), C.byref(o), l, None, 0, None)

    assert call(q=_fake5(ptr=0)) == -1                       # NULL data
    assert call(k=_fake5(ptr=0x1008)) == -6                  # misaligned
    assert call(v=_fake5(stride=(1, 1, 1, 31))) == -5        # stride not 16-byte multiple
    assert call(v=_fake5(stride=(0, 0, 0, 16))) == -5        # rows overlap
    assert call(b=_lib.T4(0x1000, (C.c_int64 * 3)(0, 0, 8))) == -5
    assert call(m=_lib.Mask(0x1000, (C.c_int64 * 2)(0, 8))) == -5
    assert call(l=None) == -1


def test_workspace_size_formula():
    lib = _lib.load()
    shp = _lib.make_shape(1, 4, 1024, 1024, 32, torch.bfloat16)
    ws = lib.trifast_backward_workspace_bytes(C.byref(shp))
    stat = 4 * 1024 * 1024 * 4
    # delta, -lse*log2e, fp32 db (3 x 16 MiB) + transposed 16-bit bias (8 MiB) + row
    # flags and packed masks + one fp32 db partial per row split
    splits = _lib.pick_plan(1, 4, 1024, 1024, 32, torch.bfloat16)["db_row_splits"]
    want = (3 + splits) * stat + stat // 2
    assert want <= ws < want + (1 << 20)
    shard = _lib.make_shape(1, 4, 1024, 128, 32, torch.bfloat16)
    assert lib.trifast_backward_workspace_bytes(C.byref(shard)) < ws


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libtrifast_b200.so")
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.load()


def test_cpu_tensors_are_rejected():
    from trifast_b200 import triangle_attention
    from trifast_b200.utils import gen_tensors
    q, k, v, b, m = gen_tensors(16, 16, 1, False, "cpu", torch.float32)
    with pytest.raises(Exception):
        triangle_attention(q, k, v, b, m)


# ---------------------------------------------------------------- debug flags, plan.bwd_fused
@pytest.mark.parametrize("n,d,dtype,flags,fused,chunks", [
    (1024, 32, torch.bfloat16, 0, 1, 1),    # 8 query tiles x 32 columns of dQ = 256: one chunk
    (1025, 32, torch.bfloat16, 0, 1, 2),    # a ninth tile: the row is walked in two query chunks
    (2048, 32, torch.bfloat16, 0, 1, 2),
    (4096, 32, torch.bfloat16, 0, 1, 4),
    (384, 64, torch.float16, 0, 1, 1),      # 3 x 64 columns next to dK, dV of 64 each
    (512, 64, torch.float16, 0, 1, 2),
    (1024, 64, torch.float16, 0, 1, 3),
    (1024, 32, torch.bfloat16, _lib.FLAG_SPLIT_BWD, 0, 0),   # forced two-kernel backward
    (256, 32, torch.float32, 0, 0, 0),      # CUDA-core path has no one-pass kernel
])
def test_fused_backward_choice(n, d, dtype, flags, fused, chunks):
    plan = _lib.Plan()
    shp = _lib.make_shape(1, 4, n, n, d, dtype, flags=flags)
    assert _lib.load().trifast_pick_plan(C.byref(shp), C.byref(plan)) == 0
    assert (plan.bwd_fused, plan.bwd_chunks) == (fused, chunks)


def test_chunked_backward_adds_its_scratch_to_the_workspace():
    """Rows walked in several query chunks keep fp32 dK / dV partials per CTA:
    160 CTAs x ceil(n / 128) x 128 keys x 2 d floats."""
    lib = _lib.load()
    one = _lib.make_shape(1, 4, 2048, 64, 32, torch.bfloat16, flags=_lib.FLAG_SPLIT_BWD)
    two = _lib.make_shape(1, 4, 2048, 64, 32, torch.bfloat16)
    extra = lib.trifast_backward_workspace_bytes(C.byref(two)) - lib.trifast_backward_workspace_bytes(C.byref(one))
    assert extra == 160 * 2048 * 2 * 32 * 4


def test_unknown_flag_bits_are_rejected():
    shp = _lib.make_shape(1, 4, 256, 256, 32, torch.bfloat16, flags=4)
    assert _lib.load().trifast_pick_plan(C.byref(shp), C.byref(_lib.Plan())) == -10


# ---------------------------------------------------------------- argument checks without a device
def test_broadcast_strides_are_rejected_before_any_launch():
    """A stride of 0 on a dimension with more than one entry (an expanded view) cannot be
    described to TMA: the library names it a stride error instead of failing at launch."""
    lib = _lib.load()
    shp = _lib.make_shape(1, 2, 64, 64, 32, torch.bfloat16, 0)
    t, bias = _fake5(), _lib.T4(0x1000, (C.c_int64 * 3)(2 * 64 * 64, 64 * 64, 64))
    mask = _lib.Mask(0x1000, (C.c_int64 * 2)(64 * 64, 64))
    expanded_heads = _fake5(stride=(64 * 64 * 32, 0, 64 * 32, 32))
    rc = lib.trifast_forward(C.byref(shp), C.byref(expanded_heads), C.byref(t), C.byref(t),
                             C.byref(bias), C.byref(mask), C.byref(t), C.c_void_p(0x1000), None, 0,
                             None)
    assert rc == -5
    # extent-1 dimensions may carry any stride, 0 included (batch = 1 here)
    ok_batch = _fake5(stride=(0, 64 * 64 * 32, 64 * 32, 32))
    rc = lib.trifast_forward(C.byref(shp), C.byref(ok_batch), C.byref(t), C.byref(t), C.byref(bias),
                             C.byref(mask), C.byref(_fake5(ptr=0)), C.c_void_p(0x1000), None, 0, None)
    assert rc == -1                                  # got past q; o is the NULL one


def test_backward_checks_outputs_before_anything_is_enqueued():
    lib = _lib.load()
    shp = _lib.make_shape(1, 2, 64, 64, 32, torch.bfloat16, 0)
    t, bias = _fake5(), _lib.T4(0x1000, (C.c_int64 * 3)(2 * 64 * 64, 64 * 64, 64))
    mask = _lib.Mask(0x1000, (C.c_int64 * 2)(64 * 64, 64))

    def call(dq=t, dk=t, dv=t, db=bias):
        return lib.trifast_backward(C.byref(shp), C.byref(t), C.byref(t), C.byref(t), C.byref(t),
                                    C.byref(bias), C.byref(mask), C.byref(t), C.c_void_p(0x1000),
                                    C.byref(dq), C.byref(dk), C.byref(dv), C.byref(db),
                                    C.c_void_p(0x1000), C.c_size_t(1 << 30), None)

    assert call(dq=_fake5(ptr=0)) == -1
    assert call(dk=_fake5(ptr=0x1004)) == -6
    assert call(dv=_fake5(stride=(1, 1, 1, 31))) == -5
    assert call(db=_lib.T4(0, (C.c_int64 * 3)(2 * 64 * 64, 64 * 64, 64))) == -1


def test_probe_and_snapshot_validate_arguments():
    lib = _lib.load()
    assert lib.trifast_debug_wait_probe(0, None) == -12
    assert lib.trifast_debug_wait_probe(100001, None) == -12
    assert lib.trifast_snapshot_device_status(None, None) == -1


def _meta(shape, dtype=torch.bfloat16, device="meta"):
    return torch.empty(shape, dtype=dtype, device=device)


def test_python_layer_rejects_mixed_devices_and_bad_saved_tensors():
    """Host pointers (or another GPU's) must never reach a kernel: every tensor has to
    live on q's device, and the backward's dO, o and lse must match q."""
    from trifast_b200.torch import _check_inputs, _check_saved
    s5, s4, s3 = (1, 2, 16, 16, 32), (1, 2, 16, 16), (1, 16, 16)
    q, k, v, b = _meta(s5), _meta(s5), _meta(s5), _meta(s4)
    m = _meta(s3, torch.bool)
    for bad in ("k", "v", "bias", "mask"):
        args = dict(k=k, v=v, bias=b, mask=m)
        args[bad] = torch.empty(args[bad].shape, dtype=args[bad].dtype, device="cpu")
        with pytest.raises(ValueError, match="same CUDA device"):
            _check_inputs(q, args["k"], args["v"], args["bias"], args["mask"])
    with pytest.raises(RuntimeError, match="no CPU path"):
        _check_inputs(q, k, v, b, m)                 # consistent, but not CUDA
    lse = _meta((1, 2, 16, 16), torch.float32)
    _check_saved(_meta(s5), q, _meta(s5), lse)
    with pytest.raises(ValueError, match="do must be"):
        _check_saved(_meta((1, 2, 16, 16, 16)), q, _meta(s5), lse)
    with pytest.raises(ValueError, match="o must be"):
        _check_saved(_meta(s5), q, _meta(s5, torch.float16), lse)
    with pytest.raises(ValueError, match="lse must be float32"):
        _check_saved(_meta(s5), q, _meta(s5), _meta((1, 2, 16, 16), torch.bfloat16))
    with pytest.raises(ValueError, match="lse is on"):
        _check_saved(_meta(s5), q, _meta(s5), torch.empty((1, 2, 16, 16), dtype=torch.float32))


def test_expanded_views_are_materialised_by_the_python_layer():
    from trifast_b200.torch import _row_vector_ok
    base = torch.zeros(1, 1, 16, 16, 32, dtype=torch.bfloat16)
    assert _row_vector_ok(base)
    assert not _row_vector_ok(base.expand(1, 4, 16, 16, 32))     # stride 0 over 4 heads
    assert _row_vector_ok(base.expand(1, 1, 16, 16, 32))


# ---------------------------------------------------------------- static-scratch capacity
@pytest.mark.parametrize("h,d,dtype,n_ok,n_too_large", [
    (4, 32, torch.bfloat16, 224, 256),    # tensor-core plan: the row-split db partials dominate
    (4, 64, torch.float16, 224, 256),
    (4, 16, torch.bfloat16, 224, 256),
    (1, 32, torch.bfloat16, 448, 480),
    (4, 128, torch.bfloat16, 576, 608),   # CUDA-core plan
    (4, 32, torch.float32, 576, 608),
])
def test_static_scratch_capacity(h, d, dtype, n_ok, n_too_large):
    """trifast_backward_static_scratch serves problems whose backward workspace fits its
    16 MiB array; these are the largest sizes on either side of that line."""
    lib = _lib.load()
    ok = _lib.make_shape(1, h, n_ok, n_ok, d, dtype)
    big = _lib.make_shape(1, h, n_too_large, n_too_large, d, dtype)
    assert 0 < lib.trifast_backward_workspace_bytes(C.byref(ok)) <= _lib.STATIC_SCRATCH_BYTES
    assert lib.trifast_backward_workspace_bytes(C.byref(big)) > _lib.STATIC_SCRATCH_BYTES


# ---------------------------------------------------------------- push reduce (host-side checks)
def test_push_reduce_staging_size_and_argument_checks():
    lib = _lib.load()
    f = lib.trifast_db_push_reduce_staging_floats
    assert f(16, 2) == 16 and f(17, 2) == 24          # slices rounded up to 4 floats
    assert f(4 * 1024 * 1024, 8) == 4 * 1024 * 1024
    assert f(0, 2) == 0 and f(16, 9) == 0 and f(16, 0) == 0
    a = _lib.PushReduce()
    a.rank, a.world, a.ctas, a.epoch, a.count = 0, 2, 8, 1, 1024
    a.partial, a.counters = 0x1000, 0x2000
    for r in range(2):
        a.staging[r], a.result[r], a.flags[r] = 0x10000, 0x20000, 0x30000
    call = lambda: lib.trifast_db_push_reduce(C.byref(a), None)
    a.epoch = 0
    assert call() == -2                               # epochs start at 1
    a.epoch, a.world = 1, 9
    assert call() == -2
    a.world, a.rank = 2, 2
    assert call() == -2
    a.rank, a.partial = 0, 0
    assert call() == -1
    a.partial = 0x1004
    assert call() == -6
    a.partial, a.flags[1] = 0x1000, 0
    assert call() == -1
    assert lib.trifast_db_push_reduce(None, None) == -1


def test_extent_one_dimensions_get_canonical_strides():
    """`contiguous()` keeps whatever strides extent-1 dimensions came with; the pointers and
    strides handed to the library are the canonical ones."""
    import torch
    from trifast_b200.torch import _prep4, _prep5, _prep_mask
    b = torch.randn(1, 1, 1, 4).permute(0, 3, 1, 2)            # (1, 4, 1, 1), last stride 4
    assert b.stride(-1) != 1 and b.is_contiguous()
    pb = _prep4(b)
    assert pb.stride() == (4, 1, 1, 1) and torch.equal(pb, b)
    q = torch.randn(1, 1, 1, 3, 16).permute(0, 3, 1, 2, 4)      # extent-1 strides of 48 elements
    assert _prep5(q).data_ptr() == q.data_ptr()                 # 16-byte multiples: passed as is
    m = torch.zeros(2, 1, 1, dtype=torch.bool).as_strided((2, 1, 1), (1, 7, 7))
    assert _prep_mask(m).stride() == (1, 1, 1)


def test_copy_blocks_argument_checks():
    lib = _lib.load()
    f = lib.trifast_copy_blocks
    assert f(None, 64, 0x1000, 64, 64, 2, 0, None) == -1            # NULL
    assert f(0x1000, 32, 0x2000, 64, 64, 2, 0, None) == -5          # blocks would overlap
    assert f(0x1000, 64, 0x2000, 64, 0, 2, 0, None) == 0            # nothing to copy


def test_share_gpu_flag_carries_the_number_of_free_sms():
    lib = _lib.load()
    plan = _lib.Plan()
    ok = lambda flags: lib.trifast_pick_plan(
        C.byref(_lib.make_shape(1, 4, 256, 256, 32, torch.bfloat16, flags=flags)), C.byref(plan))
    assert _lib.share_gpu_flags() == _lib.FLAG_SHARE_GPU
    assert _lib.share_gpu_flags(1) == _lib.FLAG_SHARE_GPU | 0x100
    assert ok(_lib.share_gpu_flags(1)) == 0 and ok(_lib.share_gpu_flags(20)) == 0
    assert ok(0x100) == -10                       # a count without the flag
    assert ok(0x10000) == -10                     # unknown bit
    with pytest.raises(ValueError):
        _lib.share_gpu_flags(256)


def test_head_dim_128_plan_and_forward_workspace():
    """d = 128: tensor-core tiles exist for the forward only.  plan.kernel (the backward's
    family) is CUDA cores, plan.fwd_kernel tensor cores; the forward workspace always holds
    the prepared row flags and packed masks (4 words per 128 keys and row) besides the ranges,
    and the padded bias copy only for ragged n; asking for CUDA cores gives them throughout."""
    lib = _lib.load()
    plan = _lib.pick_plan(1, 4, 1024, 1024, 128, torch.bfloat16)
    assert (plan["kernel"], plan["fwd_kernel"], plan["bwd_fused"]) == (_lib.KERNEL_SIMT, _lib.KERNEL_TCGEN05, 0)
    assert _lib.pick_plan(1, 4, 1024, 1024, 128, torch.bfloat16, _lib.KERNEL_SIMT)["fwd_kernel"] == _lib.KERNEL_SIMT
    assert _lib.pick_plan(1, 4, 1024, 1024, 128, torch.float32)["fwd_kernel"] == _lib.KERNEL_SIMT
    assert _lib.pick_plan(1, 4, 48, 48, 128, torch.bfloat16)["fwd_kernel"] == _lib.KERNEL_SIMT
    size = lambda n: lib.trifast_forward_workspace_bytes(C.byref(_lib.make_shape(1, 4, n, n, 128, torch.bfloat16)))
    assert size(1024) == 4096 + 1024 + 1024 * 32 * 4                  # ranges, row flags, packed masks
    assert size(1000) < 4 * 1000 * 1000 * 2 < size(1001)              # the bias copy only when ragged
    # the backward of d = 128 has no tensor-core family to force
    shp = _lib.make_shape(1, 4, 256, 256, 128, torch.bfloat16, _lib.KERNEL_TCGEN05)
    assert lib.trifast_backward_workspace_bytes(C.byref(shp)) > 0     # sized for the CUDA-core kernels


def test_host_pipeline_block_bounds():
    from trifast_b200.host import block_bounds
    for rows, chunk in ((1024, 64), (128, 32), (100, 64), (1000, 64), (50, 8), (7, 64), (200, 64), (129, 64)):
        b = block_bounds(rows, chunk)
        sizes = [b[i + 1] - b[i] for i in range(len(b) - 1)]
        assert b[0] == 0 and b[-1] == rows and all(0 < x <= chunk for x in sizes), (rows, chunk, b)
    assert [y - x for x, y in zip(block_bounds(1024, 64), block_bounds(1024, 64)[1:])][:3] == [16, 32, 64]
