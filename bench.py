"""Benchmark of the triangle-attention hot path (forward + backward).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One step = one forward + backward of the workload (default: the headline shape
n = 1024, h = 4, d = 32, bf16, batch 1, nothing masked) on synthetic, seeded
inputs.  With N > 1 (launched under torchrun, one rank per GPU) the pair rows of
that one problem are sharded over the ranks (strong scaling) and the step
includes the NCCL all-reduce of the bias gradient.  Rank 0 prints ONE JSON line.

Keys beyond the usual ones:
  value / ms_per_step : kernels only, inputs resident in HBM, CUDA events, max over ranks
  e2e                 : the same step through the package's host-resident API with pinned-host
                        inputs copied in and o, dq, dk, dv, db copied out every step
  public_api          : the same step through trifast_b200.triangle_attention(...) and
                        o.backward(dO) (the row-sharded operator at N > 1): allocator, operator
                        dispatch and autograd included
  roofline            : the dominant single kernel against the measured bf16 tensor peak,
                        with the FLOP count used
  phases_ms           : forward / db / dq+dk+dv phase times of this rank (CUDA events); at
                        N > 1 also the exposed part of the db all-reduce
  parity_ok           : N > 1 only: rank 0 repeats the whole problem alone and compares o
                        (bit for bit on its rows, checksum over all ranks) and the reduced db
  cpu_baseline        : the PyTorch CPU restatement on a bounded row sample (N = 1)

``--impl reference`` times the reference algorithm's CPU implementation (the
PyTorch restatement under oracle/, all host threads) on a bounded row sample of
the same workload and prints the same line with "impl": "reference".
"""

from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from trifast_b200.configs import WORKLOADS, make_inputs  # noqa: E402

METRIC = "triangle_attention_fwd_bwd_tflops"


def flops_fwd(w, rows=None):
    rows = w.n if rows is None else rows
    return 4.0 * w.batch * w.h * rows * w.n * w.n * w.d


def flops_step(w, rows=None):
    return flops_fwd(w, rows) * (3.5 if w.backward else 1.0)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"burst": p["bf16_tflops"], "sustained": p["bf16_tflops_sustained"],
                "hbm_gbs": p["hbm_gbs"], "source": "measured"}
    return {"burst": 1590.0, "sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi during the timed region."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc = index, None
        self.thread, self.samples, self.halt = None, [], None

    def _nvml_loop(self, pynvml, handle):
        names = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
                 0x4: "sw_power_cap"}
        mx = pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM)
        while not self.halt.is_set():
            sm = pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)
            try:
                bits = pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle)
            except AttributeError:
                bits = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
            self.samples.append((sm, mx, [n for b, n in names.items() if bits & b]))
            self.halt.wait(0.002)

    def start(self):
        # in-process NVML reads every 2 ms (a timed region can be a few tens of ms long);
        # the nvidia-smi loop is the fallback.  Both only read.
        try:
            import threading
            import pynvml
            pynvml.nvmlInit()
            handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.halt = threading.Event()
            self.thread = threading.Thread(target=self._nvml_loop, args=(pynvml, handle), daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.thread is not None:
            self.halt.set()
            self.thread.join(timeout=2)
            sm = sorted(x[0] for x in self.samples)
            reasons = sorted({r for x in self.samples for r in x[2]})
            return {"sm_mhz": sm[len(sm) // 2] if sm else None,
                    "sm_max_mhz": self.samples[0][1] if self.samples else None,
                    "reasons": reasons, "samples": len(sm), "source": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        self.proc.terminate()
        try:
            out = self.proc.communicate(timeout=5)[0]
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


# ---------------------------------------------------------------------------
# reference arm / CPU baseline: the PyTorch CPU restatement on a row sample
# ---------------------------------------------------------------------------

def cpu_sample_step(w, rows, seed=0):
    """Returns a callable running fwd(+bwd) of `rows` pair rows on the CPU."""
    from oracle import triangle_oracle as orc
    q, k, v, b, m, do = make_inputs(w, seed=seed, sample_rows=rows)
    # fp32 compute on fp32 copies of the rounded inputs: the reference's test oracle
    # runs in fp32 (tests/unit/test_trifast.py:50 of the reference).
    q, k, v, b, do = (t.float() for t in (q, k, v, b, do))

    def step():
        orc.forward_backward_chunked(q, k, v, b, m, do=do if w.backward else None,
                                     rows_per_chunk=4)
    return step


def cpu_rows_for_budget(w, seconds):
    """Rows whose fwd+bwd should take about `seconds` on this host (>= 4)."""
    probe = 4
    step = cpu_sample_step(w, probe)
    step()
    t0 = time.perf_counter()
    step()
    per_row = (time.perf_counter() - t0) / probe
    return int(max(4, min(w.n, (seconds / max(per_row, 1e-6)) // 4 * 4)))


def run_reference(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # every host core, also under torchrun (which exports OMP_NUM_THREADS=1)
    torch.set_num_threads(os.cpu_count() or 1)
    cores = torch.get_num_threads()
    rows = cpu_rows_for_budget(w, 4.0)
    step = cpu_sample_step(w, rows)
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    value = flops_step(w, rows) / dt / 1e12
    sample = f"{rows} of {w.n} pair rows per step, fp32 PyTorch CPU, time scaled by rows"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt * 1e3 * w.n / rows, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(w, args.gpus),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": sample, "host_cpus": os.cpu_count()},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(w, gpus):
    return {"workload": w.name, "n": w.n, "heads": w.h, "head_dim": w.d, "batch": w.batch,
            "mask": w.mask, "backward": w.backward,
            "parallelism": f"row-shard x{gpus}" if gpus > 1 else "single GPU",
            "l2": "inputs larger than L2 (no flush)"}


# ---------------------------------------------------------------------------
# native arm
# ---------------------------------------------------------------------------

class DirectStep:
    """fwd (+bwd) through the C ABI with every buffer preallocated."""

    def __init__(self, w, q, k, v, b, m, do, group_size, db_reduce="nccl", push_ctas=4, free_sms=8):
        from trifast_b200 import _lib
        self.lib, self._lib = _lib.load(), _lib
        self.w, self.world = w, group_size
        bs, h, rows, n, d = q.shape
        dev = q.device
        self.t = dict(q=q, k=k, v=v, b=b, do=do)
        self.m8 = m.view(torch.uint8)
        self.o = torch.empty_like(q)
        self.lse = torch.empty((bs, h, rows, n), dtype=torch.float32, device=dev)
        self.shape = _lib.make_shape(bs, h, n, rows, d, q.dtype,
                                     flags=_lib.share_gpu_flags(free_sms) if group_size > 1 else None)
        self.fws_bytes = self.lib.trifast_forward_workspace_bytes(C.byref(self.shape))
        self.fws = torch.empty(self.fws_bytes, dtype=torch.uint8, device=dev) if self.fws_bytes else None
        if w.backward:
            self.dq, self.dk, self.dv = (torch.empty_like(q) for _ in range(3))
            self.db = torch.empty_like(b)
            self.db32 = torch.empty(b.shape, dtype=torch.float32, device=dev)
            nbytes = self.lib.trifast_backward_workspace_bytes(C.byref(self.shape))
            self.ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        self.stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        L = _lib
        self.a = {k_: L.t5(x) for k_, x in dict(q=q, k=k, v=v, do=do, o=self.o).items()}
        self.ab, self.am = L.t4(b), L.mask_view(self.m8)
        if w.backward:
            self.a.update(dq=L.t5(self.dq), dk=L.t5(self.dk), dv=L.t5(self.dv))
            self.adb = L.t4(self.db)
        plan = L.pick_plan(bs, h, n, rows, d, q.dtype)
        self.plan = plan
        # launches per step: forward 1 (+ the live key-tile ranges of the rows on the tensor-core
        # path, + the padded bias copy for n % 8 != 0); backward: row flags + packed mask, bias
        # transpose (tensor-core path only), delta, db, split reduce (if split), dq, dk/dv, cast
        self.launches = 1 + ((1 + (1 if n % 8 else 0)) if plan["fwd_kernel"] == 2 else 0)
        if w.backward:
            self.launches += 1 + (1 if plan["kernel"] == 2 else 0) + 1 + 1 + \
                (1 if plan["db_row_splits"] > 1 else 0) + (1 if plan["bwd_fused"] else 2) + 1
        self.exposed = None   # (event after dq/dk/dv, event after the all-reduce wait)
        self.reducer = None
        if w.backward and group_size > 1 and db_reduce == "push":
            from trifast_b200.dist import PushReducer
            self.reducer = PushReducer(self.db32.numel(), dev, ctas=push_ctas)

    def forward(self):
        a, B = self.a, C.byref
        rc = self.lib.trifast_forward(B(self.shape), B(a["q"]), B(a["k"]), B(a["v"]), B(self.ab),
                                      B(self.am), B(a["o"]), C.c_void_p(self.lse.data_ptr()),
                                      C.c_void_p(self.fws.data_ptr() if self.fws is not None else None),
                                      C.c_size_t(self.fws_bytes), self.stream)
        self._lib.check(rc, "trifast_forward")

    def backward_db(self):
        a, B = self.a, C.byref
        rc = self.lib.trifast_backward_db(
            B(self.shape), B(a["do"]), B(a["q"]), B(a["k"]), B(a["v"]), B(self.ab), B(self.am),
            B(a["o"]), C.c_void_p(self.lse.data_ptr()), C.c_void_p(self.db32.data_ptr()),
            C.c_void_p(self.ws.data_ptr()), C.c_size_t(self.ws.numel()), self.stream)
        self._lib.check(rc, "trifast_backward_db")

    def backward_dqkv(self):
        a, B = self.a, C.byref
        rc = self.lib.trifast_backward_dqkv(
            B(self.shape), B(a["do"]), B(a["q"]), B(a["k"]), B(a["v"]), B(self.ab), B(self.am),
            C.c_void_p(self.lse.data_ptr()), B(a["dq"]), B(a["dk"]), B(a["dv"]),
            C.c_void_p(self.ws.data_ptr()), C.c_size_t(self.ws.numel()), self.stream)
        self._lib.check(rc, "trifast_backward_dqkv")

    def finalize(self, src=None):
        src = self.db32 if src is None else src
        rc = self.lib.trifast_db_finalize(C.byref(self.shape), C.c_void_p(src.data_ptr()),
                                          C.byref(self.adb), self.stream)
        self._lib.check(rc, "trifast_db_finalize")

    def step(self):
        import torch.distributed as dist
        self.forward()
        if not self.w.backward:
            return
        self.backward_db()
        work, summed = None, None
        if self.world > 1:
            if self.reducer is not None:
                summed = self.reducer.reduce(self.db32)
            else:
                work = dist.all_reduce(self.db32, async_op=True)
        self.backward_dqkv()
        if self.world > 1:
            if self.exposed is not None:
                self.exposed[0].record()
            if work is not None:
                work.wait()
            else:
                self.reducer.join()
            if self.exposed is not None:
                self.exposed[1].record()
        self.finalize(summed)


def time_events(fn, iters):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def time_events_each(fn, iters):
    """Per-iteration device times (one event pair per call), for quantiles."""
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
           for _ in range(iters)]
    for e0, e1 in evs:
        e0.record()
        fn()
        e1.record()
    torch.cuda.synchronize()
    return sorted(e0.elapsed_time(e1) for e0, e1 in evs)


def quantiles(xs):
    pick = lambda f: xs[min(len(xs) - 1, int(f * len(xs)))]
    return {"p10": pick(0.1), "p50": pick(0.5), "p90": pick(0.9)}


def share_policy(world):
    """(NCCL CTA cap, SMs the dq/dk/dv kernel leaves free) for the db all-reduce.  The NCCL
    kernel only runs beside the dq/dk/dv kernel when it finds as many free SMs as it has
    CTAs (measured on 4 GPUs: 2 CTAs on 1 free SM did not start before that kernel ended, 0.67
    of 0.67 ms exposed; 4 CTAs on 1 SM: 0.29 of 0.34 ms), so both numbers are the same; with 8
    the all-reduce (0.2 ms alone) ends well inside the kernel at every N."""
    return 8, 8


def run_native(args, w):
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # the db all-reduce runs beside the dq/dk/dv kernels, which leave SMs free for it: as
        # many as NCCL may use CTAs (see share_policy)
        os.environ.setdefault("NCCL_MAX_CTAS", str(share_policy(world)[0]))
        dist.init_process_group("nccl", device_id=dev)
    from trifast_b200.dist import shard_rows, triangle_attention_row_sharded
    rows = shard_rows(w.n, rank, world)
    if args.rows and world == 1:
        rows = slice(0, min(args.rows, w.n))
    q, k, v, b, m, do = make_inputs(w, seed=0, rows=rows if (world > 1 or args.rows) else None,
                                    device=dev)
    torch.cuda.synchronize()
    free_sms = args.free_sms or share_policy(world)[1]
    if args.db_reduce == "push" and args.push_ctas > free_sms:
        raise SystemExit("--push-ctas must not exceed --free-sms: the exchange kernel's CTAs run at once")
    step = DirectStep(w, q, k, v, b, m, do, world, args.db_reduce, args.push_ctas, free_sms)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- kernels only, inputs resident -------------------------------------------------
    for _ in range(max(args.warmup, 3)):
        step.step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms = time_events(step.step, args.steps)
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t)
    rc = step.lib.trifast_check_device_status(step.stream)
    step._lib.check(rc, "device status after the timed region")

    if args.kernels_only:
        if rank == 0:
            print(json.dumps({"profiling_aid": True, "rows": q.shape[2], "ms_per_step": ms,
                              "plan": step.plan, "clocks": clocks}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- the same step through the public operator (allocations, dispatch, autograd) ----
    from trifast_b200 import triangle_attention
    qa, ka, va, ba = (t.detach().requires_grad_(w.backward) for t in (q, k, v, b))

    def api_step():
        if world > 1:
            o_ = triangle_attention_row_sharded(qa, ka, va, ba, m, db_reduce=args.db_reduce)
        else:
            o_ = triangle_attention(qa, ka, va, ba, m)
        if w.backward:
            o_.backward(do)
            qa.grad = ka.grad = va.grad = ba.grad = None

    for _ in range(3):
        api_step()
    barrier()
    api_ms = time_events(api_step, args.steps)
    barrier()
    if world > 1:
        t = torch.tensor([api_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        api_ms = float(t)

    # ---- N > 1: are the sharded results those of one GPU? -------------------------------
    parity = None
    if world > 1:
        step.step()
        cs = torch.stack([step.o.double().sum(), step.o.double().abs().sum()])
        dist.all_reduce(cs)
        if rank == 0:
            fq, fk, fv, fb, fm, fdo = make_inputs(w, seed=0, device=dev)
            full = DirectStep(w, fq, fk, fv, fb, fm, fdo, 1)
            full.step()
            torch.cuda.synchronize()
            ref = torch.stack([full.o.double().sum(), full.o.double().abs().sum()])
            o_rows_equal = bool(torch.equal(full.o[:, :, rows], step.o))
            sums_equal = bool(torch.allclose(cs, ref, rtol=1e-9, atol=0))
            parity = {"o_rows_bitwise": o_rows_equal, "o_checksum": sums_equal}
            if w.backward:
                num = (step.db.float() - full.db.float()).abs().max()
                den = full.db.float().abs().max()
                parity["db_rel_err"] = float(num / den)
                parity["dq_rows_bitwise"] = bool(torch.equal(full.dq[:, :, rows], step.dq))
            parity["ok"] = o_rows_equal and sums_equal and parity.get("db_rel_err", 0.0) < 1e-2 \
                and parity.get("dq_rows_bitwise", True)
            del full, fq, fk, fv, fb, fm, fdo
        barrier()

    # ---- end to end through the public API with host buffers ---------------------------
    # Pinned host tensors in, pinned host tensors out, through the host-resident entry
    # point of the package (trifast_b200.host): every step copies this rank's q, k, v,
    # dO, mask and the bias to the GPU and o, dq, dk, dv, db back, in blocks of rows
    # that overlap with the kernels.
    from trifast_b200.host import HostPipeline
    host = [t.cpu().pin_memory() for t in (q, k, v, b, m, do)]
    bs_, h_, rows_, n_, d_ = q.shape
    # blocks small enough that a shard still has several of them in flight
    chunk = max(8, min(args.e2e_chunk_rows, (rows_ + 3) // 4))
    pipe = HostPipeline(bs_, h_, n_, d_, q.dtype, dev, rows=rows_, chunk_rows=chunk,
                        backward=w.backward)
    outs_host = None
    group = dist.group.WORLD if world > 1 else None

    def e2e_step():
        nonlocal outs_host
        hq, hk, hv, hb, hm, hdo = host
        outs_host = pipe.run(hq, hk, hv, hb, hm, do=hdo if w.backward else None, out=outs_host,
                             group=group)

    e2e_iters = max(2, min(args.steps, 5))
    e2e_step()
    e2e_step()
    barrier()
    e2e_ms = time_events(e2e_step, e2e_iters)
    barrier()
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t)
    h2d = sum(t.numel() * t.element_size() for t in host)
    d2h = sum(t.numel() * t.element_size() for t in outs_host.values())
    if world > 1:   # bytes moved by the whole job, not by rank 0
        t = torch.tensor([h2d, d2h], device=dev, dtype=torch.float64)
        dist.all_reduce(t)
        h2d, d2h = int(t[0]), int(t[1])
    del host, outs_host, pipe
    total_flops = flops_step(w)

    # ---- per-phase timing (every N), roofline and the CPU baseline (single GPU only) ---
    phases, roofline, cpu = None, None, None
    peaks = measured_peaks()
    step_q = None
    phases = {"forward": time_events(step.forward, args.steps)}
    if w.backward:
        phases["backward_db"] = time_events(step.backward_db, args.steps)
        phases["backward_dqkv"] = time_events(step.backward_dqkv, args.steps)
        phases["db_finalize"] = time_events(step.finalize, args.steps)
    if world > 1 and w.backward:
        # the part of the db all-reduce that the dq/dk/dv kernels do not hide: device time
        # between the end of those kernels and the end of the wait, and the collective alone
        step.exposed = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        exp = []
        for _ in range(args.steps):
            step.step()
            torch.cuda.synchronize()
            exp.append(step.exposed[0].elapsed_time(step.exposed[1]))
        step.exposed = None
        phases["allreduce_exposed"] = sum(exp) / len(exp)
        if step.reducer is not None:
            def alone():
                step.reducer.reduce(step.db32)
                step.reducer.join()
            phases["allreduce_alone"] = time_events(alone, args.steps)
        else:
            phases["allreduce_alone"] = time_events(lambda: dist.all_reduce(step.db32), args.steps)
        t = torch.tensor([phases[k_] for k_ in sorted(phases)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        phases = {k_: float(x) for k_, x in zip(sorted(phases), t)}
    if world == 1:
        step_q = quantiles(time_events_each(step.step, max(args.steps, 10)))
        # Algorithmic FLOPs per kernel (4 h n^3 d per contraction pair of the forward):
        # forward S and PV = 4; the one-pass dq/dk/dv kernel S, dP, dV, dK, dQ = 10 (with two
        # kernels the phase holds both and S, dP are executed twice: still 10 algorithmic);
        # db recomputes S and dP = 4 executed, none of them algorithmic beyond the 10.
        kernels_flops = {"forward": flops_fwd(w)}
        names = {"forward": "tc_fwd_d128_kernel" if w.d == 128 else "tc_fwd_kernel"}
        if w.backward:
            kernels_flops["backward_dqkv"] = 2.5 * flops_fwd(w)
            names["backward_dqkv"] = "tc_dqkv_kernel" if step.plan["bwd_fused"] else \
                "tc_dq_kernel + tc_dkv_kernel"
        top = max(kernels_flops, key=lambda k_: phases[k_])
        ach = kernels_flops[top] / (phases[top] * 1e-3) / 1e12
        peak = peaks["burst"]
        roofline = {"bound": "tensor", "kernel": names[top], "phase": top, "achieved": ach,
                    "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
                    "flops_per_launch": kernels_flops[top],
                    "flops_formula": "10*b*h*n^3*d" if top == "backward_dqkv" else "4*b*h*n^3*d",
                    "ms_per_launch": phases[top],
                    "peak_source": f"bf16 burst, {peaks['source']}", "traffic": None,
                    "step_frac_of_peak": total_flops / (ms * 1e-3) / 1e12 / peak,
                    "step_frac_of_sustained": total_flops / (ms * 1e-3) / 1e12 / peaks["sustained"]}
        try:
            prof = os.path.join(ROOT, "profiles", "traffic.json")
            if os.path.exists(prof):
                with open(prof) as f:
                    roofline["traffic"] = json.load(f).get(w.name, {}).get(top)
        except (OSError, ValueError):
            pass
        if rank == 0 and not args.no_cpu_baseline:
            torch.set_num_threads(os.cpu_count() or 1)
            crow = cpu_rows_for_budget(w, 8.0)
            cstep = cpu_sample_step(w, crow)
            cstep()
            t0 = time.perf_counter()
            cstep()
            dt = time.perf_counter() - t0
            cpu = {"value": flops_step(w, crow) / dt / 1e12, "unit": "TFLOP/s",
                   "cores": torch.get_num_threads(), "kind": "port", "host_cpus": os.cpu_count(),
                   "sample": f"{crow} of {w.n} pair rows, fp32 PyTorch CPU restatement, "
                             f"{dt:.1f} s; full step would be {dt * w.n / crow:.0f} s"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": total_flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": str(w.dtype).replace("torch.", ""),
            "data": "synthetic",
            "config": dict(workload_config(w, world),
                           **({"db_reduce": args.db_reduce,
                               "nccl_max_ctas": os.environ.get("NCCL_MAX_CTAS"),
                               "free_sms": free_sms, "push_ctas": args.push_ctas}
                              if world > 1 and w.backward else {})),
            "plan": step.plan, "clocks": clocks,
            "e2e": {"value": total_flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "public_api": {"value": total_flops / (api_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                           "ms_per_step": api_ms,
                           "call": "triangle_attention_row_sharded" if world > 1 else
                                   "triangle_attention", "backward": "o.backward(dO)"},
            "gpu_launches": step.launches * args.steps,
            # fraction of the N GPUs' combined dense bf16 tensor peak
            "frac_of_bf16_peak": {
                "measured_burst": total_flops / (ms * 1e-3) / 1e12 / (peaks["burst"] * world),
                "measured_sustained": total_flops / (ms * 1e-3) / 1e12 / (peaks["sustained"] * world),
                "nominal_2250": total_flops / (ms * 1e-3) / 1e12 / (2250.0 * world)},
        }
        line["phases_ms"] = phases
        if parity is not None:
            line["parity_ok"] = parity["ok"]
            line["parity"] = parity
        if roofline is not None:
            line["ms_per_step_quantiles"] = step_q
            line["forward_only"] = {"ms": phases["forward"],
                                    "tflops": flops_fwd(w) / (phases["forward"] * 1e-3) / 1e12}
            line["roofline"] = roofline
        if cpu is not None:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--workload", default="metric_n1024", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--db-reduce", default="nccl", choices=["nccl", "push"],
                    help="N > 1: how the db partials of the row shards are summed: NCCL all-reduce "
                         "or the library's own peer-store exchange")
    ap.add_argument("--push-ctas", type=int, default=4,
                    help="CTAs (1024 threads each) of the peer-store exchange kernel (--db-reduce push)")
    ap.add_argument("--free-sms", type=int, default=0,
                    help="SMs the dq/dk/dv kernel leaves free for the db exchange at N > 1 (0: 8)")
    ap.add_argument("--rows", type=int, default=0,
                    help="profiling aid: only this many pair rows of the workload (a row shard on "
                         "one GPU; the printed line is then not the benchmark)")
    ap.add_argument("--kernels-only", action="store_true",
                    help="profiling aid: only the kernels-only leg (no host-resident, operator or "
                         "CPU legs)")
    ap.add_argument("--e2e-chunk-rows", type=int, default=64,
                    help="pair rows per block of the host-resident pipeline (e2e figure)")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, w)
    else:
        run_native(args, w)


if __name__ == "__main__":
    main()
