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
  roofline            : the dominant kernel phase against the measured bf16 tensor peak
  phases_ms           : forward / db / dq+dk+dv phase times (CUDA events, N = 1)
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

    def __init__(self, w, q, k, v, b, m, do, group_size):
        from trifast_b200 import _lib
        self.lib, self._lib = _lib.load(), _lib
        self.w, self.world = w, group_size
        bs, h, rows, n, d = q.shape
        dev = q.device
        self.t = dict(q=q, k=k, v=v, b=b, do=do)
        self.m8 = m.view(torch.uint8)
        self.o = torch.empty_like(q)
        self.lse = torch.empty((bs, h, rows, n), dtype=torch.float32, device=dev)
        self.shape = _lib.make_shape(bs, h, n, rows, d, q.dtype)
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
        # launches per step: forward 1; backward: row flags + packed mask, bias transpose
        # (tensor-core path only), delta, db, split reduce (if split), dq, dk/dv, cast
        self.launches = 1
        if w.backward:
            self.launches += 1 + (1 if plan["kernel"] == 2 else 0) + 1 + 1 + \
                (1 if plan["db_row_splits"] > 1 else 0) + 2 + 1

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

    def finalize(self):
        rc = self.lib.trifast_db_finalize(C.byref(self.shape), C.c_void_p(self.db32.data_ptr()),
                                          C.byref(self.adb), self.stream)
        self._lib.check(rc, "trifast_db_finalize")

    def step(self):
        import torch.distributed as dist
        self.forward()
        if not self.w.backward:
            return
        self.backward_db()
        work = None
        if self.world > 1:
            work = dist.all_reduce(self.db32, async_op=True)
        self.backward_dqkv()
        if work is not None:
            work.wait()
        self.finalize()


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
        dist.init_process_group("nccl", device_id=dev)
    from trifast_b200.dist import shard_rows, triangle_attention_row_sharded
    rows = shard_rows(w.n, rank, world)
    q, k, v, b, m, do = make_inputs(w, seed=0, rows=rows if world > 1 else None, device=dev)
    torch.cuda.synchronize()
    step = DirectStep(w, q, k, v, b, m, do, world)

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

    # ---- per-phase timing, roofline and the CPU baseline (single GPU only) ------------
    phases, roofline, cpu = None, None, None
    peaks = measured_peaks()
    step_q = None
    if world == 1:
        step_q = quantiles(time_events_each(step.step, max(args.steps, 10)))
        phases = {"forward": time_events(step.forward, args.steps)}
        kernels_flops = {"forward": flops_fwd(w)}
        if w.backward:
            phases["backward_db"] = time_events(step.backward_db, args.steps)
            phases["backward_dqkv"] = time_events(step.backward_dqkv, args.steps)
            # contractions each phase executes: db recomputes S and dP (2 of them);
            # dq+dk+dv executes S, dP (twice when dq and dk/dv are separate kernels), dQ, dK, dV
            kernels_flops["backward_db"] = flops_fwd(w)
            kernels_flops["backward_dqkv"] = 2.5 * flops_fwd(w)
        top = max(phases, key=phases.get)
        ach = kernels_flops[top] / (phases[top] * 1e-3) / 1e12
        peak = peaks["burst"]
        roofline = {"bound": "tensor", "kernel": top, "achieved": ach, "peak": peak,
                    "unit": "TFLOP/s", "frac": ach / peak,
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
            "data": "synthetic", "config": workload_config(w, world),
            "plan": step.plan, "clocks": clocks,
            "e2e": {"value": total_flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": step.launches * args.steps,
            # fraction of the N GPUs' combined dense bf16 tensor peak
            "frac_of_bf16_peak": {
                "measured_burst": total_flops / (ms * 1e-3) / 1e12 / (peaks["burst"] * world),
                "measured_sustained": total_flops / (ms * 1e-3) / 1e12 / (peaks["sustained"] * world),
                "nominal_2250": total_flops / (ms * 1e-3) / 1e12 / (2250.0 * world)},
        }
        if phases is not None:
            line["phases_ms"] = phases
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
