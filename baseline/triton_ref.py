"""Same-GPU measurement of the unmodified reference (its Triton kernels).

    python baseline/triton_ref.py [--steps K] [--warmup W] [--workload metric_n1024]

Runs ``trifast.triangle_attention`` from ``baseline/_ref`` (see install_ref.py) through
the reference's own public API and stock code path: forward and forward + backward times of
the workload (CUDA events), and the maximum absolute error of its bf16 / fp16 outputs and
gradients against the fp64 oracle at n = 128 and 256 -- the "error the reference's own
Triton kernel shows", which the parity tests may use as their bound.  Prints one JSON line
with "impl": "triton_reference".  The process sees ``baseline/_ref`` before anything else
named ``trifast``; the autotune cache of the reference goes to a temporary directory.
If the reference cannot be imported or run here the line says why and the exit code is 0.
"""

import argparse
import importlib.util
import json
import os
import sys
import tempfile
import traceback

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="metric_n1024")
    ap.add_argument("--skip-errors", action="store_true")
    args = ap.parse_args()
    os.environ["XDG_CONFIG_HOME"] = tempfile.mkdtemp(prefix="trifast_ref_cfg_")
    sys.path[:] = [p for p in sys.path if os.path.abspath(p or ".") != ROOT]
    sys.path.insert(0, os.path.join(HERE, "_ref"))
    line = {"impl": "triton_reference", "metric": "triangle_attention_fwd_bwd_tflops"}
    try:
        import torch
        configs = load(os.path.join(ROOT, "trifast_b200", "configs.py"), "ref_arm_configs")
        orc = load(os.path.join(ROOT, "oracle", "triangle_oracle.py"), "ref_arm_oracle")
        import trifast                                  # baseline/_ref/trifast
        assert os.path.abspath(trifast.__file__).startswith(os.path.join(HERE, "_ref")), trifast.__file__
        from trifast import triangle_attention
        import triton
        w = configs.WORKLOADS[args.workload]
        dev = torch.device("cuda")
        q, k, v, b, m, do = configs.make_inputs(w, seed=0, device=dev)
        for t in (q, k, v, b):
            t.requires_grad_(True)

        def fwd():
            return triangle_attention(q, k, v, b, m)

        def fwd_bwd():
            o = fwd()
            o.backward(do)
            q.grad = k.grad = v.grad = b.grad = None

        def timed(fn, iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / iters

        with torch.no_grad():
            for _ in range(max(args.warmup, 3)):     # first call autotunes
                fwd()
            torch.cuda.synchronize()
            fwd_ms = timed(fwd, args.steps)
        for _ in range(max(args.warmup, 3)):
            fwd_bwd()
        torch.cuda.synchronize()
        step_ms = timed(fwd_bwd, args.steps)
        flops_fwd = 4.0 * w.batch * w.h * w.n ** 3 * w.d
        line.update({
            "value": 3.5 * flops_fwd / (step_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "ms_per_step": step_ms, "forward_ms": fwd_ms,
            "forward_tflops": flops_fwd / (fwd_ms * 1e-3) / 1e12,
            "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
            "dtype": str(w.dtype).replace("torch.", ""), "data": "synthetic",
            "config": {"workload": w.name, "n": w.n, "heads": w.h, "head_dim": w.d},
            "versions": {"triton": triton.__version__, "torch": torch.__version__,
                         "gpu": torch.cuda.get_device_name()},
        })
        if not args.skip_errors:
            errs = {}
            for dtype in (torch.bfloat16, torch.float16):
                for n in (128, 256):
                    torch.manual_seed(1337)
                    h, d = 4, 32
                    qs, ks, vs = (torch.randn(1, h, n, n, d) for _ in range(3))
                    bs = torch.randn(1, h, n, n)
                    ms = torch.randint(0, 2, (1, n, n), dtype=torch.bool)
                    ms[:, torch.arange(n), torch.arange(n)] = False
                    dos = torch.randn(1, h, n, n, d)
                    lo = [t.to(dtype) for t in (qs, ks, vs, bs, dos)]
                    ref_o, _ = orc.forward(*(t.float() for t in lo[:4]), ms, torch.float64)
                    ref_g = orc.backward(lo[4].float(), *(t.float() for t in lo[:4]), ms, torch.float64)
                    g = [t.to(dev).requires_grad_(True) for t in lo[:4]]
                    o = triangle_attention(g[0], g[1], g[2], g[3], ms.to(dev))
                    o.backward(lo[4].to(dev))
                    torch.cuda.synchronize()
                    got = [o] + [t.grad for t in g]
                    key = f"{str(dtype).replace('torch.', '')}_n{n}"
                    errs[key] = {nm: float((x.detach().double().cpu() - r.double()).abs().max())
                                 for nm, x, r in zip(("o", "dq", "dk", "dv", "db"), got, (ref_o,) + tuple(ref_g))}
            line["max_abs_err_vs_fp64_oracle"] = errs
    except Exception as e:  # noqa: BLE001 - the reason is the result
        line["unavailable"] = f"{type(e).__name__}: {e}".splitlines()[0][:300]
        line["traceback_tail"] = traceback.format_exc().splitlines()[-6:]
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
