"""Generate the golden vectors in this directory from the reference checkout.

Run where the reference source tree is present:

    python tests/golden/make_golden.py /path/to/reference

It loads the reference's ``src/trifast/equiv.py`` and ``src/trifast/utils.py``
by file path (the package itself needs a GPU to import), draws inputs with the
reference's own ``gen_tensors`` after ``torch.manual_seed(seed)``, runs
``attention_reference`` forward and autograd backward on the CPU and stores
inputs and results as ``<case>.npz``.  The committed ``.npz`` files are what the
oracle and the CUDA kernels are pinned against; this script is kept so they can
be regenerated.
"""

import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# name: (n, h, d, batch, std, mask kind, dtype, seed)
CASES = {
    "ragged17_randmask_fp32": (17, 2, 16, 2, 1.0, "random", torch.float32, 1337),
    "n32_h4_d32_drop10_fp32": (32, 4, 32, 1, 1.0, "drop10", torch.float32, 1337),
    "n24_padrows_fp32": (24, 2, 16, 1, 1.0, "padding", torch.float32, 7),
    "n25_d64_std2_nomask_fp32": (25, 1, 64, 1, 2.0, "none", torch.float32, 11),
    "n19_d128_randmask_fp32": (19, 1, 128, 1, 1.0, "random", torch.float32, 5),
    "n40_d32_randmask_bf16": (40, 1, 32, 1, 1.0, "random", torch.bfloat16, 3),
}


def load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main(ref_root):
    equiv = load(os.path.join(ref_root, "src/trifast/equiv.py"), "ref_equiv")
    utils = load(os.path.join(ref_root, "src/trifast/utils.py"), "ref_utils")
    for name, (n, h, d, batch, std, mkind, dtype, seed) in CASES.items():
        torch.manual_seed(seed)
        q, k, v, b, m = utils.gen_tensors(n, d, h, mkind == "random", "cpu",
                                          dtype=torch.float32, batch=batch, std=std)
        do = torch.randn(q.shape)
        if mkind == "drop10":
            m = torch.rand((batch, n, n)) < 0.10
            idx = torch.arange(n)
            m[:, idx, idx] = False
        elif mkind == "padding":
            pad = torch.arange(n) >= int(0.8 * n)
            m = (pad[:, None] | pad[None, :]).expand(batch, n, n).clone()
        with torch.no_grad():
            q, k, v, b, do = (t.to(dtype) for t in (q, k, v, b, do))
        for t in (q, k, v, b):
            t.requires_grad_(True)
        o = equiv.attention_reference(q, k, v, b, m)
        o.backward(do)
        f = lambda t: t.detach().float().numpy()
        np.savez_compressed(
            os.path.join(HERE, name + ".npz"),
            q=f(q), k=f(k), v=f(v), bias=f(b), mask=m.numpy(), do=f(do),
            o=f(o), dq=f(q.grad), dk=f(k.grad), dv=f(v.grad), db=f(b.grad),
            dtype=str(dtype).replace("torch.", ""),
        )
        print(name, "o", tuple(o.shape), "max|o|", float(o.detach().abs().max()))


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path to a checkout of latkins/trifast>")
    main(sys.argv[1])
