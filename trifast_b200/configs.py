"""Synthetic workloads: the measured configurations of the triangle-attention path.

Every workload is fully determined by its name and a seed.  Values follow the
reference generator's convention (``src/trifast/utils.py:5-33``: normal draws in
the order q, k, v, bias); q, k, v are then scaled to std d**-0.5 and the bias to
its own std; the upstream gradient dO ~ N(0, 1) is drawn next from the same
generator and masks come from a second generator seeded with ``seed + 1``.
Tensors are drawn once on the CPU in fp32 and rounded to the workload dtype, so
the CPU checker and the GPU kernels see identical bits.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class Workload:
    name: str
    n: int
    h: int
    d: int
    dtype: torch.dtype
    mask: str            # "none" | "random:<p>" | "padding:<valid fraction>"
    bias_std: float = 1.0
    batch: int = 1
    backward: bool = True


WORKLOADS = {
    # CPU plumbing case: fp32, ~10 % random key drops, never a full row.
    "c1_cpu_plumbing": Workload("c1_cpu_plumbing", 32, 4, 32, torch.float32, "random:0.10"),
    # AF2/OpenFold-scale pair stack, nothing masked.
    "c2_n256": Workload("c2_n256", 256, 4, 32, torch.bfloat16, "none"),
    # AF3/Boltz Pairformer scale, last 15 % of residues padded in i and k.
    "c3_n512_pad": Workload("c3_n512_pad", 512, 4, 32, torch.bfloat16, "padding:0.85"),
    # Inference-only forward, sharper softmax, ~5 % random key drops.
    "c4_n1024_h8_d64_fwd": Workload("c4_n1024_h8_d64_fwd", 1024, 8, 64, torch.float16,
                                    "random:0.05", bias_std=2.0, backward=False),
    # Large-complex training step, last 10 % padded.
    "c5_n2048_pad": Workload("c5_n2048_pad", 2048, 4, 32, torch.bfloat16, "padding:0.90"),
    # Head dim 128, inference-only forward: the one head dim of the reference's test matrix at
    # which the contraction, not the exponentials, is the larger load.
    "d128_n1024_fwd": Workload("d128_n1024_fwd", 1024, 4, 128, torch.bfloat16, "none",
                               backward=False),
    # Headline metric shape.
    "metric_n1024": Workload("metric_n1024", 1024, 4, 32, torch.bfloat16, "none"),
}


def make_mask(w: Workload, seed: int, device="cpu") -> torch.Tensor:
    """(batch, n, n) bool, True = key masked out, indexed (b, i, k)."""
    n, b = w.n, w.batch
    if w.mask == "none":
        return torch.zeros((b, n, n), dtype=torch.bool, device=device)
    kind, arg = w.mask.split(":")
    if kind == "random":
        g = torch.Generator(device=device).manual_seed(seed + 1)
        m = torch.rand((b, n, n), generator=g, device=device) < float(arg)
        idx = torch.arange(n, device=device)
        m[:, idx, idx] = False          # never a fully masked row
        return m
    if kind == "padding":
        n_valid = int(float(arg) * n)
        pad = torch.arange(n, device=device) >= n_valid
        return (pad[:, None] | pad[None, :]).expand(b, n, n).clone()
    raise ValueError(w.mask)


def make_inputs(w: Workload, seed: int = 1337, rows: slice | None = None, device="cpu",
                sample_rows: int | None = None):
    """Tensors (q, k, v, bias, mask, dO) of workload ``w`` in its dtype.

    Drawn on ``device`` (parity tests draw on the CPU and copy, so checker and
    kernels see the same bits; the benchmark draws on the GPU).  ``rows``
    selects a pair-row shard of q, k, v, mask and dO after the draw, so every
    shard of one seed comes from the same full-size tensors.  ``sample_rows``
    instead draws only that many pair rows directly (same distributions, not the
    same values as the full draw): the bounded sample of the CPU timing legs.
    """
    g = torch.Generator(device=device).manual_seed(seed)
    shape = (w.batch, w.h, sample_rows or w.n, w.n, w.d)
    s = w.d ** -0.5

    def draw(shp, std):
        # Rounded to the workload dtype at once: fp32 copies of the n = 2048
        # workload would not fit beside each other on a small host.
        return (torch.randn(shp, generator=g, device=device) * std).to(w.dtype)

    q, k, v = draw(shape, s), draw(shape, s), draw(shape, s)
    bias = draw((w.batch, w.h, w.n, w.n), w.bias_std)
    do = draw(shape, 1.0)
    mask = make_mask(w, seed, device)
    if sample_rows:
        mask = mask[:, :sample_rows].contiguous()
    if rows is not None:
        q, k, v, do = (t[:, :, rows].contiguous() for t in (q, k, v, do))
        mask = mask[:, rows].contiguous()
    return q, k, v, bias, mask, do
