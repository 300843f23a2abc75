"""Optimizer stage benchmark: one full step (gradient norm + clip, AdamW groups, Muon shape groups) on a preset's
parameter set, with the time of every Muon shape group. Counterpart of the reference's `muon_benchmark`
(backends/cuda/kernels/muon_benchmark.cc); its published H100 numbers for the d20-sized parameter set
(360,448,600 matrix elements in 5 shape groups, docs/model.md:402-416) are printed beside the measurement.

    python -m nanochat_cpp_b200.bench.optim_bench [--model d20] [--ns-steps 5] [--iters 5] [--json out.json]

Timing: CUDA events on the launching stream, 3 warm-up steps, a 256 MB write between iterations to flush L2.
"""
from __future__ import annotations

import argparse
import json

import torch

REFERENCE_H100_MS = {5: 29.09, 1: 12.34, 0: 8.12}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="d20")
    ap.add_argument("--ns-steps", type=int, default=5)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--json", default="")
    a = ap.parse_args()
    from ..config import preset
    from ..models import GPT
    from ..optim import Optimizer, OptimizerConfig, SchedulerConfig, muon_cuda
    from ..train import mfu
    from .. import ops
    dev = torch.device("cuda")
    cfg = preset(a.model)
    model = GPT(cfg, dev, torch.bfloat16, seed=0)
    opt = Optimizer(model.params, OptimizerConfig(muon_ns_steps=a.ns_steps), SchedulerConfig(num_iterations=1000))
    model.params.grad.normal_(0, 1e-3)
    flush = torch.empty(64 * 1024 * 1024, dtype=torch.float32, device=dev)
    for s in (1, 2, 3):
        opt.step(s)
    torch.cuda.synchronize()
    groups = {}
    orig = muon_cuda.muon_group_step

    def timed(*args, **kw):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        r = orig(*args, **kw)
        e1.record()
        shape = tuple(args[1][0].shape)
        groups.setdefault(f"{shape[0]}x{shape[1]} x{len(args[0])}", []).append((e0, e1))
        return r

    muon_cuda.muon_group_step = timed
    totals, norms = [], []
    try:
        for it in range(a.iters):
            flush.fill_(float(it))
            e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            e0.record()
            opt.step(4 + it)
            e1.record()
            ops.grad_norm_and_clip([model.params.grad], 1.0)
            e2.record()
            torch.cuda.synchronize()
            totals.append(e0.elapsed_time(e1))
            norms.append(e1.elapsed_time(e2))
    finally:
        muon_cuda.muon_group_step = orig
    med = lambda xs: sorted(xs)[len(xs) // 2]
    per_group = {k: med([x.elapsed_time(y) for x, y in v]) for k, v in groups.items()}
    muon_ms = sum(per_group.values())
    matrix_elements = sum(s.count for s in model.params.specs if s.kind == "matrix")
    flops = mfu.muon_flops_per_step(cfg, a.ns_steps)
    out = {"model": a.model, "ns_steps": a.ns_steps, "matrix_elements": matrix_elements,
           "optimizer_step_ms": med(totals), "muon_groups_ms": per_group, "muon_ms": muon_ms,
           "muon_product_tflops": flops / (muon_ms * 1e-3) / 1e12 if muon_ms > 0 else 0.0,
           "grad_norm_and_clip_ms": med(norms),
           "reference_h100_muon_ms": REFERENCE_H100_MS.get(a.ns_steps),
           "reference_h100_matrix_elements": 360448600}
    print(json.dumps(out))
    if a.json:
        with open(a.json, "w") as f:
            json.dump(out, f)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
