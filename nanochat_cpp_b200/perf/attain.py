"""Attainment: join measured benchmark rows with the roofline's rows and report measured / bound.

    python -m nanochat_cpp_b200.perf.attain --profile profiles/step_profile_d20_batch32.txt --preset d20 --batch 32

The reference's `tools/nanochat attain` joins `nanochat.bench.v3` rows with `nanochat.roofline.v3` rows on (family,
phase) and writes `nanochat.attainment.v1`; this does the same for the operator table of `bench.step_profile`.
"""
from __future__ import annotations

import argparse
import json
import re
from typing import Dict

from ..config import preset
from .roofline import RooflinePlan, estimate

# operator of the step profile -> (roofline family prefix, phase)
JOIN = {
    "linear_fwd": ("gemm_", "forward"), "linear_relu2_fwd": ("gemm_mlp_fc", "forward"), "linear_relu2_act_fwd": ("gemm_mlp_fc", "forward"),
    "linear_dgrad_relu2_act": ("gemm_mlp_proj", "backward"),
    "linear_dgrad": ("gemm_", "backward"), "linear_wgrad": ("gemm_", "backward"),
    "linear_dgrad_relu2": ("gemm_mlp_proj", "backward"), "linear_wgrad_relu2": ("gemm_mlp_proj", "backward"),
    "attention_fwd": ("attention", "forward"), "attention_bwd": ("attention", "backward"),
    "classifier_fwd_bwd": ("classifier", "both"),
}


def read_profile(path: str) -> Dict[str, float]:
    out = {}
    for line in open(path):
        m = re.match(r"^(\w+)\s+([0-9.]+)\s+(\d+)\s*$", line)
        if m:
            out[m.group(1)] = float(m.group(2))
    return out


def attainment(measured_ms: Dict[str, float], cfg, plan: RooflinePlan) -> dict:
    est = estimate(cfg, plan)
    groups = {"gemm": [0.0, 0.0], "attention.forward": [0.0, 0.0], "attention.backward": [0.0, 0.0],
              "classifier": [0.0, 0.0]}
    for r in est.rows:
        if r.name.startswith("gemm_"):
            groups["gemm"][1] += r.bound_seconds * 1e3
        elif r.name == "attention":
            groups[f"attention.{r.phase}"][1] += r.bound_seconds * 1e3
        elif r.name == "classifier":
            groups["classifier"][1] += r.bound_seconds * 1e3
    for op, ms in measured_ms.items():
        if op.startswith("linear_"):
            groups["gemm"][0] += ms
        elif op == "attention_fwd":
            groups["attention.forward"][0] += ms
        elif op == "attention_bwd":
            groups["attention.backward"][0] += ms
        elif op == "classifier_fwd_bwd":
            groups["classifier"][0] += ms
    rows = [dict(family=k, measured_ms=round(m, 3), bound_ms=round(b, 3), attainment=round(b / m, 3) if m > 0 else None)
            for k, (m, b) in groups.items()]
    total = sum(measured_ms.values())
    return dict(schema="nanochat.attainment.v1", device=est.device, shape=est.shape, rows=rows,
                step_measured_ms=round(total, 3), step_bound_ms=round(est.step_seconds * 1e3, 3),
                step_attainment=round(est.step_seconds * 1e3 / total, 3) if total > 0 else None)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--profile", required=True)
    ap.add_argument("--preset", default="d20")
    ap.add_argument("--batch", type=int, default=32)
    a = ap.parse_args()
    print(json.dumps(attainment(read_profile(a.profile), preset(a.preset), RooflinePlan(batch=a.batch)), indent=1))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
