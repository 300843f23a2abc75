"""GEMM micro-benchmark: the tcgen05 kernel against torch.matmul (cuBLAS) on the model's shapes.

Counterpart of the reference's `gemm_benchmark` (docs/performance.md:167-203). Prints one JSON line per
shape with both timings, TFLOP/s and the fraction of the measured cuBLAS peak.

    python -m nanochat_cpp_b200.bench.gemm_bench --preset d20 [--tokens 65536] [--json out.jsonl] [--report out.json]

`--report` also writes one `nanochat.bench.v3` document (family "linear", phase fwd / dgrad / wgrad, MFU against the
measured cuBLAS burst rate).
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from ..config import preset
from ..ops import cuda as K
from .timing import time_cuda


def shapes_for(cfg, tokens):
    C, F = cfg.hidden_dim, cfg.mlp_dim
    qkv = cfg.query_dim + 2 * cfg.kv_dim
    M = tokens
    rows = []
    for name, n, k in (("qkv", qkv, C), ("attn_proj", C, C), ("fc", F, C), ("mlp_proj", C, F)):
        rows.append((name + ".fwd", "fwd", M, n, k))
        rows.append((name + ".dgrad", "dgrad", M, k, n))
        rows.append((name + ".wgrad", "wgrad", n, k, M))
    hm = min(M, 8192)
    rows.append(("lm_head.fwd", "fwd", hm, cfg.padded_vocab_size, C))
    rows.append(("lm_head.dgrad", "dgrad", hm, C, cfg.padded_vocab_size))
    rows.append(("lm_head.wgrad", "wgrad", cfg.padded_vocab_size, C, hm))
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="d20")
    ap.add_argument("--tokens", type=int, default=65536)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--json", default="")
    ap.add_argument("--report", default="", help="write a nanochat.bench.v3 document here")
    ap.add_argument("--only", default="", help="run a single row, e.g. fc.fwd")
    ap.add_argument("--no-lib", action="store_true", help="skip the cuBLAS timing")
    args = ap.parse_args()
    cfg = preset(args.preset)
    peaks = {}
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                     "MEASURED_PEAKS.json")
    if os.path.exists(p):
        peaks = json.load(open(p))
    peak = float(peaks.get("bf16_tflops", 1590.0))
    out = open(args.json, "w") if args.json else None
    from .report import BenchReport
    report = BenchReport().use_device_peak("bf16")
    dev = "cuda"
    for name, kind, m, n, k in shapes_for(cfg, args.tokens):
        if args.only and args.only != name:
            continue
        # the GEMM is C[m,n] = sum_k; operands are laid out as the training step meets them
        if kind == "fwd":
            a = torch.randn(m, k, device=dev, dtype=torch.bfloat16)
            b = torch.randn(n, k, device=dev, dtype=torch.bfloat16)
            ours = lambda: K.gemm(a, b)
            lib = lambda: torch.matmul(a, b.t())
        elif kind == "dgrad":
            a = torch.randn(m, k, device=dev, dtype=torch.bfloat16)   # dy [M, N']
            b = torch.randn(k, n, device=dev, dtype=torch.bfloat16)   # w  [N', K']
            ours = lambda: K.gemm(a, b, b_mn=True)
            lib = lambda: torch.matmul(a, b)
        else:
            a = torch.randn(k, m, device=dev, dtype=torch.bfloat16)   # dy [tokens, N']
            b = torch.randn(k, n, device=dev, dtype=torch.bfloat16)   # x  [tokens, K']
            g = torch.zeros(m, n, device=dev, dtype=torch.float32)
            ours = lambda: K.gemm(a, b, a_mn=True, b_mn=True, epi=K.EPI_F32, out=g, beta=1.0)
            lib = lambda: g.add_(torch.matmul(a.t(), b))
        t_ours = time_cuda(ours, iters=args.iters)
        t_lib = t_ours if args.no_lib else time_cuda(lib, iters=args.iters)
        fl = 2.0 * m * n * k
        row = dict(name=name, m=m, n=n, k=k, ours_ms=round(t_ours["median_ms"], 4),
                   cublas_ms=round(t_lib["median_ms"], 4),
                   ours_tflops=round(fl / t_ours["median_ms"] / 1e9, 1),
                   cublas_tflops=round(fl / t_lib["median_ms"] / 1e9, 1),
                   frac_of_measured_peak=round(fl / t_ours["median_ms"] / 1e9 / peak, 3),
                   speedup_vs_cublas=round(t_lib["median_ms"] / t_ours["median_ms"], 3))
        print(json.dumps(row), flush=True)
        if out:
            out.write(json.dumps(row) + "\n")
        report.add("gemm:" + name, f"M={m} N={n} K={k}", t_ours["median_ms"], fl / t_ours["median_ms"] / 1e6,
                   iterations=args.iters, family="linear", phase=kind)
    if args.report:
        report.extras["preset"] = args.preset
        report.write(args.report)
    K.check_status()


if __name__ == "__main__":
    main()
