"""Attention micro-benchmark on the reference's published shapes (docs/baselines.json `attention_flash_exp`,
`attention_hopper`): forward and backward time, achieved TFLOP/s over the visible (causal / windowed) area.

    python -m nanochat_cpp_b200.bench.attn_bench [--json out.jsonl] [--only NAME] [--iters N]
"""
from __future__ import annotations

import argparse
import json

import torch

from ..ops import cuda as K
from .timing import time_cuda

SHAPES = [
    # name, B, T, H, KV, D, window, reference fwd ms (H100), reference bwd ms (H100)
    ("b4_s2048_win512", 4, 2048, 8, 8, 128, 512, 0.113781, 0.866912),
    ("d8_s512", 8, 512, 4, 4, 128, -1, 0.021537, 0.176469),
    ("gqa_b2_t512_h8_kv2", 2, 512, 8, 2, 128, -1, 0.021013, 0.374443),
    ("d20_S_layer", 32, 2048, 10, 10, 128, 1024, None, None),
    ("d20_L_layer", 32, 2048, 10, 10, 128, -1, None, None),
]


def visible_pairs(T, window):
    n = 0
    for q in range(T):
        lo = 0 if window < 0 else max(0, q - window)
        n += q - lo + 1
    return n


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default="")
    ap.add_argument("--only", default="")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--variant", type=int, default=2)
    ap.add_argument("--report", default="", help="write a nanochat.bench.v3 document here")
    args = ap.parse_args()
    out = open(args.json, "w") if args.json else None
    from .report import BenchReport
    report = BenchReport().use_device_peak("bf16")
    for name, B, T, H, KV, D, window, ref_f, ref_b in SHAPES:
        if args.only and args.only != name:
            continue
        q = torch.randn(B, T, H, D, device="cuda").to(torch.bfloat16)
        k = torch.randn(B, T, KV, D, device="cuda").to(torch.bfloat16)
        v = torch.randn(B, T, KV, D, device="cuda").to(torch.bfloat16)
        do = torch.randn(B, T, H, D, device="cuda").to(torch.bfloat16)
        o, lse = K.attention_fwd(q, k, v, window, variant=args.variant)
        tf = time_cuda(lambda: K.attention_fwd(q, k, v, window, variant=args.variant), iters=args.iters)
        tb = time_cuda(lambda: K.attention_bwd(q, k, v, o, lse, do, window), iters=args.iters)
        pairs = visible_pairs(T, window) * B * H
        f_flops = 4.0 * pairs * D
        b_flops = 10.0 * pairs * D
        row = dict(name=name, B=B, T=T, H=H, KV=KV, D=D, window=window,
                   fwd_ms=round(tf["median_ms"], 4), bwd_ms=round(tb["median_ms"], 4),
                   fwd_tflops=round(f_flops / tf["median_ms"] / 1e9, 1),
                   bwd_tflops=round(b_flops / tb["median_ms"] / 1e9, 1),
                   ref_h100_fwd_ms=ref_f, ref_h100_bwd_ms=ref_b)
        print(json.dumps(row), flush=True)
        if out:
            out.write(json.dumps(row) + "\n")
        shape = f"B={B} T={T} H={H} KV={KV} D={D} window={window}"
        report.add("attention_fwd:" + name, shape, tf["median_ms"], f_flops / tf["median_ms"] / 1e6,
                   iterations=args.iters, family="attention", phase="fwd")
        report.add("attention_bwd:" + name, shape, tb["median_ms"], b_flops / tb["median_ms"] / 1e6,
                   iterations=args.iters, family="attention", phase="bwd")
    if args.report:
        report.write(args.report)
    K.check_status()


if __name__ == "__main__":
    main()
