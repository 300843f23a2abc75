"""Block-scaled fp8 GEMMs (fp32 scales with CUDA-core promotion, and MXFP8 with the scales inside the MMA) against
this package's bf16 GEMM and cuBLAS bf16 on the d26 / d20 linear shapes.

    python -m nanochat_cpp_b200.bench.fp8_bench [--only d20.qkv] [--rows 16384] [--mx-only | --sustained]

`--only`, `--rows` and `--mx-only` cut the run down to a few launches of one kernel on a small case (for a profiler).

Times (CUDA events, 3 warm-ups, L2 flushed between iterations) the GEMM alone and the GEMM plus the activation
quantization that a forward pass needs (weights are quantized once per optimizer step, not per call).
"""
from __future__ import annotations

import json

import torch

from ..ops import cuda as K
from ..ops import fp8
from .timing import time_cuda

SHAPES = [("d26.qkv", 32768, 4992, 1664), ("d26.fc", 32768, 6656, 1664), ("d26.mlp_proj", 32768, 1664, 6656),
          ("d20.qkv", 65536, 3840, 1280), ("d20.fc", 65536, 5120, 1280), ("d20.mlp_proj", 65536, 1280, 5120)]


def sustained(fn, label: str, flops: float, secs: float = 3.0) -> dict:
    """Back-to-back launches for `secs` seconds with the SM clock and board power sampled every 100 ms: what the
    kernel delivers once the power cap has settled (a burst of ten launches runs at a higher clock)."""
    import statistics
    import subprocess
    import time
    for _ in range(5):
        fn()
    torch.cuda.synchronize()
    smi = subprocess.Popen(["nvidia-smi", "--query-gpu=clocks.sm,power.draw,clocks_event_reasons.sw_power_cap",
                            "--format=csv,noheader,nounits", "-lms", "100", "-i", str(torch.cuda.current_device())],
                           stdout=subprocess.PIPE, text=True)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n, t0 = 0, time.time()
    a.record()
    while time.time() - t0 < secs:
        for _ in range(50):
            fn()
        n += 50
        torch.cuda.synchronize()
    b.record()
    torch.cuda.synchronize()
    smi.terminate()
    rows = [l.split(",") for l in smi.stdout.read().strip().splitlines()[3:] if l.count(",") == 2]
    ms = a.elapsed_time(b) / n
    return dict(kernel=label, ms=round(ms, 4), tflops=round(flops / ms / 1e9, 1),
                sm_mhz_median=statistics.median(float(r[0]) for r in rows) if rows else None,
                power_w_median=statistics.median(float(r[1]) for r in rows) if rows else None,
                power_cap_active_samples=sum(r[2].strip() == "Active" for r in rows), samples=len(rows))


def main():
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default=None, help="one shape name")
    ap.add_argument("--rows", type=int, default=0, help="override M")
    ap.add_argument("--mx-only", action="store_true", help="three launches of the MXFP8 GEMM, nothing else timed")
    ap.add_argument("--sustained", action="store_true",
                    help="3-second loops of the MXFP8 and bf16 GEMMs with clock and power sampling")
    args = ap.parse_args()
    for name, M, N, Kd in SHAPES:
        if args.only and name != args.only:
            continue
        M = args.rows or M
        if args.sustained:
            x = torch.randn(M, Kd, device="cuda").to(torch.bfloat16)
            w = (torch.randn(N, Kd, device="cuda") * 0.02).to(torch.bfloat16)
            mq, ms = fp8.mx_quantize(w, fp8.mx_tile_n(N))
            aq, as_ = fp8.mx_quantize(x, 128)
            out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
            fl = 2.0 * M * N * Kd
            print(json.dumps(dict(name=name, **sustained(lambda: fp8.mx_gemm(aq, as_, mq, ms, out), "mxfp8", fl))))
            print(json.dumps(dict(name=name, **sustained(lambda: K.gemm(x, w, out=out), "bf16", fl))))
            print(json.dumps(dict(name=name, **sustained(lambda: torch.matmul(x, w.t(), out=out), "cublas_bf16", fl))))
            continue
        if args.mx_only:
            x = torch.randn(M, Kd, device="cuda").to(torch.bfloat16)
            w = (torch.randn(N, Kd, device="cuda") * 0.02).to(torch.bfloat16)
            mq, ms = fp8.mx_quantize(w, fp8.mx_tile_n(N))
            aq, as_ = fp8.mx_quantize(x, 128)
            out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
            for _ in range(3):
                fp8.mx_gemm(aq, as_, mq, ms, out)
            torch.cuda.synchronize()
            print(json.dumps(dict(name=name, m=M, n=N, k=Kd, launches=3)))
            continue
        Np = (N + 127) // 128 * 128
        x = torch.randn(M, Kd, device="cuda").to(torch.bfloat16)
        w = (torch.randn(Np, Kd, device="cuda") * 0.02).to(torch.bfloat16)
        wq, sw = fp8.quantize_blocks(w)
        wq = wq[:N].contiguous()
        xq, sx = fp8.quantize_rows(x)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        t_fp8 = time_cuda(lambda: fp8.fp8_gemm(xq, sx, wq, sw, out))["median_ms"]
        t_q = time_cuda(lambda: fp8.quantize_rows(x))["median_ms"]
        mq, ms = fp8.mx_quantize(w[:N].contiguous(), fp8.mx_tile_n(N))
        aq, as_ = fp8.mx_quantize(x, 128)
        t_mx = time_cuda(lambda: fp8.mx_gemm(aq, as_, mq, ms, out))["median_ms"]
        t_mx1 = time_cuda(lambda: fp8.mx_gemm(aq, as_, mq, ms, out, variant=1))["median_ms"]
        t_mq = time_cuda(lambda: fp8.mx_quantize(x, 128))["median_ms"]
        t_bf16 = time_cuda(lambda: K.gemm(x, w[:N], out=out))["median_ms"]
        t_lib = time_cuda(lambda: torch.matmul(x, w[:N].t(), out=out))["median_ms"]
        flops = 2.0 * M * N * Kd
        print(json.dumps(dict(name=name, m=M, n=N, k=Kd, fp8_ms=round(t_fp8, 4), quantize_ms=round(t_q, 4),
                              bf16_ms=round(t_bf16, 4), cublas_bf16_ms=round(t_lib, 4),
                              mx_ms=round(t_mx, 4), mx_single_cta_ms=round(t_mx1, 4), mx_quantize_ms=round(t_mq, 4),
                              mx_tflops=round(flops / t_mx / 1e9, 1), mx_speedup_gemm=round(t_bf16 / t_mx, 3),
                              mx_speedup_with_quantize=round(t_bf16 / (t_mx + t_mq), 3),
                              fp8_tflops=round(flops / t_fp8 / 1e9, 1), bf16_tflops=round(flops / t_bf16 / 1e9, 1),
                              speedup_gemm=round(t_bf16 / t_fp8, 3),
                              speedup_with_quantize=round(t_bf16 / (t_fp8 + t_q), 3))))
    K.check_status()


if __name__ == "__main__":
    main()
