"""Device timing protocol shared by the micro-benchmarks.

Follows the reference's bench protocol (`backends/cuda/kernels/testing/bench_protocol.h`,
docs/performance.md:40-45): warm-up, then one CUDA-event pair per call on the launching stream with an
L2 flush (a write larger than the 126 MB L2) before each timed call, reporting min and median.
"""
from __future__ import annotations

import statistics
from typing import Callable, Dict

import torch

_flush_buf = None


def flush_l2() -> None:
    global _flush_buf
    if _flush_buf is None:
        _flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _flush_buf.zero_()


def time_cuda(fn: Callable[[], None], warmup: int = 3, iters: int = 10, flush: bool = True) -> Dict[str, float]:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush:
            flush_l2()
        start = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end))
    return {"min_ms": min(times), "median_ms": statistics.median(times)}
