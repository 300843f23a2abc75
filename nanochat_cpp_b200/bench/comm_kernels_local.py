"""The data-parallel transport's kernels on ONE GPU, with the peers' buffers standing in as local allocations.

    python -m nanochat_cpp_b200.bench.comm_kernels_local [--world 8] [--mb 256] [--iters 10]

What crosses NVLink in a real run lands in this GPU's own memory here, so the numbers are the kernels' HBM-side cost
(how fast they read, convert, scatter and reduce), not link time: the lower bound that the link adds to. The module
exists so that each kernel can be captured by a profiler on a small bucket (one process, one GPU, a few hundred MB)
and so that its byte counts can be checked against the algorithmic ones:

  grad_push          reads the fp32 gradient of what other ranks own, writes it as bf16 into their receive slots
                     algorithmic bytes: 4 read + 2 written per pushed element
  grad_reduce_local  owner: own fp32 gradient + (world - 1) bf16 slots -> fp32 sum, scaled, and the sum of squares
                     algorithmic bytes: 4 + 2 (world - 1) read + 4 written per owned element
  adamw_push         owner: AdamW on its slice (fp32 master, m, v, grad) and a bf16 store of the new values into every
                     rank's parameter buffer: 16 read + 12 written + 2 world written per element

The pipeline these kernels form, its flags and its overlap with the backward pass are timed across real GPUs by
`dp_comm_bench`.
"""
from __future__ import annotations

import argparse
import json

import torch


def _time(fn, iters, flush):
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times = []
    for _ in range(iters):
        flush.zero_()                       # L2 flush: 256 MB > 126 MB
        torch.cuda.synchronize()
        ev0.record()
        fn()
        ev1.record()
        torch.cuda.synchronize()
        times.append(ev0.elapsed_time(ev1))
    times.sort()
    return times[len(times) // 2]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--mb", type=int, default=256, help="size of the fp32 gradient bucket in MB")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--ctas", type=int, default=296,
                    help="CTAs of the two gradient kernels (the transport's default is 2 per SM = 296)")
    a = ap.parse_args(argv)
    from ..ops import cuda as K
    from ..train import mfu
    C = K._C
    dev = torch.device("cuda", 0)
    world = a.world
    n = a.mb * (1 << 20) // 4
    share = n // world // 64 * 64                     # elements each rank owns (one run per owner)
    n = share * world
    cap = share
    grad = torch.randn(n, device=dev)
    recv = [torch.zeros(world * cap, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    rptrs = [t.data_ptr() for t in recv]
    flags = [torch.zeros(2 * world, dtype=torch.int32, device=dev) for _ in range(world)]
    status = C.status_tensor(0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    me = 0
    rows, first = [], 0
    for owner in range(world):
        if owner == me:
            continue
        rows.append([first, owner * share, 0, owner, share])
        first += share // 8
    push_rows = torch.tensor(rows, dtype=torch.int64, device=dev)
    own_rows = torch.tensor([[0, me * share, 0, share]], dtype=torch.int64, device=dev)
    acc = torch.zeros(1, dtype=torch.float64, device=dev)

    def push():
        C.comm_grad_push(grad, rptrs, cap, me, push_rows, first, 1.0 / world, a.ctas)

    def reduce_local():                                # flag value 0: every "peer" has already arrived
        C.comm_grad_reduce_local(grad, recv[me], cap, world, me, own_rows, share // 8, 1.0 / world, flags[me], 1,
                                 0, acc, status, a.ctas)

    # AdamW + push of the owned slice into `world` parameter buffers
    values = [torch.zeros(n, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    vptrs = [v.data_ptr() for v in values]
    master = torch.randn(share, device=dev)
    g_own = torch.randn(share, device=dev)
    m1, v1 = torch.zeros(share, device=dev), torch.zeros(share, device=dev)
    scale = torch.ones(1, device=dev)

    def adamw_push():
        C.comm_adamw_push(master, vptrs, me * share, g_own, m1, v1, 1e-3, 0.8, 0.95, 1e-10, 0.0, 3, scale)

    for _ in range(a.warmup):
        push(), reduce_local(), adamw_push()
    torch.cuda.synchronize()
    K.check_status()
    peaks = mfu.measured_peaks()
    hbm = peaks["hbm_gbs"]
    pushed = share * (world - 1)
    out = {"world": world, "bucket_mb": a.mb, "hbm_gbs_measured": hbm, "kernels": {}}
    for name, fn, nbytes in (("grad_push", push, pushed * 6),
                             ("grad_reduce_local", reduce_local, share * (4 + 2 * (world - 1) + 4)),
                             ("adamw_push", adamw_push, share * (16 + 12 + 2 * world))):
        ms = _time(fn, a.iters, flush)
        gbs = nbytes / ms / 1e6
        out["kernels"][name] = {"ms": round(ms, 4), "algorithmic_mb": round(nbytes / 1e6, 1), "gb_per_s": round(gbs, 1),
                                "of_measured_hbm": round(gbs / hbm, 3)}
    K.check_status()
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
