"""Roofline fractions of the fused data-parallel kernels, per rank, max over ranks.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29533 \
        -m nanochat_cpp_b200.bench.dp_comm_bench [--preset d20]

Sets up the d20 parameter store in symmetric memory exactly as training does and times, with CUDA events after
warm-up, each kernel in isolation (every rank has published its flags before the timed launch, so a kernel never
waits for a peer inside the timed region):

  reduce_pull   every bucket of the step: this rank's shard of the fp32 gradient loaded from all N ranks (N-1 over
                NVLink), summed, scaled, stored, sum of squares accumulated. Bytes that must cross NVLink per GPU:
                (N-1) * shard bytes inbound. Roofline time = that / 770 GB/s (measured peer-copy bandwidth).
  adamw_push    owner AdamW update writing bf16 parameters into all N ranks: (N-1) * 2 bytes/param outbound.
  muon_push     owner Muon apply writing bf16 matrices into all N ranks.
  gemm_wait     the first forward GEMM with its in-kernel flag wait against the same GEMM without it.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..config import preset
from ..models import GPT
from ..optim import Optimizer
from ..parallel import DataParallel

LINK_GBS = 770.0


def _time(fn, stream=None, iters=5, warmup=2):
    out = []
    for i in range(warmup + iters):
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s = stream or torch.cuda.current_stream()
        a.record(s)
        fn()
        b.record(s)
        torch.cuda.synchronize()
        if i >= warmup:
            out.append(a.elapsed_time(b))
    out.sort()
    return out[len(out) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="d20")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    cfg = preset(args.preset)
    dp = DataParallel(rank, world, transport="fused", device=dev)
    model = GPT(cfg, dev, torch.bfloat16, seed=0, allocator=dp.allocator())
    dp.prepare(model.params)
    opt = Optimizer(model.params, owned=dp.owned, adamw_slices=dp.slices)
    dp.attach(model, opt)
    f = dp.fused
    from ..ops import cuda as K
    model.params.grad.normal_(0, 1e-3)
    step = [0]

    # ---- reduce_pull over all buckets
    def reduce_all():
        step[0] += 1
        for b in range(len(f.buckets)):
            f.signal(b, step[0])
        torch.cuda.synchronize()
        dist.barrier()                       # every rank's flags are out before anything is timed

    def run_reduce():
        with torch.cuda.stream(f.comm_stream):
            for b, bk in enumerate(f.buckets):
                if bk["total"]:
                    K._C.comm_reduce_pull(f.grad.ptrs, f.rank, bk["segs"], bk["total"], 1.0, f.flags.tensor, b, step[0],
                                          f.sumsq, K._C.status_tensor(dev.index), f.reduce_ctas)
    times = []
    for i in range(6):
        reduce_all()
        a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(f.comm_stream)
        run_reduce()
        b_.record(f.comm_stream)
        torch.cuda.synchronize()
        if i >= 2:
            times.append(a.elapsed_time(b_))
    reduce_ms = sorted(times)[len(times) // 2]
    shard_elems = sum(bk["total"] for bk in f.buckets)
    reduce_link_bytes = (world - 1) * shard_elems * 4

    # ---- owner updates that push parameters
    K.check_status(dev)
    t_opt = []
    for i in range(5):
        dist.barrier()
        torch.cuda.synchronize()
        a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        opt.step(i + 1, clip_scale=torch.ones((), device=dev))
        b_.record()
        torch.cuda.synchronize()
        if i >= 2:
            t_opt.append(a.elapsed_time(b_))
    opt_ms = sorted(t_opt)[len(t_opt) // 2]
    owned_adamw = sum(max(0, dp.slices[s.name][1] - dp.slices[s.name][0]) for s in model.params.specs
                      if dp.owners[s.name] == -1)
    owned_muon = sum(s.count for s in model.params.specs if dp.owners[s.name] == rank)
    push_link_bytes = (world - 1) * (owned_adamw + owned_muon) * 2

    # ---- GEMM with the in-kernel flag wait (flags already satisfied) vs without
    x = torch.randn(32 * cfg.seq_len, cfg.hidden_dim, device=dev).to(torch.bfloat16)
    w = model.params.qkv_view(0)
    out = torch.empty(x.shape[0], w.shape[0], device=dev, dtype=torch.bfloat16)
    flags = f.flag_view(f.slot_muon)
    plain = _time(lambda: K.gemm(x, w, out=out))
    waited = _time(lambda: K.gemm(x, w, out=out, wait_flags=flags, wait_value=0))

    vals = torch.tensor([reduce_ms, opt_ms, plain, waited], device=dev, dtype=torch.float64)
    dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    reduce_ms, opt_ms, plain, waited = [float(v) for v in vals]
    K.check_status(dev)
    if rank == 0:
        red_roof = reduce_link_bytes / (LINK_GBS * 1e9) * 1e3
        push_roof = push_link_bytes / (LINK_GBS * 1e9) * 1e3
        print(json.dumps(dict(
            n_gpus=world, model=args.preset, link_gbs_measured_reference=LINK_GBS,
            reduce_pull=dict(ms=round(reduce_ms, 3), link_bytes_per_gpu=reduce_link_bytes,
                             achieved_gbs=round(reduce_link_bytes / reduce_ms / 1e6, 1),
                             roofline_ms=round(red_roof, 3), fraction_of_roofline=round(red_roof / reduce_ms, 3)),
            owner_update_and_push=dict(ms=round(opt_ms, 3), link_bytes_per_gpu=push_link_bytes,
                                       push_roofline_ms=round(push_roof, 3),
                                       note="includes the Newton-Schulz products of the owned matrices"),
            gemm_flag_wait=dict(plain_ms=round(plain, 4), with_wait_ms=round(waited, 4),
                                overhead_us=round((waited - plain) * 1e3, 2)))))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
