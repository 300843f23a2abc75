"""Roofline fractions of the fused data-parallel kernels, per rank, max over ranks.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29533 \
        -m nanochat_cpp_b200.bench.dp_comm_bench [--preset d20]

Sets up the d20 parameter store in symmetric memory exactly as training does and times, with CUDA events after
warm-up and a barrier, each stage in isolation (all ranks start together, so waits for peers are short):

  reduce_scatter  every bucket of the step. Default (bf16 by stores): `grad_push` of everything other ranks own into
                  their receive slots, signal, then `grad_reduce_local` of this rank's shard; bytes that must cross
                  NVLink per GPU and direction: (N-1)/N * parameters * 2. With `NANOCHAT_DP_REDUCE=pull`: the fp32
                  pull (`reduce_pull`), (N-1) * shard * 4 bytes inbound.
  update_and_push the owner's whole optimizer step (AdamW slices and Muon with its Newton-Schulz products), whose
                  final stores write the bf16 parameters into all N ranks: (N-1) * owned * 2 bytes outbound, and as
                  many inbound from the other owners. Roofline = max(Newton-Schulz FLOPs at the measured sustained
                  GEMM rate, AdamW state bytes at the measured copy bandwidth, link bytes / link rate).
  gemm_wait       the first forward GEMM with its in-kernel flag wait against the same GEMM without it.

Link rate: 900 GB/s per direction per GPU (NVLink 5 nominal, the denominator the benchmark names); the fraction
against this pool's measured peer-copy rate (770 GB/s) is printed beside it.
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

LINK_GBS = 900.0            # nominal per direction per GPU: the roofline denominator
LINK_GBS_MEASURED = 770.0   # peer copy measured on this pool, for context


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

    # ---- reduce-scatter over all buckets
    push_mode = f.reduce_mode == "push"
    status = K._C.status_tensor(dev.index)

    # The transport's own pipeline, as the training step drives it: every bucket is announced back to back on the
    # compute stream (as if the whole backward had just finished); pushes, signals and reductions then run on the
    # transport's streams. Timed from the first announcement to the moment both streams have drained.
    times = []
    cur = torch.cuda.current_stream()
    for i in range(6):
        step[0] += 1
        torch.cuda.synchronize()
        dist.barrier()
        a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(cur)
        f.begin_reduction()
        for b in range(len(f.buckets)):
            f.reduce_bucket(b, step[0])
        cur.wait_stream(f.comm_stream)
        cur.wait_stream(f.push_stream)
        b_.record(cur)
        torch.cuda.synchronize()
        if i >= 2:
            times.append(a.elapsed_time(b_))
    reduce_ms = sorted(times)[len(times) // 2]
    shard_elems = sum(bk["total"] for bk in f.buckets)
    n_params = model.params.num_params()
    if push_mode:
        reduce_link_bytes = int((world - 1) / world * n_params * 2)
    else:
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
        from ..train import mfu as perf
        peaks = perf.measured_peaks()
        red_roof = reduce_link_bytes / (LINK_GBS * 1e9) * 1e3
        push_roof = push_link_bytes / (LINK_GBS * 1e9) * 1e3
        ns_flops = perf.muon_flops_per_step(cfg, 5) / world
        ns_ms = ns_flops / (peaks["bf16_tflops_sustained"] * 1e12) * 1e3
        adamw_ms = owned_adamw * 30.0 / (peaks["hbm_gbs"] * 1e9) * 1e3      # master, grad, m, v read; master, m, v, bf16 written
        upd_roof = max(push_roof, ns_ms, adamw_ms)
        print(json.dumps(dict(
            n_gpus=world, model=args.preset, link_gbs_roofline=LINK_GBS, link_gbs_measured_peer_copy=LINK_GBS_MEASURED,
            reduce_scatter=dict(mode="bf16 push + local reduce" if push_mode else "fp32 pull", ms=round(reduce_ms, 3),
                                link_bytes_per_gpu_per_direction=reduce_link_bytes,
                                achieved_gbs=round(reduce_link_bytes / reduce_ms / 1e6, 1),
                                roofline_ms=round(red_roof, 3), fraction_of_roofline=round(red_roof / reduce_ms, 3),
                                fraction_of_measured_link=round(reduce_link_bytes / (LINK_GBS_MEASURED * 1e6) / reduce_ms, 3)),
            update_and_push=dict(ms=round(opt_ms, 3), link_bytes_per_gpu_per_direction=push_link_bytes,
                                 link_roofline_ms=round(push_roof, 3), newton_schulz_at_peak_ms=round(ns_ms, 3),
                                 adamw_hbm_ms=round(adamw_ms, 3), roofline_ms=round(upd_roof, 3),
                                 fraction_of_roofline=round(upd_roof / opt_ms, 3)),
            gemm_flag_wait=dict(plain_ms=round(plain, 4), with_wait_ms=round(waited, 4),
                                overhead_us=round((waited - plain) * 1e3, 2)))))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
