"""Batched KV-cache inference benchmark: prefill tok/s, decode tok/s and p50 per-token latency.

    python -m nanochat_cpp_b200.bench.decode_bench --preset d20 --prompts 64 --prompt-len 512 --new-tokens 256
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29521 \
        -m nanochat_cpp_b200.bench.decode_bench          # one replica per GPU, `--prompts` sequences each

Random-init bf16 weights, uniform-random prompts, greedy decoding over a paged KV cache (16-token pages), sliding
windows honoured. One replica per GPU; rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import statistics

import torch

from ..config import preset
from ..inference import InferenceEngine
from ..models import GPT


def run(preset_name: str = "d20", prompts_n: int = 64, prompt_len: int = 512, new_tokens: int = 256,
        use_graph: bool = True, sampler_cls=None, warmup: int = 3) -> dict:
    """Runs the benchmark on this rank's GPU (one replica per GPU) and returns the JSON document on rank 0, None
    elsewhere. Two timed passes over the same prompts:
      device-timed   prompts already on the device; prefill and every decode step bracketed by CUDA events;
      end to end     through `generate_multi`-style use of the public engine: the prompts start in pinned host
                     memory and are copied to the device inside the timed region, and every step's token ids are
                     read back to the host (as a serving loop that streams tokens does); wall clock.
    """
    import os
    import time
    cfg = preset(preset_name)
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        if not dist.is_initialized():
            dist.init_process_group("nccl", device_id=dev)
    from ..ops import cuda as K
    model = GPT(cfg, dev, torch.bfloat16, seed=0)
    eng = InferenceEngine(model, use_cuda_graph=use_graph)
    g = torch.Generator().manual_seed(rank)       # different prompts per replica
    host_prompts = torch.randint(0, cfg.vocab_size, (prompts_n, prompt_len), generator=g).pin_memory()
    prompts = host_prompts.to(dev)
    cache = eng.new_cache(prompts_n, prompt_len + new_tokens + 1)
    # warm-up (also builds tensor maps and the decode graph)
    logits = eng.prefill(cache, prompts)
    nxt = logits.argmax(-1)
    for _ in range(max(warmup, 1)):
        nxt = eng.decode_graphed(cache, nxt, greedy=True)
    torch.cuda.synchronize()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = None
    if rank == 0 and sampler_cls is not None:
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        sampler = sampler_cls(int(vis.split(",")[local]) if vis else local)
        sampler.start()
    # ---- device-timed pass
    cache.reset()
    barrier()
    launches0 = K.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    logits = eng.prefill(cache, prompts)
    e1.record()
    torch.cuda.synchronize()
    prefill_ms = e0.elapsed_time(e1)
    lat = []
    nxt = logits.argmax(-1)
    for _ in range(new_tokens):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        nxt = eng.decode_graphed(cache, nxt, greedy=True)     # next token ids straight from the step (greedy)
        b.record()
        b.synchronize()
        lat.append(a.elapsed_time(b))
    launches = K.launch_count() - launches0
    K.check_status()
    total_ms = sum(lat)
    p50 = statistics.median(lat)
    # ---- end-to-end pass
    cache.reset()
    barrier()
    t0 = time.perf_counter()
    dev_prompts = host_prompts.to(dev, non_blocking=True)
    logits = eng.prefill(cache, dev_prompts)
    nxt = logits.argmax(-1)
    first = nxt.tolist()
    t1 = time.perf_counter()
    produced = [first]
    for _ in range(new_tokens):
        nxt = eng.decode_graphed(cache, nxt, greedy=True)
        produced.append(nxt.tolist())                          # device -> host read of the step's result
    torch.cuda.synchronize()
    t2 = time.perf_counter()
    e2e_prefill_ms, e2e_decode_ms = (t1 - t0) * 1e3, (t2 - t1) * 1e3
    clocks = sampler.stop() if sampler is not None else {}
    K.check_status()
    if dist is not None:     # replicas are independent: the job's time is the slowest replica's (max over ranks)
        t = torch.tensor([total_ms, prefill_ms, p50, e2e_prefill_ms, e2e_decode_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, prefill_ms, p50, e2e_prefill_ms, e2e_decode_ms = (float(v) for v in t.tolist())
        dist.barrier()
    if rank != 0:
        return None
    return {
        "metric": "decode_tokens_per_sec", "n_gpus": world,
        "value": round(world * prompts_n * new_tokens / (total_ms / 1e3), 1), "unit": "tokens/s",
        "steps": new_tokens, "warmup": max(warmup, 1), "ms_per_step": round(total_ms / new_tokens, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "impl": "ours",
        "data": "uniform-random prompt ids, random-init weights",
        "prefill_tokens_per_sec": round(world * prompts_n * prompt_len / (prefill_ms / 1e3), 1),
        "p50_token_latency_ms": round(p50, 4), "prefill_ms": round(prefill_ms, 3),
        "cuda_graph": bool(eng._graph is not None), "kv_cache_gb": round(cache.bytes() / 1e9, 3),
        "e2e": {"value": round(world * prompts_n * new_tokens / (e2e_decode_ms / 1e3), 1), "unit": "tokens/s",
                "prefill_tokens_per_sec": round(world * prompts_n * prompt_len / (e2e_prefill_ms / 1e3), 1),
                "h2d_bytes_per_step": 0, "d2h_bytes_per_step": prompts_n * 8,
                "h2d_bytes_prompts": prompts_n * prompt_len * 8, "ms_per_step": round(e2e_decode_ms / new_tokens, 4)},
        "gpu_launches": int(launches), "clocks": clocks,
        "config": {"model": preset_name, "prompts_per_gpu": prompts_n, "prompt_len": prompt_len,
                   "new_tokens": new_tokens, "page_size": 16, "dtype": "bf16", "sampling": "greedy",
                   "parallelism": f"{world} replicas", "short_window": cfg.short_window,
                   "l2": "a decode step streams ~5 GB of weights and K/V, far more than the 126 MB L2"}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="d20")
    ap.add_argument("--prompts", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--new-tokens", type=int, default=256)
    ap.add_argument("--no-graph", action="store_true")
    args = ap.parse_args()
    doc = run(args.preset, args.prompts, args.prompt_len, args.new_tokens, use_graph=not args.no_graph)
    if doc is not None:
        print(json.dumps(doc))
    if torch.distributed.is_available() and torch.distributed.is_initialized():
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
