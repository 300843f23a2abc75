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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="d20")
    ap.add_argument("--prompts", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--new-tokens", type=int, default=256)
    ap.add_argument("--no-graph", action="store_true")
    args = ap.parse_args()
    cfg = preset(args.preset)
    import os
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    model = GPT(cfg, dev, torch.bfloat16, seed=0)
    eng = InferenceEngine(model, use_cuda_graph=not args.no_graph)
    g = torch.Generator().manual_seed(rank)       # different prompts per replica
    prompts = torch.randint(0, cfg.vocab_size, (args.prompts, args.prompt_len), generator=g).to(dev)
    cache = eng.new_cache(args.prompts, args.prompt_len + args.new_tokens + 1)
    # warm-up (also builds tensor maps and the decode graph)
    logits = eng.prefill(cache, prompts)
    nxt = logits.argmax(-1)
    for _ in range(3):
        nxt = eng.decode_graphed(cache, nxt, greedy=True)
    torch.cuda.synchronize()
    cache.reset()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    logits = eng.prefill(cache, prompts)
    e1.record()
    torch.cuda.synchronize()
    prefill_ms = e0.elapsed_time(e1)
    lat = []
    nxt = logits.argmax(-1)
    for _ in range(args.new_tokens):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        nxt = eng.decode_graphed(cache, nxt, greedy=True)     # next token ids straight from the step (greedy)
        b.record()
        b.synchronize()
        lat.append(a.elapsed_time(b))
    from ..ops import cuda as K
    K.check_status()
    total_ms = sum(lat)
    p50 = statistics.median(lat)
    if world > 1:     # replicas are independent: the job's time is the slowest replica's (device-timed, max over ranks)
        t = torch.tensor([total_ms, prefill_ms, p50], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, prefill_ms, p50 = (float(v) for v in t.tolist())
        dist.barrier()
        dist.destroy_process_group()
        if rank != 0:
            return
    print(json.dumps({
        "metric": "decode_tokens_per_sec", "n_gpus": world,
        "value": round(world * args.prompts * args.new_tokens / (total_ms / 1e3), 1),
        "unit": "tokens/s", "prefill_tokens_per_sec": round(world * args.prompts * args.prompt_len / (prefill_ms / 1e3), 1),
        "p50_token_latency_ms": round(p50, 4), "prefill_ms": round(prefill_ms, 3),
        "cuda_graph": bool(eng._graph is not None), "kv_cache_gb": round(cache.bytes() / 1e9, 3),
        "config": {"model": args.preset, "prompts_per_gpu": args.prompts, "prompt_len": args.prompt_len,
                   "new_tokens": args.new_tokens, "page_size": 16, "dtype": "bf16", "sampling": "greedy"}}))


if __name__ == "__main__":
    main()
