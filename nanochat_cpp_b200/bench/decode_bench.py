"""Batched KV-cache inference benchmark: prefill tok/s, decode tok/s and p50 per-token latency.

    python -m nanochat_cpp_b200.bench.decode_bench --preset d20 --prompts 64 --prompt-len 512 --new-tokens 256

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
    dev = torch.device("cuda")
    model = GPT(cfg, dev, torch.bfloat16, seed=0)
    eng = InferenceEngine(model, use_cuda_graph=not args.no_graph)
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, cfg.vocab_size, (args.prompts, args.prompt_len), generator=g).to(dev)
    cache = eng.new_cache(args.prompts, args.prompt_len + args.new_tokens + 1)
    # warm-up (also builds tensor maps and the decode graph)
    logits = eng.prefill(cache, prompts)
    for _ in range(3):
        logits = eng.decode_graphed(cache, logits.argmax(-1))
    torch.cuda.synchronize()
    cache.reset()
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
        logits = eng.decode_graphed(cache, nxt)
        nxt = logits.argmax(-1)
        b.record()
        b.synchronize()
        lat.append(a.elapsed_time(b))
    from ..ops import cuda as K
    K.check_status()
    total_ms = sum(lat)
    print(json.dumps({
        "metric": "decode_tokens_per_sec", "value": round(args.prompts * args.new_tokens / (total_ms / 1e3), 1),
        "unit": "tokens/s", "prefill_tokens_per_sec": round(args.prompts * args.prompt_len / (prefill_ms / 1e3), 1),
        "p50_token_latency_ms": round(statistics.median(lat), 4), "prefill_ms": round(prefill_ms, 3),
        "cuda_graph": bool(eng._graph is not None), "kv_cache_gb": round(cache.bytes() / 1e9, 3),
        "config": {"model": args.preset, "prompts": args.prompts, "prompt_len": args.prompt_len,
                   "new_tokens": args.new_tokens, "page_size": 16, "dtype": "bf16", "sampling": "greedy"}}))


if __name__ == "__main__":
    main()
