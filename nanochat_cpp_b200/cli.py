"""Command line: `python -m nanochat_cpp_b200.cli <train|eval|generate|score|sft|rl_worker|rl_step|roofline|
eval_bench|tok_train|dist> [flags]`.

Sub-commands and flag names follow the reference binary `nanochat_cli` (src/commands.cc, src/train_command.cc:27-61,
src/generate_command.cc:37-50, src/eval_command.cc:42-54, src/score_command.cc:70-74, src/sft_command.cc:82-112,
src/rl_worker_command.cc:197-205, src/rl_step_command.cc:216-219, src/roofline_command.cc:38-54,
src/eval_bench_command.cc:39-44). Multi-GPU runs are launched with `dist --world-size N -- <sub-command ...>`
(one process per GPU) and read RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT, or the reference's
NANOCHAT_RANK / NANOCHAT_WORLD_SIZE / NANOCHAT_MASTER_ADDR / NANOCHAT_MASTER_PORT.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time
from typing import List, Optional

import numpy as np


# ------------------------------------------------------------------------------------------ shared flags
def _model_flags(ap: argparse.ArgumentParser) -> None:
    g = ap.add_argument_group("model")
    g.add_argument("--preset-model", default="", help="tiny | d12 | d20 | d26")
    g.add_argument("--layers", type=int, default=12)
    g.add_argument("--heads", type=int, default=6)
    g.add_argument("--kv-heads", type=int, default=0, help="0 = same as --heads")
    g.add_argument("--hidden", type=int, default=768)
    g.add_argument("--seq", type=int, default=2048)
    g.add_argument("--vocab", type=int, default=32768)
    g.add_argument("--padded-vocab", type=int, default=0, help="0 = vocab rounded up to a multiple of 64")
    g.add_argument("--rope-base", type=float, default=100000.0)
    g.add_argument("--window-pattern", default="SSSL")
    g.add_argument("--short-window", type=int, default=0, help="0 = ceil(seq/4/128)*128")
    g.add_argument("--no-value-embedding", action="store_true")


def _config(a):
    from .config import Config, preset
    if a.preset_model:
        cfg = preset(a.preset_model)
        if "--seq" in sys.argv:
            cfg.seq_len = a.seq
        return cfg
    pv = a.padded_vocab or (a.vocab + 63) // 64 * 64
    cfg = Config(num_layers=a.layers, num_heads=a.heads, num_kv_heads=a.kv_heads or a.heads, hidden_dim=a.hidden,
                 seq_len=a.seq, vocab_size=a.vocab, padded_vocab_size=pv, rope_base=a.rope_base,
                 window_pattern=a.window_pattern, value_embedding=not a.no_value_embedding,
                 short_window_override=a.short_window)
    cfg.validate()
    return cfg


def _device(name: str):
    import torch
    if name in ("", "auto"):
        if torch.cuda.is_available():
            return torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        return torch.device("cpu")
    return torch.device(name)


def _dist_env(a) -> tuple:
    env = os.environ
    rank = a.rank if getattr(a, "rank", -1) >= 0 else int(env.get("RANK", env.get("NANOCHAT_RANK", "0")))
    world = a.world_size if getattr(a, "world_size", 0) > 0 else int(env.get("WORLD_SIZE",
                                                                               env.get("NANOCHAT_WORLD_SIZE", "1")))
    return rank, world


def _init_dp(a, device):
    rank, world = _dist_env(a)
    if world <= 1:
        return None
    import torch
    import torch.distributed as dist
    from .parallel import DataParallel
    addr = getattr(a, "master", "") or os.environ.get("MASTER_ADDR", os.environ.get("NANOCHAT_MASTER_ADDR",
                                                                                     "127.0.0.1"))
    port = getattr(a, "port", 0) or int(os.environ.get("MASTER_PORT", os.environ.get("NANOCHAT_MASTER_PORT", "29500")))
    if not dist.is_initialized():
        backend = "nccl" if device.type == "cuda" else "gloo"
        if device.type == "cuda":
            torch.cuda.set_device(device)
        dist.init_process_group(backend, init_method=f"tcp://{addr}:{port}", rank=rank, world_size=world)
    transport = os.environ.get("NANOCHAT_DP_TRANSPORT", "fused" if device.type == "cuda" else "nccl")
    return DataParallel(rank, world, transport=transport, device=device)


def _loaders(a, cfg, rank, world, batch):
    from .data import native
    tok = native.Tokenizer.load(a.tokenizer) if a.tokenizer else None
    kw = dict(batch=batch, seq=cfg.seq_len, buffer_docs=a.buffer_docs)
    train = val = None
    if getattr(a, "train_parquet", ""):
        train = native.DataLoader.from_parquet(a.train_parquet.split(","), tok, text_column=a.text_column, rank=rank,
                                               world=world, **kw)
    elif getattr(a, "synthetic", False) or not getattr(a, "val_parquet", ""):
        train = native.DataLoader.zipf(cfg.vocab_size, batch, cfg.seq_len, seed=a.seed + rank)
    if getattr(a, "val_parquet", ""):
        val = native.DataLoader.from_parquet(a.val_parquet.split(","), tok, text_column=a.text_column, rank=rank,
                                             world=world, **kw)
    return tok, train, val


# ------------------------------------------------------------------------------------------ train
def _train_parser(sub):
    ap = sub.add_parser("train", help="pretraining")
    _model_flags(ap)
    ap.add_argument("--preset", default="", help="track3: the reference's three-GPU-hour baseline settings")
    for f in ("--train-parquet", "--val-parquet", "--tokenizer", "--checkpoint", "--resume", "--log", "--metrics-dir"):
        ap.add_argument(f, default="")
    ap.add_argument("--text-column", default="text")
    ap.add_argument("--tokenizer-threads", type=int, default=1)
    ap.add_argument("--buffer-docs", type=int, default=1000)
    ap.add_argument("--synthetic", action="store_true", help="Zipf token stream instead of parquet shards")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--grad-accum", type=int, default=1)
    ap.add_argument("--cuda-graph", default="auto", choices=["auto", "on", "off"],
                    help="replay micro-batches from a CUDA graph (auto: launch-bound shapes with grad-accum >= 2)")
    ap.add_argument("--num-iterations", type=int, default=100)
    ap.add_argument("--log-every", type=int, default=10)
    ap.add_argument("--eval-every", type=int, default=0)
    ap.add_argument("--save-every", type=int, default=0)
    ap.add_argument("--eval-steps", type=int, default=10)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--device", default="auto")
    ap.add_argument("--dtype", default="", help="bf16 | fp32 (default bf16 on a GPU)")
    ap.add_argument("--hw-check", default="auto", choices=["auto", "on", "off"])
    ap.add_argument("--rank", type=int, default=-1)
    ap.add_argument("--world-size", type=int, default=0)
    ap.add_argument("--master", default="")
    ap.add_argument("--port", type=int, default=0)
    o = ap.add_argument_group("optimizer")
    o.add_argument("--embedding-lr", type=float, default=0.2)
    o.add_argument("--unembedding-lr", type=float, default=0.004)
    o.add_argument("--matrix-lr", type=float, default=0.02)
    o.add_argument("--scalar-lr", type=float, default=0.5)
    o.add_argument("--weight-decay", type=float, default=0.0)
    o.add_argument("--weight-decay-base", type=float, default=0.0)
    o.add_argument("--clip", type=float, default=1.0)
    o.add_argument("--adam-eps", type=float, default=1e-10)
    o.add_argument("--muon-ns-steps", type=int, default=5)
    o.add_argument("--muon-beta2", type=float, default=0.9)
    s = ap.add_argument_group("schedule")
    s.add_argument("--warmup-steps", type=int, default=0)
    s.add_argument("--warmdown-ratio", type=float, default=0.65)
    s.add_argument("--final-lr-frac", type=float, default=0.0)
    s.add_argument("--muon-momentum-warmup-steps", type=float, default=400.0)
    s.add_argument("--muon-momentum-start", type=float, default=0.85)
    s.add_argument("--muon-momentum-peak", type=float, default=0.97)
    s.add_argument("--muon-momentum-final", type=float, default=0.90)
    ap.set_defaults(fn=cmd_train)


def cmd_train(a) -> int:
    import torch
    from .eval import token_bytes_table
    from .optim import OptimizerConfig, SchedulerConfig
    from .train.loop import TrainConfig, Trainer
    cfg = _config(a)
    dev = _device(a.device)
    dp = _init_dp(a, dev)
    rank, world = (0, 1) if dp is None else (dp.rank, dp.world_size)
    dtype = a.dtype or ("bf16" if dev.type == "cuda" else "fp32")
    tc = TrainConfig(batch=a.batch, grad_accum=a.grad_accum, num_iterations=a.num_iterations, log_every=a.log_every,
                     eval_every=a.eval_every, save_every=a.save_every, eval_steps=a.eval_steps, seed=a.seed,
                     checkpoint=a.checkpoint, resume=a.resume, log=a.log, dtype=dtype,
                     optim=OptimizerConfig(unembedding_lr=a.unembedding_lr, embedding_lr=a.embedding_lr,
                                           matrix_lr=a.matrix_lr, scalar_lr=a.scalar_lr, weight_decay=a.weight_decay,
                                           muon_ns_steps=a.muon_ns_steps, muon_beta2=a.muon_beta2,
                                           adam_eps=a.adam_eps, clip=a.clip),
                     sched=SchedulerConfig(num_iterations=a.num_iterations, warmup_steps=a.warmup_steps,
                                           warmdown_ratio=a.warmdown_ratio, final_lr_frac=a.final_lr_frac,
                                           weight_decay_base=a.weight_decay_base or a.weight_decay,
                                           muon_momentum_warmup_steps=a.muon_momentum_warmup_steps,
                                           muon_momentum_start=a.muon_momentum_start,
                                           muon_momentum_peak=a.muon_momentum_peak,
                                           muon_momentum_final=a.muon_momentum_final))
    tc.cuda_graph = getattr(a, "cuda_graph", "auto")
    if a.hw_check == "on" or (a.hw_check == "auto" and dev.type == "cuda"):
        from .hwgate import run_hardware_gate
        ok, report = run_hardware_gate(dev)
        if rank == 0:
            print(f"[nanochat] hardware gate: {'pass' if ok else 'FAIL'} ({len(report)} checks)")
        if not ok:
            for r in report:
                if not r["ok"]:
                    print(f"[nanochat]   {r['name']}: err {r['err']:.3g} > tol {r['tol']:.3g}")
            return 3
    tok, train, val = _loaders(a, cfg, rank, world, a.batch)
    trainer = Trainer(cfg, tc, device=dev, dp=dp)
    if rank == 0:
        from .perf import RooflinePlan, estimate
        est = estimate(cfg, RooflinePlan(batch=a.batch, grad_accum=a.grad_accum, world_size=world,
                                         muon_ns_steps=a.muon_ns_steps))
        print(f"[nanochat] params {trainer.model.num_params():,} | device {dev} x{world} | dtype {dtype} | "
              f"roofline {est.tokens_per_second:.0f} tok/s ({est.step_seconds * 1e3:.1f} ms/step)")
    if a.resume:
        at = trainer.resume(a.resume, train)
        if rank == 0:
            print(f"[nanochat] resumed {a.resume} at step {at}")
    table = token_bytes_table(tok) if tok is not None else None
    trainer.run(train, val, token_bytes=table, metrics_dir=a.metrics_dir)
    if dev.type == "cuda":
        from .ops import cuda as K
        K.check_status(dev)
    return 0


# ------------------------------------------------------------------------------------------ model loading
def _load_model(path: str, device, a=None, dtype=None):
    """A checkpoint when `path` is given, else a seeded random model of the flag configuration."""
    import torch
    from .models import GPT
    from .train.checkpointer import load_checkpoint
    dtype = dtype or (torch.bfloat16 if device.type == "cuda" else torch.float32)
    if path:
        model, meta = load_checkpoint(path, device=device, dtype=dtype)
        return model, meta
    return GPT(_config(a), device, dtype, seed=getattr(a, "seed", 0)), {}


# ------------------------------------------------------------------------------------------ eval
def _eval_parser(sub):
    ap = sub.add_parser("eval", help="bits per byte on parquet shards")
    _model_flags(ap)
    for f in ("--train-parquet", "--val-parquet", "--tokenizer", "--model"):
        ap.add_argument(f, default="")
    ap.add_argument("--text-column", default="text")
    ap.add_argument("--tokenizer-threads", type=int, default=1)
    ap.add_argument("--buffer-docs", type=int, default=1000)
    ap.add_argument("--steps", type=int, default=0)
    ap.add_argument("--split-tokens", type=int, default=0, help="token budget per split (steps = tokens / (batch*seq))")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--device", default="auto")
    ap.add_argument("--synthetic", action="store_true")
    ap.set_defaults(fn=cmd_eval)


def cmd_eval(a) -> int:
    from .eval import eval_bpb, token_bytes_table
    dev = _device(a.device)
    model, _ = _load_model(a.model, dev, a)
    cfg = model.cfg
    if "--seq" in sys.argv:
        cfg.seq_len = a.seq
    tok, train, val = _loaders(a, cfg, 0, 1, a.batch)
    table = token_bytes_table(tok) if tok is not None else None
    steps = a.steps or (a.split_tokens // (a.batch * cfg.seq_len) if a.split_tokens else 10)
    out = {}
    for name, ld in (("train", train if a.train_parquet or a.synthetic else None), ("val", val)):
        if ld is not None:
            out[name] = eval_bpb(model, ld, max(steps, 1), table)
            print(f"{name} bpb {out[name]:.6f}")
    return 0 if out else 2


# ------------------------------------------------------------------------------------------ generate
def _generate_parser(sub):
    ap = sub.add_parser("generate", help="sample continuations")
    _model_flags(ap)
    for f in ("--model", "--tokenizer", "--prompt", "--text-file", "--tokens", "--prompt-file", "--out"):
        ap.add_argument(f, default="")
    ap.add_argument("--max-tokens", type=int, default=64)
    ap.add_argument("--num-samples", type=int, default=1)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--stop-id", type=int, default=-1)
    ap.add_argument("--bos-id", type=int, default=-1)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--device", default="auto")
    ap.set_defaults(fn=cmd_generate)


def cmd_generate(a) -> int:
    import torch
    from .data import native
    from .inference import GenerateParams, InferenceEngine, generate_multi
    dev = _device(a.device)
    model, _ = _load_model(a.model, dev, a)
    tok = native.Tokenizer.load(a.tokenizer) if a.tokenizer else None
    prompts: List[List[int]] = []
    if a.tokens:
        prompts.append([int(x) for x in a.tokens.replace(",", " ").split()])
    if a.prompt_file:      # one prompt of token ids per line
        for line in open(a.prompt_file):
            if line.strip():
                prompts.append([int(x) for x in line.replace(",", " ").split()])
    text = a.prompt or (open(a.text_file).read() if a.text_file else "")
    if text:
        if tok is None:
            print("generate: --prompt / --text-file need --tokenizer", file=sys.stderr)
            return 2
        bos = a.bos_id if a.bos_id >= 0 else tok.bos_id
        prompts.append(tok.encode(text, prepend=bos))
    if not prompts:
        print("generate: no prompt (--prompt, --text-file, --tokens or --prompt-file)", file=sys.stderr)
        return 2
    eng = InferenceEngine(model)
    params = GenerateParams(num_samples=a.num_samples, max_tokens=a.max_tokens, temperature=a.temperature,
                            top_k=a.top_k, seed=a.seed, stop_id=a.stop_id, bos_id=a.bos_id)
    rows = []
    by_len = {}
    for i, p in enumerate(prompts):                # prompts of one length decode as one batch
        by_len.setdefault(len(p), []).append(i)
    results = [None] * len(prompts)
    for L, idx in by_len.items():
        seqs = generate_multi(eng, torch.tensor([prompts[i] for i in idx]), params)
        for k, i in enumerate(idx):
            results[i] = seqs[k * params.num_samples:(k + 1) * params.num_samples]
    sink = open(a.out, "w") if a.out else sys.stdout
    for i, group in enumerate(results):
        for s, seq in enumerate(group):
            new = [t for t, m in zip(seq.tokens, seq.mask) if m]
            rec = dict(prompt=i, sample=s, tokens=seq.tokens, mask=seq.mask)
            if tok is not None:
                rec["text"] = tok.decode(new)
            print(json.dumps(rec), file=sink)
    if a.out:
        sink.close()
    return 0


# ------------------------------------------------------------------------------------------ score
def _score_parser(sub):
    ap = sub.add_parser("score", help="per-position nll / argmax / focus logits over a NANOEVL1 fixture")
    _model_flags(ap)
    ap.add_argument("--fixture", required=True)
    ap.add_argument("--out", default="")
    ap.add_argument("--model", default="")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--device", default="auto")
    ap.set_defaults(fn=cmd_score)


def _model_from_fixture(recs, device, dtype=None):
    """A fixture may carry its own model (config/* + param/* records)."""
    import torch
    from .config import Config
    from .models import GPT
    g = lambda k: int(recs["config/" + k][0])
    cfg = Config(num_layers=g("layers"), num_heads=g("heads"), num_kv_heads=g("kv_heads"), hidden_dim=g("embd"),
                 seq_len=g("seq"), vocab_size=g("vocab"), padded_vocab_size=g("padded_vocab"), rope_base=100000.0,
                 window_pattern=bytes(recs["config/window_pattern"]).decode())
    m = GPT(cfg, device, dtype or torch.float32, init=False)
    m.load_state_dict({s.name: torch.from_numpy(np.array(recs["param/" + s.name])).reshape(s.shape)
                       for s in m.params.specs})
    return m


def cmd_score(a) -> int:
    from .data.record_file import read_records, write_records
    from .eval import score_batch
    dev = _device(a.device)
    magic, recs = read_records(a.fixture)
    if a.model:
        model, _ = _load_model(a.model, dev, a)
    elif any(k.startswith("param/") for k in recs):
        model = _model_from_fixture(recs, dev)
    else:
        model, _ = _load_model("", dev, a)
    tokens, lengths = np.array(recs["input/tokens"]), np.array(recs["input/lengths"])
    focus = None
    if "input/focus_positions" in recs:
        pos, off, ids = recs["input/focus_positions"], recs["input/focus_offsets"], recs["input/focus_ids"]
        focus = [(int(pos[b]), [int(x) for x in ids[off[b]:off[b + 1]]]) if pos[b] >= 0 else None
                 for b in range(tokens.shape[0])]
    res = score_batch(model, tokens, lengths, focus)
    offs = np.cumsum([0] + [len(r.focus_logits) for r in res]).astype(np.int32)
    out = {"result/nll": np.array([r.nll for r in res], dtype=np.float32),
           "result/argmax": np.array([r.argmax for r in res], dtype=np.int32),
           "result/focus_offsets": offs,
           "result/focus_logits": np.array([x for r in res for x in r.focus_logits], dtype=np.float32)}
    if a.out:
        write_records(a.out, "NANOEVL1", out)
    else:
        for b, r in enumerate(res):
            n = int(lengths[b]) - 1
            print(f"row {b}: mean nll {float(np.mean(r.nll[:n])) if n > 0 else 0.0:.6f} focus {r.focus_logits}")
    return 0


# ------------------------------------------------------------------------------------------ sft
def _sft_parser(sub):
    ap = sub.add_parser("sft", help="supervised fine-tuning over a packed NCSFT001 shard")
    ap.add_argument("--rows", "--shard", dest="rows", required=True)
    ap.add_argument("--warm-start", default="")
    ap.add_argument("--resume", default="")
    ap.add_argument("--val-rows", default="")
    ap.add_argument("--token-bytes", default="", help="record file with an int32 `token_bytes` record")
    ap.add_argument("--checkpoint", default="")
    ap.add_argument("--num-iterations", type=int, default=100)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--grad-accum", type=int, default=1)
    ap.add_argument("--eval-every", type=int, default=200)
    ap.add_argument("--eval-tokens", type=int, default=40 * 524288)
    ap.add_argument("--chatcore-every", type=int, default=200)
    ap.add_argument("--seq", type=int, default=0)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--device", default="auto")
    ap.set_defaults(fn=cmd_sft)


def cmd_sft(a) -> int:
    import torch
    from .data.record_file import read_records
    from .optim import Optimizer
    from .post import SftConfig, load_sft_shard, run_sft, sft_optimizer_config, sft_scheduler_config
    from .train.checkpointer import load_checkpoint, save_checkpoint
    dev = _device(a.device)
    shard = load_sft_shard(a.rows)
    if a.seq and a.seq != shard.seq:
        print(f"sft: the shard has seq {shard.seq}, the run asked for {a.seq}", file=sys.stderr)
        return 2
    src = a.warm_start or a.resume
    if not src:
        print("sft: --warm-start or --resume is required", file=sys.stderr)
        return 2
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    model, meta = load_checkpoint(src, device=dev, dtype=dtype)
    opt = Optimizer(model.params, sft_optimizer_config(), sft_scheduler_config(a.num_iterations))
    load_checkpoint(src, model, opt)
    first = 1
    if a.resume:
        first = int(meta.get("step", 0)) + 1
    else:
        opt.step_count = 0          # warm start: weights and moments, fresh schedule
    val = load_sft_shard(a.val_rows) if a.val_rows else None
    table = None
    if a.token_bytes:
        table = np.array(read_records(a.token_bytes)[1]["token_bytes"])
    logs = run_sft(model, opt, shard, SftConfig(num_iterations=a.num_iterations, batch=a.batch,
                                                grad_accum=a.grad_accum, eval_every=a.eval_every,
                                                eval_tokens=a.eval_tokens, chatcore_every=a.chatcore_every,
                                                first_step=first), val_shard=val, token_bytes=table)
    if a.checkpoint:
        save_checkpoint(a.checkpoint, model, opt, step=logs[-1].step if logs else 0, stage="sft")
    return 0


# ------------------------------------------------------------------------------------------ rl
def _rl_parsers(sub):
    ap = sub.add_parser("rl_step", help="replay the policy-gradient steps of a fixture")
    ap.add_argument("--fixture", required=True)
    ap.add_argument("--out", default="")
    ap.add_argument("--device", default="cpu")
    ap.set_defaults(fn=cmd_rl_step)
    ap = sub.add_parser("rl_worker", help="persistent worker: line protocol on stdin/stdout, or a fixture replay")
    _model_flags(ap)
    ap.add_argument("--fixture", default="")
    ap.add_argument("--checkpoint", default="")
    ap.add_argument("--steps", type=int, default=0)
    ap.add_argument("--out", default="")
    ap.add_argument("--save", default="")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--device", default="auto")
    ap.set_defaults(fn=cmd_rl_worker)


def _rl_optim(recs):
    from .optim import OptimizerConfig, SchedulerConfig
    o = lambda k, d: float(recs["config/opt/" + k][0]) if "config/opt/" + k in recs else d
    s = lambda k, d: float(recs["config/sched/" + k][0]) if "config/sched/" + k in recs else d
    return (OptimizerConfig(unembedding_lr=o("unembedding_lr", .004), embedding_lr=o("embedding_lr", .2),
                            matrix_lr=o("matrix_lr", .02), scalar_lr=o("scalar_lr", .5),
                            weight_decay=o("weight_decay", 0.0), clip=o("clip", 0.0), adam_eps=o("adam_eps", 1e-10),
                            muon_ns_steps=int(o("muon_ns_steps", 5)), muon_beta2=o("muon_beta2", .9)),
            SchedulerConfig(num_iterations=int(s("num_iterations", 0)), warmup_steps=int(s("warmup_steps", 0)),
                            warmdown_ratio=s("warmdown_ratio", 0.0), final_lr_frac=s("final_lr_frac", 0.0),
                            weight_decay_base=s("weight_decay_base", 0.0),
                            muon_momentum_warmup_steps=s("muon_momentum_warmup_steps", 0.0),
                            muon_momentum_start=s("muon_momentum_start", .95),
                            muon_momentum_peak=s("muon_momentum_peak", .95),
                            muon_momentum_final=s("muon_momentum_final", .95)))


def _replay_rl(recs, device, steps=0, through_worker=False):
    from .optim import Optimizer
    from .post import RlWorker, rl_step
    model = _model_from_fixture(recs, device)
    oc, sc = _rl_optim(recs)
    opt = Optimizer(model.params, oc, sc)
    n = steps or int(recs["config/steps"][0])
    passes, per = int(recs["config/num_passes"][0]), int(recs["config/examples_per_rank"][0])
    out = {}
    worker = RlWorker(model, opt)
    for k in range(n):
        tok, tgt = np.array(recs[f"rollout/{k}/tokens"]), np.array(recs[f"rollout/{k}/targets"])
        adv = np.array(recs[f"rollout/{k}/advantages"])
        if through_worker:
            res = worker.advantage(tok.ravel().tolist(), tgt.ravel().tolist(), adv.ravel().tolist(), tok.shape[0],
                                   tok.shape[1], passes, per)
        else:
            res = rl_step(model, opt, tok, tgt, adv, passes, per, k + 1)
        out[f"step/{k}/loss"] = np.array([res.loss], dtype=np.float32)
        out[f"step/{k}/grad_norm"] = np.array([res.grad_norm], dtype=np.float32)
        out[f"step/{k}/valid_targets"] = np.array([res.valid_targets], dtype=np.int32)
        out[f"step/{k}/divisor"] = np.array([res.divisor], dtype=np.int64)
        print(f"rl: step {k + 1} loss {res.loss:.6f} grad_norm {res.grad_norm:.6f} valid {res.valid_targets} "
              f"divisor {res.divisor}", file=sys.stderr)
    for s in model.params.specs:
        out["param/" + s.name] = model.params.m(s.name).detach().cpu().numpy()
    return worker, out


def cmd_rl_step(a) -> int:
    from .data.record_file import read_records, write_records
    _, recs = read_records(a.fixture)
    _, out = _replay_rl(recs, _device(a.device))
    if a.out:
        write_records(a.out, "NANOORC1", out)
    return 0


def cmd_rl_worker(a) -> int:
    from .data.record_file import read_records, write_records
    from .optim import Optimizer
    from .post import RlWorker
    dev = _device(a.device)
    if a.fixture:
        _, recs = read_records(a.fixture)
        worker, out = _replay_rl(recs, dev, a.steps, through_worker=True)
        if a.out:
            write_records(a.out, "NANOORC1", out)
        if a.save:
            worker.save(a.save)
        return 0
    model, meta = _load_model(a.checkpoint, dev, a)
    opt = Optimizer(model.params)
    step = 0
    if a.checkpoint:
        from .train.checkpointer import load_checkpoint
        load_checkpoint(a.checkpoint, model, opt)
        step = int(meta.get("step", 0)) if meta.get("stage", 0) == 2 else 0
    worker = RlWorker(model, opt, step=step)
    rc = worker.serve(sys.stdin, sys.stdout)
    if a.save:
        worker.save(a.save)
    return rc


# ------------------------------------------------------------------------------------------ roofline / benches
def _perf_parsers(sub):
    ap = sub.add_parser("roofline", help="analytic step-time model")
    _model_flags(ap)
    ap.add_argument("--device", default="b200")
    ap.add_argument("--precision", default="bf16")
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--grad-accum", type=int, default=1)
    ap.add_argument("--devices", type=int, default=1)
    ap.add_argument("--tokens", type=int, default=0)
    ap.add_argument("--link-gbps", type=float, default=0.0)
    ap.add_argument("--latency-us", type=float, default=5.0)
    ap.add_argument("--overlap", type=float, default=0.0)
    ap.add_argument("--muon-ns-steps", type=int, default=5)
    ap.add_argument("--json", action="store_true")
    ap.set_defaults(fn=cmd_roofline)
    ap = sub.add_parser("eval_bench", help="time the evaluation forward (loss over a batch)")
    _model_flags(ap)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--device", default="auto")
    ap.set_defaults(fn=cmd_eval_bench)


def cmd_roofline(a) -> int:
    from .perf import RooflinePlan, estimate, format_report, report_json
    e = estimate(_config(a), RooflinePlan(device=a.device, precision=a.precision, batch=a.batch,
                                          grad_accum=a.grad_accum, world_size=a.devices, total_tokens=a.tokens,
                                          link_gbps=a.link_gbps, latency_us=a.latency_us, overlap=a.overlap,
                                          muon_ns_steps=a.muon_ns_steps))
    sys.stdout.write(report_json(e) + "\n" if a.json else format_report(e))
    return 0


def cmd_eval_bench(a) -> int:
    import torch
    from .models import GPT
    dev = _device(a.device)
    cfg = _config(a)
    model = GPT(cfg, dev, torch.bfloat16 if dev.type == "cuda" else torch.float32, seed=a.seed)
    g = torch.Generator().manual_seed(a.seed)
    tok = torch.randint(0, cfg.vocab_size, (a.batch, cfg.seq_len), generator=g).to(dev)
    tgt = torch.roll(tok, -1, 1)
    times = []
    for i in range(a.warmup + a.iters):
        if dev.type == "cuda":
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            model.forward_loss(tok, tgt)
            e1.record()
            e1.synchronize()
            ms = e0.elapsed_time(e1)
        else:
            t0 = time.perf_counter()
            model.forward_loss(tok, tgt)
            ms = (time.perf_counter() - t0) * 1e3
        if i >= a.warmup:
            times.append(ms)
    times.sort()
    rep = dict(schema="nanochat.bench.v3", family="eval_forward", device=str(dev), precision="bf16"
               if dev.type == "cuda" else "fp32", shape=f"b{a.batch}-s{cfg.seq_len}-L{cfg.num_layers}-h{cfg.hidden_dim}",
               iters=a.iters, warmup=a.warmup, min_ms=times[0], median_ms=times[len(times) // 2],
               tokens_per_second=a.batch * cfg.seq_len / (times[len(times) // 2] / 1e3))
    print(json.dumps(rep) if a.json else
          f"eval forward: min {rep['min_ms']:.3f} ms  median {rep['median_ms']:.3f} ms  "
          f"{rep['tokens_per_second']:.0f} tok/s")
    return 0


# ------------------------------------------------------------------------------------------ tokenizer / launcher
def _misc_parsers(sub):
    ap = sub.add_parser("tok_train", help="train a byte-level BPE tokenizer (NCTOKEN1)")
    ap.add_argument("--text", default="")
    ap.add_argument("--parquet", default="")
    ap.add_argument("--text-column", default="text")
    ap.add_argument("--vocab-size", type=int, default=32768)
    ap.add_argument("--doc-cap", type=int, default=10000)
    ap.add_argument("--max-chars", type=int, default=0)
    ap.add_argument("--out", required=True)
    ap.set_defaults(fn=cmd_tok_train)
    ap = sub.add_parser("dist", help="launch one process per GPU: dist --world-size N -- <sub-command ...>")
    ap.add_argument("--world-size", type=int, required=True)
    ap.add_argument("--master-port", type=int, default=29500)
    ap.add_argument("--max-restarts", type=int, default=0,
                    help="start the group again after a failure, resuming from --checkpoint when it exists")
    ap.add_argument("rest", nargs=argparse.REMAINDER)
    ap.set_defaults(fn=cmd_dist)


def cmd_tok_train(a) -> int:
    from .data import native
    tok = native.Tokenizer.train(text=a.text, parquet=a.parquet, text_column=a.text_column, vocab_size=a.vocab_size,
                                 doc_cap=a.doc_cap, max_chars=a.max_chars)
    tok.save(a.out)
    print(f"tok_train: vocab {tok.vocab_size} -> {a.out}")
    return 0


def cmd_dist(a) -> int:
    """Rank 0 first, then the others (the reference's launcher order, python/nanochat_cpp/cli.py:827-945); the
    children get both the torch and the NANOCHAT_* environment contract and one GPU each. The first rank that fails
    stops the group; with `--max-restarts N` the group is started again (from `--checkpoint` when it exists)."""
    from .parallel import launcher
    rest = [x for x in a.rest if x != "--"]
    if not rest:
        print("dist: nothing to launch", file=sys.stderr)
        return 2
    envs = launcher.rank_environments(a.world_size, a.master_port)

    def commands(attempt: int):
        argv = launcher.with_resume(rest, attempt)
        return [[sys.executable, "-m", "nanochat_cpp_b200.cli"] + argv for _ in range(a.world_size)]

    res = launcher.run_group(commands, envs, max_restarts=a.max_restarts)
    if res.returncode != 0:
        print(f"[nanochat] dist: rank {res.failed_rank} failed with exit code {res.returncode} "
              f"after {res.starts} start(s); the other ranks were stopped", file=sys.stderr)
    return res.returncode


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="nanochat_cli", description=__doc__.splitlines()[0])
    sub = ap.add_subparsers(dest="command", required=True)
    _train_parser(sub)
    _eval_parser(sub)
    _generate_parser(sub)
    _score_parser(sub)
    _sft_parser(sub)
    _rl_parsers(sub)
    _perf_parsers(sub)
    _misc_parsers(sub)
    from . import tools_cli
    tools_cli.register(sub)
    a = ap.parse_args(argv)
    return int(a.fn(a) or 0)


if __name__ == "__main__":
    sys.exit(main())
