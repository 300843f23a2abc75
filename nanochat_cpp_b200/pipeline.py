"""The whole recipe as one call: base pretraining -> supervised fine-tuning -> reinforcement learning -> evaluation.

Counterpart of the reference's `pipeline.py` (python/nanochat_cpp/pipeline.py: base -> sft -> rl -> eval chain with
named profiles). Every stage reads the previous stage's checkpoint and writes its own, so a stage can be re-run
alone; stage outputs and a `pipeline.json` summary land in `workdir`.
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

PROFILES: Dict[str, dict] = {
    # a CPU smoke run: seconds
    "tiny": dict(model=dict(num_layers=2, num_heads=2, hidden_dim=64, head_dim=32, seq_len=64, window_pattern="L"),
                 base=dict(batch=4, grad_accum=1, num_iterations=8), sft=dict(num_iterations=4, batch=2, grad_accum=1),
                 rl=dict(steps=1, num_samples=2, max_tokens=8), eval=dict(steps=2, batch=2)),
    # the d20 recipe on B200s
    "big": dict(model=dict(depth=20, vocab_size=65536, seq_len=2048),
                base=dict(batch=32, grad_accum=1, num_iterations=20000),
                sft=dict(num_iterations=700, batch=8, grad_accum=4), rl=dict(steps=400, num_samples=16, max_tokens=256),
                eval=dict(steps=50, batch=16)),
}


@dataclass
class PipelineReport:
    profile: str
    base: dict = field(default_factory=dict)
    sft: dict = field(default_factory=dict)
    rl: dict = field(default_factory=dict)
    eval: dict = field(default_factory=dict)


def run_pipeline(profile: str, workdir: str, tokenizer_path: str, *, train_parquet: Sequence[str] = (),
                 val_parquet: Sequence[str] = (), sft_conversations: Optional[List[dict]] = None,
                 rl_task=None, rl_conversations: Optional[List[dict]] = None, device: Optional[str] = None,
                 stages: Sequence[str] = ("base", "sft", "rl", "eval")) -> PipelineReport:
    from . import api
    from .chat import pack_rows
    from .data import native
    from .eval import eval_bpb, token_bytes_table
    from .optim import Optimizer
    from .post import RlWorker, SftConfig, SftShard, run_sft, sft_optimizer_config, sft_scheduler_config
    from .post.rl_loop import InProcessWorker, run as run_rl
    from .train.checkpointer import load_checkpoint, save_checkpoint
    from .train.loop import TrainConfig, Trainer
    prof = PROFILES[profile]
    os.makedirs(workdir, exist_ok=True)
    dev = torch.device(device) if device else (torch.device("cuda") if torch.cuda.is_available()
                                               else torch.device("cpu"))
    dtype = "bf16" if dev.type == "cuda" else "fp32"
    tok = api.Tokenizer.load(tokenizer_path)
    cfg = api.Config(vocab_size=tok.vocab_size, **{k: v for k, v in prof["model"].items() if k != "vocab_size"})
    rep = PipelineReport(profile)
    ck = {s: os.path.join(workdir, f"{s}.ckpt") for s in ("base", "sft", "rl")}
    table = token_bytes_table(tok.handle)

    def loader(paths, batch):
        if paths:
            return native.DataLoader.from_parquet(list(paths), tok.handle, batch, cfg.seq_len)
        return native.DataLoader.zipf(cfg.vocab_size, batch, cfg.seq_len, seed=1)

    if "base" in stages:
        b = prof["base"]
        tc = TrainConfig(batch=b["batch"], grad_accum=b["grad_accum"], num_iterations=b["num_iterations"],
                         log_every=max(1, b["num_iterations"] // 4), checkpoint=ck["base"], dtype=dtype)
        trainer = Trainer(cfg, tc, device=dev)
        rep.base = trainer.run(loader(train_parquet, b["batch"]), metrics_dir=os.path.join(workdir, "base"))
    if "sft" in stages and sft_conversations:
        s = prof["sft"]
        tokens, targets = pack_rows(sft_conversations, tok, cfg.seq_len)
        model, _ = load_checkpoint(ck["base"], device=dev, dtype=torch.bfloat16 if dtype == "bf16" else torch.float32)
        opt = Optimizer(model.params, sft_optimizer_config(), sft_scheduler_config(s["num_iterations"]))
        load_checkpoint(ck["base"], model, opt)
        opt.step_count = 0
        logs = run_sft(model, opt, SftShard(tokens, targets), SftConfig(num_iterations=s["num_iterations"],
                                                                        batch=s["batch"], grad_accum=s["grad_accum"],
                                                                        eval_every=0), log=None)
        save_checkpoint(ck["sft"], model, opt, step=logs[-1].step, stage="sft")
        rep.sft = dict(steps=len(logs), first_loss=logs[0].loss, final_loss=logs[-1].loss, rows=int(tokens.shape[0]))
    if "rl" in stages and rl_task is not None and rl_conversations:
        r = prof["rl"]
        src = ck["sft"] if os.path.exists(ck["sft"]) else ck["base"]
        model, _ = load_checkpoint(src, device=dev, dtype=torch.bfloat16 if dtype == "bf16" else torch.float32)
        opt = Optimizer(model.params)
        out = run_rl(InProcessWorker(RlWorker(model, opt)), rl_task, rl_conversations, tok, num_samples=r["num_samples"],
                     steps=r["steps"], max_tokens=r["max_tokens"], checkpoint=ck["rl"])
        rep.rl = dict(steps=out.steps, losses=out.losses, mean_rewards=out.mean_rewards)
    if "eval" in stages:
        e = prof["eval"]
        last = next(p for p in (ck["rl"], ck["sft"], ck["base"]) if os.path.exists(p))
        model, _ = load_checkpoint(last, device=dev, dtype=torch.bfloat16 if dtype == "bf16" else torch.float32)
        rep.eval = dict(checkpoint=last, val_bpb=eval_bpb(model, loader(val_parquet or train_parquet, e["batch"]),
                                                          e["steps"], table))
    with open(os.path.join(workdir, "pipeline.json"), "w") as f:
        json.dump(asdict(rep), f, indent=1)
    return rep
