"""Supervised fine-tuning over packed rows.

The loop is the reference's (`src/sft_command.cc:436-560`): rows of an `NCSFT001` shard (tokens + targets with
-1 on every position that is not an assistant token) are consumed in order and wrap around (one wrap = one
epoch); each step runs `grad_accum` micro-batches of `batch` rows scaled by 1/grad_accum; the learning rate
follows dataset progress (`lr_multiplier_for_progress` over the running maximum of done/total) instead of a
step count; the Muon momentum keeps its step-based ramp; validation is bits per byte over packed rows.
Pinned recipe (`src/sft_command.cc:63-80`): embedding lr 0.3, unembedding 0.004, matrix 0.02, scalar 0.5,
Adam eps 1e-10, every rate scaled once by init_lr_frac 0.8, no warm-up, warm-down over the last half to 0,
momentum 0.85 -> 0.95 over 300 steps.
"""
from __future__ import annotations

import sys
from dataclasses import dataclass
from typing import Callable, List, Optional

import numpy as np
import torch

from ..data import record_file
from ..eval import PackedBpb, evaluate_packed_rows
from ..models import GPT
from ..optim import Optimizer, OptimizerConfig, SchedulerConfig


@dataclass
class SftShard:
    tokens: np.ndarray   # int32 [rows, seq]
    targets: np.ndarray  # int32 [rows, seq], -1 = not trained on

    @property
    def rows(self) -> int:
        return self.tokens.shape[0]

    @property
    def seq(self) -> int:
        return self.tokens.shape[1]


def load_sft_shard(path: str) -> SftShard:
    magic, recs = record_file.read_records(path)
    if magic != "NCSFT001":
        raise ValueError(f"{path}: not an SFT shard (magic {magic!r})")
    if "tokens" not in recs or "targets" not in recs or recs["tokens"].ndim != 2 or recs["targets"].ndim != 2:
        raise ValueError("the SFT shard must hold two rank-2 records, tokens and targets")
    if recs["tokens"].shape != recs["targets"].shape:
        raise ValueError("the SFT shard records have different shapes")
    return SftShard(np.ascontiguousarray(recs["tokens"], dtype=np.int32),
                    np.ascontiguousarray(recs["targets"], dtype=np.int32))


def save_sft_shard(path: str, shard: SftShard) -> None:
    record_file.write_records(path, "NCSFT001", {"tokens": shard.tokens.astype(np.int32),
                                                 "targets": shard.targets.astype(np.int32)})


def sft_optimizer_config(clip: float = 0.0) -> OptimizerConfig:
    return OptimizerConfig(unembedding_lr=0.004, embedding_lr=0.3, matrix_lr=0.02, scalar_lr=0.5, adam_eps=1e-10,
                           init_lr_frac=0.8, clip=clip)


def sft_scheduler_config(num_iterations: int) -> SchedulerConfig:
    return SchedulerConfig(num_iterations=num_iterations, warmup_ratio=0.0, warmdown_ratio=0.5, final_lr_frac=0.0,
                           muon_momentum_warmup_steps=300.0, muon_momentum_start=0.85, muon_momentum_peak=0.95,
                           muon_momentum_final=0.95)


@dataclass
class SftConfig:
    num_iterations: int = 100
    batch: int = 1
    grad_accum: int = 1
    eval_every: int = 200
    eval_tokens: int = 40 * 524288
    chatcore_every: int = 200
    first_step: int = 1


@dataclass
class SftStepLog:
    step: int
    epoch: int
    progress: float
    lr_multiplier: float
    momentum: float
    loss: float
    grad_norm: float = 0.0
    val_bpb: Optional[float] = None


@torch.no_grad()
def run_sft(model: GPT, optimizer: Optimizer, shard: SftShard, cfg: SftConfig, *,
            val_shard: Optional[SftShard] = None, token_bytes: Optional[np.ndarray] = None,
            on_step: Optional[Callable[[SftStepLog], None]] = None, log="stderr") -> List[SftStepLog]:
    dev = model.device
    if log == "stderr":
        log = sys.stderr
    first = max(cfg.first_step, 1)
    target = max(first - 1 + cfg.num_iterations, cfg.num_iterations)
    cursor, epoch, consumed, progress = 0, 1, 0, 0.0
    logs: List[SftStepLog] = []
    for current in range(first, target + 1):
        model.zero_grad()
        loss = None
        for _ in range(cfg.grad_accum):
            idx = []
            for _ in range(cfg.batch):
                if cursor >= shard.rows:
                    cursor, epoch = 0, epoch + 1
                idx.append(cursor)
                cursor += 1
                consumed += 1
            tok = torch.as_tensor(shard.tokens[idx], device=dev).long()
            tgt = torch.as_tensor(shard.targets[idx], device=dev).long()
            loss = model.forward_backward(tok, tgt, grad_scale=1.0 / cfg.grad_accum)
        done = current - first + 1
        approx = done / cfg.num_iterations if cfg.num_iterations > 0 else consumed / max(shard.rows, 1)
        progress = min(1.0, max(progress, approx))
        mult = optimizer.scheduler.lr_multiplier_for_progress(progress)
        optimizer.set_progress_multiplier(mult)
        optimizer.step(current)
        entry = SftStepLog(current, epoch, progress, mult, optimizer.scheduler.muon_momentum(current), float(loss),
                           optimizer.grad_norm())
        if log is not None:
            print(f"sft: step {current} epoch {epoch} progress {progress:.6f} lr_multiplier {mult:.6f} "
                  f"momentum {entry.momentum:.6f} loss {entry.loss:.6f}", file=log)
        final = current == target
        if val_shard is not None and cfg.eval_every > 0 and (current % cfg.eval_every == 0 or final):
            steps = val_shard.rows // max(cfg.batch, 1)
            if cfg.eval_tokens > 0:
                steps = min(steps, cfg.eval_tokens // (cfg.batch * shard.seq))
            steps = max(steps, 1)
            table = token_bytes if token_bytes is not None else np.ones(model.cfg.padded_vocab_size, dtype=np.int32)
            bpb: PackedBpb = evaluate_packed_rows(model, val_shard.tokens, val_shard.targets, table, cfg.batch, steps)
            entry.val_bpb = bpb.bpb
            if log is not None:
                print(f"sft: eval step {current} bpb {bpb.bpb:.6f} valid_targets {bpb.valid_targets} "
                      f"target_bytes {bpb.target_bytes}", file=log)
        logs.append(entry)
        if on_step is not None:
            on_step(entry)
    return logs
