"""Training step and loop.

The step is the reference's (`src/train.cc:792-945`): zero the gradients, run `grad_accum`
forward/backward micro-batches scaled by `1/(grad_accum * world)`, synchronise gradients across ranks,
take one optimizer step, and log `step | loss | lr | grad_norm | tok/s | mfu | ...` on logging steps.
Nothing in the step reads the device: the loss stays on the device and is fetched only when a caller
asks for it, so non-logging steps are fully asynchronous.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Iterable, List, Optional, Sequence, Tuple

import torch

from ..config import Config
from ..models import GPT
from ..optim import Optimizer, OptimizerConfig, SchedulerConfig
from . import mfu as perf


@dataclass
class TrainConfig:
    batch: int = 8
    grad_accum: int = 1
    num_iterations: int = 100
    log_every: int = 10
    eval_every: int = 0
    save_every: int = 0
    eval_steps: int = 10
    seed: int = 42
    checkpoint: str = ""
    resume: str = ""
    log: str = ""
    dtype: str = "bf16"
    head_chunk_rows: int = 8192
    optim: OptimizerConfig = field(default_factory=OptimizerConfig)
    sched: SchedulerConfig = field(default_factory=SchedulerConfig)


class Trainer:
    """One rank of a (possibly data-parallel) training job."""

    def __init__(self, cfg: Config, tc: TrainConfig, device="cuda", dp=None, model: Optional[GPT] = None):
        self.cfg, self.tc = cfg, tc
        self.device = torch.device(device)
        dtype = torch.bfloat16 if tc.dtype == "bf16" else torch.float32
        self.model = model or GPT(cfg, self.device, dtype, seed=tc.seed, head_chunk_rows=tc.head_chunk_rows,
                                  allocator=None if dp is None else dp.allocator())
        if tc.sched.num_iterations == 0:
            tc.sched.num_iterations = tc.num_iterations
        self.dp = dp
        self.world = 1 if dp is None else dp.world_size
        if dp is not None:
            dp.prepare(self.model.params)
        self.optimizer = Optimizer(self.model.params, tc.optim, tc.sched,
                                   owned=None if dp is None else dp.owned,
                                   adamw_slices=None if dp is None else dp.slices)
        if dp is not None:
            dp.attach(self.model, self.optimizer)
        self.step_count = 0
        self.last_loss: Optional[torch.Tensor] = None

    @torch.no_grad()
    def train_step(self, micro_batches: Sequence[Tuple[torch.Tensor, torch.Tensor]]) -> torch.Tensor:
        """`micro_batches`: `grad_accum` pairs of (tokens [B,T], targets [B,T]) already on the device.
        Returns the mean micro-batch loss as a 0-d device tensor."""
        m = self.model
        accum = len(micro_batches)
        scale = 1.0 / (accum * self.world)
        if self.dp is not None:
            self.dp.begin_step(self.step_count + 1)
        m.zero_grad()
        total = None
        for k, (tokens, targets) in enumerate(micro_batches):
            if self.dp is not None:
                self.dp.set_last_micro(k == accum - 1)
            loss = m.forward_backward(tokens, targets, grad_scale=scale)
            total = loss if total is None else total + loss
        self.step_count += 1
        if self.dp is not None:
            self.dp.finish_step(self.step_count)
        else:
            self.optimizer.step(self.step_count)
        self.last_loss = total / accum
        return self.last_loss

    def tokens_per_step(self) -> int:
        return self.tc.batch * self.cfg.seq_len * self.tc.grad_accum * self.world


def format_log_line(step: int, loss: float, lr: float, grad_norm: float, tok_s: float, mfu_v: float,
                    model_tflops: float, optim_tflops: float, step_ms: float, data_ms: float = 0.0,
                    fwd_ms: float = 0.0, bwd_ms: float = 0.0, sync_ms: float = 0.0, opt_ms: float = 0.0,
                    eval_ms: float = 0.0) -> str:
    """One text line per logged step, fields in the reference's order (`src/train.cc:74-101`)."""
    return (f"step {step:6d} | loss {loss:.6f} | lr {lr:.6g} | grad_norm {grad_norm:.4f} | tok/s {tok_s:.0f} | "
            f"mfu {mfu_v:.4f} | model_tflops {model_tflops:.1f} | optim_tflops {optim_tflops:.2f} | "
            f"step_ms {step_ms:.2f} | data_ms {data_ms:.2f} | fwd_ms {fwd_ms:.2f} | bwd_ms {bwd_ms:.2f} | "
            f"sync_ms {sync_ms:.2f} | opt_ms {opt_ms:.2f} | eval_ms {eval_ms:.2f}")
