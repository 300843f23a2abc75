"""Learning-rate, Muon-momentum and weight-decay schedules.

Same curves as the reference `Scheduler` (`src/optim.cc:679-754`,
`include/nanochat/scheduler.h:10-30`): steps are 1-based and evaluated at `it = step-1`;
linear warm-up, constant, linear warm-down over the last `warmdown_ratio` of the run
(rounded half-to-even like Python's `round`); Muon momentum .85 -> .97 over 400 steps and
-> .90 during warm-down; cosine weight decay; and the progress-indexed SFT multiplier.
"""
from __future__ import annotations

import math
from dataclasses import dataclass


@dataclass
class SchedulerConfig:
    num_iterations: int = 0
    warmup_steps: int = 0
    warmup_ratio: float = 0.0
    warmdown_ratio: float = 0.65
    final_lr_frac: float = 0.0
    weight_decay_base: float = 0.0
    muon_momentum_warmup_steps: float = 400.0
    muon_momentum_start: float = 0.85
    muon_momentum_peak: float = 0.97
    muon_momentum_final: float = 0.90


class Scheduler:
    def __init__(self, config: SchedulerConfig):
        self.config = config

    def warmdown_iters(self) -> int:
        return int(round(float(self.config.warmdown_ratio) * float(self.config.num_iterations)))

    def lr_multiplier(self, step: int) -> float:
        c = self.config
        it = step - 1
        warmdown = self.warmdown_iters()
        if c.warmup_steps > 0 and it < c.warmup_steps:
            return (it + 1) / float(c.warmup_steps)
        if warmdown <= 0 or it <= c.num_iterations - warmdown:
            return 1.0
        progress = (c.num_iterations - it) / float(warmdown)
        return progress + (1.0 - progress) * c.final_lr_frac

    def lr_multiplier_for_progress(self, progress: float) -> float:
        c = self.config
        if c.warmup_ratio > 0.0 and progress < c.warmup_ratio:
            return (progress + 1e-8) / c.warmup_ratio
        if progress <= 1.0 - c.warmdown_ratio:
            return 1.0
        if c.warmdown_ratio <= 0.0:
            return c.final_lr_frac
        decay = (progress - (1.0 - c.warmdown_ratio)) / c.warmdown_ratio
        return 1.0 + decay * (c.final_lr_frac - 1.0)

    def muon_momentum(self, step: int) -> float:
        c = self.config
        it = step - 1
        warmdown = self.warmdown_iters()
        warmdown_start = c.num_iterations - warmdown
        if c.muon_momentum_warmup_steps > 0.0 and it < c.muon_momentum_warmup_steps:
            frac = it / c.muon_momentum_warmup_steps
            return (1.0 - frac) * c.muon_momentum_start + frac * c.muon_momentum_peak
        if warmdown > 0 and it >= warmdown_start:
            progress = (it - warmdown_start) / float(warmdown)
            return c.muon_momentum_peak * (1.0 - progress) + c.muon_momentum_final * progress
        return c.muon_momentum_peak

    def weight_decay(self, step: int) -> float:
        c = self.config
        if c.num_iterations <= 0:
            return c.weight_decay_base
        ratio = (step - 1) / float(c.num_iterations)
        return c.weight_decay_base * 0.5 * (1.0 + math.cos(math.pi * ratio))
