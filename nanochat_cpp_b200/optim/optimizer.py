"""Muon on the matrices, AdamW on embeddings / head / scalars.

Grouping, rates and arithmetic follow the reference (`src/optim.cc:154-232, 400-500`):

* AdamW groups, every rate times `sqrt(768/hidden)` where marked (*):
  lm_head (unembedding_lr*, betas .8/.96, wd .01), wte (embedding_lr*, .8/.995, wd .001),
  value_embeds (embedding_lr*/2, .8/.995, wd .01), resid (scalar_lr/100, .8/.95, wd .05),
  x0 (scalar_lr, .96/.95, wd 0), smear gate + smear/backout lambdas (0.2, .8/.95, wd 0).
* Muon groups: all remaining matrices grouped by shape in ascending (rows, cols) order,
  rate `matrix_lr * sqrt(max(1, rows/cols))`, momentum and decay from the scheduler.
* One global gradient norm over every parameter gives the clip scale `min(1, clip/norm)`.

Ownership: with data parallelism every parameter has one owner rank that keeps its fp32
master and optimizer state and computes its update; `owned` selects this rank's
parameters (None = all). The gradient-norm partial of the owned set is what a rank
contributes to the global norm.
"""
from __future__ import annotations

import contextlib
import math
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import torch

from .. import ops
from ..models.params import ParamSpec, ParamStore
from .scheduler import Scheduler, SchedulerConfig


@dataclass
class OptimizerConfig:
    unembedding_lr: float = 0.004
    embedding_lr: float = 0.2
    matrix_lr: float = 0.02
    scalar_lr: float = 0.5
    weight_decay: float = 0.0
    muon_ns_steps: int = 5
    muon_beta2: float = 0.9
    adam_eps: float = 1e-10
    clip: float = 1.0
    init_lr_frac: float = 1.0


@dataclass
class AdamWGroup:
    kind: str
    lr: float
    beta1: float
    beta2: float
    eps: float
    weight_decay: float
    params: List[ParamSpec] = field(default_factory=list)


@dataclass
class MuonGroup:
    rows: int
    cols: int
    lr: float
    params: List[ParamSpec] = field(default_factory=list)


def dmodel_lr_scale(hidden: int) -> float:
    return math.sqrt(768.0 / float(hidden))


def build_groups(store: ParamStore, cfg: OptimizerConfig):
    scale = dmodel_lr_scale(store.cfg.hidden_dim)
    f = cfg.init_lr_frac
    adamw = [
        AdamWGroup("lm_head", cfg.unembedding_lr * scale * f, 0.8, 0.96, cfg.adam_eps, 0.01),
        AdamWGroup("wte", cfg.embedding_lr * scale * f, 0.8, 0.995, cfg.adam_eps, 0.001),
        AdamWGroup("value_embed", cfg.embedding_lr * scale * 0.5 * f, 0.8, 0.995, cfg.adam_eps, 0.01),
        AdamWGroup("resid", cfg.scalar_lr * 0.01 * f, 0.8, 0.95, cfg.adam_eps, 0.05),
        AdamWGroup("x0", cfg.scalar_lr * f, 0.96, 0.95, cfg.adam_eps, 0.0),
        AdamWGroup("smear", 0.2 * f, 0.8, 0.95, cfg.adam_eps, 0.0),
    ]
    by_kind = {g.kind: g for g in adamw}
    shapes: Dict[tuple, List[ParamSpec]] = {}
    for s in store.specs:
        if s.kind in by_kind:
            by_kind[s.kind].params.append(s)
        else:
            shapes.setdefault((s.rows, s.cols), []).append(s)
    muon = []
    for (r, c) in sorted(shapes):
        lr = cfg.matrix_lr * f * math.sqrt(max(1.0, float(r) / float(c)))
        muon.append(MuonGroup(r, c, lr, shapes[(r, c)]))
    return adamw, muon


class Optimizer:
    def __init__(self, store: ParamStore, config: OptimizerConfig = None, sched: SchedulerConfig = None,
                 owned: Optional[Callable[[ParamSpec], bool]] = None,
                 adamw_slices: Optional[Dict[str, tuple]] = None):
        self.store = store
        self.config = config or OptimizerConfig()
        self.scheduler = Scheduler(sched or SchedulerConfig())
        self.adamw_groups, self.muon_groups = build_groups(store, self.config)
        self.owned = owned or (lambda s: True)
        dev = store.device
        self.state: Dict[str, Dict[str, torch.Tensor]] = {}
        self.adamw_slices = dict(adamw_slices or {})  # name -> (begin, end) owned by this rank
        for g in self.adamw_groups:
            for s in g.params:
                if self.owned(s):
                    a, b = self.adamw_slices.get(s.name, (0, s.count))
                    self.state[s.name] = dict(m=torch.zeros(max(b - a, 0), dtype=torch.float32, device=dev),
                                              v=torch.zeros(max(b - a, 0), dtype=torch.float32, device=dev))
        for g in self.muon_groups:
            lines = g.rows if g.rows >= g.cols else g.cols
            for s in g.params:
                if self.owned(s):
                    self.state[s.name] = dict(buf1=torch.zeros(s.shape, dtype=torch.float32, device=dev),
                                              buf2=torch.zeros(lines, dtype=torch.float32, device=dev))
        self._muon_scratch = {}
        self.pusher = None   # data-parallel engine: pushes updated parameters to every rank (parallel.fused)
        self.lr_multiplier_override: float = -1.0
        self.last_grad_norm: Optional[torch.Tensor] = None
        self.step_count = 0

    # ------------------------------------------------------------------
    def set_progress_multiplier(self, value: float) -> None:
        self.lr_multiplier_override = value

    def grad_norm(self) -> float:
        return 0.0 if self.last_grad_norm is None else float(self.last_grad_norm.item())

    def local_sumsq(self) -> torch.Tensor:
        """Sum of squares of this rank's owned gradients (fp64 0-d tensor)."""
        total = torch.zeros((), dtype=torch.float64, device=self.store.device)
        for s in self.store.specs:
            if self.owned(s):
                a, b = self.adamw_slices.get(s.name, (0, s.count))
                total += self.store.grad[s.offset + a:s.offset + b].to(torch.float64).square().sum()
        return total

    @torch.no_grad()
    def step(self, step: int, clip_scale: Optional[torch.Tensor] = None) -> None:
        """One update of every owned parameter. `step` is 1-based. When `clip_scale` is None
        the global norm is taken over this rank's gradients (single-rank training)."""
        st = self.store
        cfg = self.config
        if clip_scale is None:
            all_owned = all(self.owned(s) for s in st.specs)
            spans = [st.grad] if all_owned else [st.g(s.name) for s in st.specs if self.owned(s)]
            norm, clip_scale = ops.grad_norm_and_clip(spans, cfg.clip)
            self.last_grad_norm = norm
        lrm = self.lr_multiplier_override if self.lr_multiplier_override >= 0.0 \
            else self.scheduler.lr_multiplier(step)
        # Under the fused data-parallel transport the AdamW slices (bound by HBM and by the NVLink stores of their
        # pushes) run on a side stream beside Newton-Schulz (bound by the tensor cores); the streams join at the end.
        side = None
        if self.pusher is not None and hasattr(self.pusher, "side_stream") and st.device.type == "cuda":
            side = self.pusher.side_stream()
            side.wait_stream(torch.cuda.current_stream(st.device))
        with torch.cuda.stream(side) if side is not None else contextlib.nullcontext():
            self._adamw_groups_step(step, lrm, clip_scale)
            if self.pusher is not None:
                self.pusher.after_adamw(step)
        momentum = self.scheduler.muon_momentum(step)
        wd = self.scheduler.weight_decay(step)
        use_kernels = st.device.type == "cuda" and ops.get_mode() == "kernels" and st.value is not st.master
        for g in self.muon_groups:
            mine = [s for s in g.params if self.owned(s)]
            if not mine:
                continue
            if use_kernels and min(g.rows, g.cols) >= 64 and g.rows % 8 == 0 and g.cols % 8 == 0:
                from .muon_cuda import MuonGroupState, muon_group_step
                key = (g.rows, g.cols)
                if key not in self._muon_scratch:
                    self._muon_scratch[key] = MuonGroupState(len(mine), g.rows, g.cols, st.device)
                muon_group_step([st.g(s.name) for s in mine], [st.m(s.name) for s in mine],
                                [st.v(s.name) for s in mine], [self.state[s.name]["buf1"] for s in mine],
                                [self.state[s.name]["buf2"] for s in mine], self._muon_scratch[key],
                                lr=g.lr * lrm, momentum=momentum, beta2=cfg.muon_beta2, weight_decay=wd,
                                ns_steps=cfg.muon_ns_steps, grad_scale=clip_scale,
                                apply_fn=None if self.pusher is None else self.pusher.make_muon_apply(mine))
                continue
            if use_kernels and g.rows * g.cols <= 1024 and min(g.rows, g.cols) <= 32 and \
                    all(st.g(s.name).is_contiguous() for s in mine):
                # the small gate projections: the whole Muon step of the group in one launch (fp32, one CTA per matrix)
                from ..ops import cuda as K
                from ..ops.ref import POLAR_COEFFS
                key = ("tiny", g.rows, g.cols)
                tabs = self._muon_scratch.get(key)
                ptrs = tuple(t.data_ptr() for s in mine for t in (st.g(s.name), self.state[s.name]["buf1"],
                                                                   self.state[s.name]["buf2"], st.m(s.name),
                                                                   st.v(s.name)))
                if tabs is None or tabs[0] != ptrs:
                    cols5 = [torch.tensor(ptrs[k::5], dtype=torch.int64, device=st.device) for k in range(5)]
                    tabs = (ptrs, cols5)
                    self._muon_scratch[key] = tabs
                gt, b1t, b2t, mt, vt = tabs[1]
                K._C.muon_tiny(gt, b1t, b2t, mt, vt, g.rows, g.cols, momentum, cfg.muon_beta2, g.lr * lrm, wd,
                               cfg.muon_ns_steps, None if clip_scale is None else clip_scale.reshape(1),
                               [list(c) for c in POLAR_COEFFS])
                if self.pusher is not None:
                    for s in mine:
                        self.pusher.push_span(s.offset, s.count)
                continue
            grads = torch.stack([st.g(s.name) for s in mine])
            master = torch.stack([st.m(s.name) for s in mine])
            buf1 = torch.stack([self.state[s.name]["buf1"] for s in mine])
            buf2 = torch.stack([self.state[s.name]["buf2"] for s in mine])
            ops.muon_update(grads, master, None, buf1, buf2, lr=g.lr * lrm, momentum=momentum,
                            beta2=cfg.muon_beta2, weight_decay=wd, ns_steps=cfg.muon_ns_steps,
                            grad_scale=clip_scale)
            for k, s in enumerate(mine):
                st.m(s.name).copy_(master[k])
                if st.value is not st.master:
                    st.v(s.name).copy_(master[k])
                if self.pusher is not None:
                    self.pusher.push_span(s.offset, s.count)
                self.state[s.name]["buf1"].copy_(buf1[k])
                self.state[s.name]["buf2"].copy_(buf2[k])
        if self.pusher is not None:
            self.pusher.after_muon(step)
        if side is not None:
            torch.cuda.current_stream(st.device).wait_stream(side)
        self.step_count = step

    def _adamw_groups_step(self, step: int, lrm: float, clip_scale) -> None:
        st = self.store
        for g in self.adamw_groups:
            for s in g.params:
                if not self.owned(s):
                    continue
                stt = self.state[s.name]
                a, b = self.adamw_slices.get(s.name, (0, s.count))
                if b <= a:
                    continue
                lo, hi = s.offset + a, s.offset + b
                if self.pusher is not None:
                    self.pusher.adamw_push(st.master[lo:hi], lo, st.grad[lo:hi], stt["m"].view(-1), stt["v"].view(-1),
                                           lr=g.lr * lrm, beta1=g.beta1, beta2=g.beta2, eps=g.eps,
                                           weight_decay=g.weight_decay, step=step, grad_scale=clip_scale)
                    continue
                ops.adamw_update(st.master[lo:hi], None if st.value is st.master else st.value[lo:hi],
                                 st.grad[lo:hi], stt["m"].view(-1), stt["v"].view(-1), lr=g.lr * lrm,
                                 beta1=g.beta1, beta2=g.beta2, eps=g.eps, weight_decay=g.weight_decay, step=step,
                                 grad_scale=clip_scale)
