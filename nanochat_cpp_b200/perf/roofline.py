"""Analytic roofline of one training step, as a table of operation families.

Same report as the reference's `EstimatePerformance` (`src/performance_model.cc:501-845`, schema
`nanochat.roofline.v3`): per family and phase the model FLOPs, the bytes that must move, the launches, and
time = max(flops / peak, bytes / bandwidth) + launches * launch latency. Differences, because the engine
differs: the B200 row uses the peaks measured on the device (`MEASURED_PEAKS.json`), and the gradient
synchronisation is the owner-sharded scheme of `parallel/` (each rank pulls its 1/N of the fp32 gradient from
N-1 peers and pushes 1/N of the bf16 parameters to N-1 peers: one hop through NVSwitch, full bandwidth to
every peer) instead of a ring all-reduce.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field
from typing import Dict, List

from ..config import Config
from ..train import mfu as counts


@dataclass
class DeviceLimits:
    name: str
    peak_flops: Dict[str, float]          # precision -> FLOP/s
    hbm_bytes_per_s: float
    launch_seconds: float = 3e-6
    link_bytes_per_s: float = 0.0         # per direction per GPU

    def peak(self, precision: str) -> float:
        return self.peak_flops.get(precision, 0.0)


def _b200() -> DeviceLimits:
    p = counts.measured_peaks()
    bf16 = p["bf16_tflops_sustained"] * 1e12
    return DeviceLimits("b200", {"bf16": bf16, "fp8": 2 * bf16, "fp32": bf16 / 16.0}, p["hbm_gbs"] * 1e9,
                        launch_seconds=2.5e-6, link_bytes_per_s=770e9)


DEVICES = {
    "b200": _b200,
    # the reference's table (backends/cuda/caps.json): dense peaks, HBM3, 3 us launch
    "h100": lambda: DeviceLimits("h100", {"bf16": 989e12, "fp8": 1979e12, "fp32": 67e12}, 3.35e12, 3e-6, 450e9),
    "t4": lambda: DeviceLimits("t4", {"fp32": 8.1e12, "bf16": 0.0, "fp8": 0.0}, 320e9, 3e-6, 0.0),
}


@dataclass
class RooflinePlan:
    device: str = "b200"
    precision: str = "bf16"
    batch: int = 32
    grad_accum: int = 1
    world_size: int = 1
    total_tokens: int = 0
    link_gbps: float = 0.0        # 0 = the device's own figure (GB/s per direction)
    latency_us: float = 5.0
    overlap: float = 0.0          # fraction of the synchronisation hidden behind backward
    muon_ns_steps: int = 5


@dataclass
class Row:
    name: str
    phase: str
    precision: str
    flops: float
    bytes: float
    launches: int
    compute_seconds: float = 0.0
    memory_seconds: float = 0.0
    bound_seconds: float = 0.0
    limit: str = ""
    mfu: float = 0.0


@dataclass
class Estimate:
    device: str
    precision: str
    shape: str
    rows: List[Row] = field(default_factory=list)
    forward_seconds: float = 0.0
    backward_seconds: float = 0.0
    optimizer_seconds: float = 0.0
    sync_seconds: float = 0.0
    step_seconds: float = 0.0
    steps: int = 1
    run_seconds: float = 0.0
    tokens_per_step: int = 0
    tokens_per_second: float = 0.0
    weighted_peak_flops: float = 0.0
    model_mfu: float = 0.0
    optim_mfu: float = 0.0
    optimizer_flops: float = 0.0


_BYTES = {"fp32": 4.0, "bf16": 2.0, "fp8": 1.0}


def _row(lim: DeviceLimits, name, phase, precision, flops, nbytes, launches, per_rank_divisor) -> Row:
    r = Row(name, phase, precision, flops, nbytes, launches)
    peak = lim.peak(precision)
    r.compute_seconds = (flops / per_rank_divisor) / peak if peak > 0 and flops > 0 else 0.0
    r.memory_seconds = (nbytes / per_rank_divisor) / lim.hbm_bytes_per_s if lim.hbm_bytes_per_s > 0 else 0.0
    lat = launches * lim.launch_seconds
    r.bound_seconds = max(r.compute_seconds, r.memory_seconds, lat)
    r.limit = "compute" if r.bound_seconds == r.compute_seconds else "memory" if r.bound_seconds == r.memory_seconds \
        else "launch"
    if r.bound_seconds > 0 and peak > 0:
        r.mfu = (flops / per_rank_divisor) / (r.bound_seconds * peak)
    return r


def estimate(cfg: Config, plan: RooflinePlan) -> Estimate:
    lim = DEVICES[plan.device]()
    world, accum = max(1, plan.world_size), max(1, plan.grad_accum)
    tokens = float(plan.batch * cfg.seq_len * accum * world)     # whole job, per step
    prec = plan.precision
    row_prec = "bf16" if prec in ("bf16", "fp8") else prec
    e = Estimate(lim.name, prec, f"L{cfg.num_layers}-h{cfg.hidden_dim}-s{cfg.seq_len}-b{plan.batch}x{accum}x{world}")
    # matrix groups: (name, rows N, cols K, count); the head stays in bf16 under fp8
    h, q, kv, mlp, V = cfg.hidden_dim, cfg.query_dim, cfg.kv_dim, cfg.mlp_dim, cfg.padded_vocab_size
    groups = [("qkv", q + 2 * kv, h, cfg.num_layers, prec), ("attn_proj", h, q, cfg.num_layers, prec),
              ("mlp_fc", mlp, h, cfg.num_layers, prec), ("mlp_proj", h, mlp, cfg.num_layers, prec),
              ("lm_head", V, h, 1, row_prec)]
    for name, n, k, count, p in groups:
        params = float(n) * k * count
        el = _BYTES[p]
        fwd_bytes = el * (tokens * k * count + params + tokens * n * count)
        e.rows.append(_row(lim, f"gemm_{name}", "forward", p, 2.0 * params * tokens, fwd_bytes, count * accum, world))
        e.rows.append(_row(lim, f"gemm_{name}", "backward", p, 4.0 * params * tokens, 2.0 * fwd_bytes,
                           2 * count * accum, world))
    att_f = att_b = 0.0
    for layer in range(cfg.num_layers):
        left = cfg.window_left(layer)
        window = cfg.seq_len if left < 0 else min(left, cfg.seq_len)
        per_tok = float(cfg.num_heads) * cfg.head_dim * window
        att_f += 4.0 * per_tok * tokens
        att_b += 8.0 * per_tok * tokens
    att_bytes = _BYTES[row_prec] * tokens * 4.0 * cfg.num_heads * cfg.head_dim * cfg.num_layers
    e.rows.append(_row(lim, "attention", "forward", row_prec, att_f, att_bytes, cfg.num_layers * accum, world))
    e.rows.append(_row(lim, "attention", "backward", row_prec, att_b, 2.0 * att_bytes, 3 * cfg.num_layers * accum,
                       world))
    width = cfg.num_layers * (6.0 * h + 2.0 * q + 4.0 * kv + 2.0 * mlp + cfg.num_kv_heads)
    pw = _BYTES[row_prec] * tokens * width
    e.rows.append(_row(lim, "norms_and_pointwise", "forward", row_prec, 0.0, pw / 2, 4 * cfg.num_layers * accum, world))
    e.rows.append(_row(lim, "norms_and_pointwise", "backward", row_prec, 0.0, pw / 2, 4 * cfg.num_layers * accum, world))
    # the chunked head keeps logits in bf16 and rewrites them in place: read + write once each way
    cls = 2.0 * _BYTES[row_prec] * tokens * V
    e.rows.append(_row(lim, "classifier", "forward", row_prec, 0.0, cls / 2, accum, world))
    e.rows.append(_row(lim, "classifier", "backward", row_prec, 0.0, cls / 2, accum, world))
    emb = 2.0 * _BYTES[row_prec] * tokens * h
    e.rows.append(_row(lim, "embedding", "forward", row_prec, 0.0, emb / 2, 1, world))
    e.rows.append(_row(lim, "embedding", "backward", row_prec, 0.0, emb / 2, 1, world))
    total_params = float(counts.count_params(cfg))
    # owner-sharded optimizer: every rank updates 1/world of the state (fp32 master, grad, two moments)
    e.rows.append(_row(lim, "optimizer", "optimizer", "fp32", 0.0, 4.0 * 4.0 * total_params, 8, world))
    muon = counts.muon_flops_per_step(cfg, plan.muon_ns_steps)
    if muon > 0:
        e.optimizer_flops = muon
        e.rows.append(_row(lim, "muon_orthogonalisation", "optimizer", row_prec, muon, 0.0, 40, world))
    link = plan.link_gbps * 1e9 if plan.link_gbps > 0 else lim.link_bytes_per_s
    if world > 1 and link > 0:
        pull = (world - 1) / world * 4.0 * total_params      # fp32 gradient shards read from peers (inbound)
        push = (world - 1) / world * 2.0 * total_params      # bf16 parameters written to peers (outbound)
        full = max(pull, push) / link + plan.latency_us * 1e-6
        e.sync_seconds = (1.0 - min(1.0, max(0.0, plan.overlap))) * full
    for r in e.rows:
        e.step_seconds += r.bound_seconds
        if r.phase == "forward":
            e.forward_seconds += r.bound_seconds
        elif r.phase == "backward":
            e.backward_seconds += r.bound_seconds
        else:
            e.optimizer_seconds += r.bound_seconds
    e.step_seconds += e.sync_seconds
    e.tokens_per_step = int(tokens + 0.5)
    e.steps = max(1, math.ceil(plan.total_tokens / tokens)) if plan.total_tokens > 0 else 1
    e.run_seconds = e.step_seconds * e.steps
    e.tokens_per_second = tokens / e.step_seconds if e.step_seconds > 0 else 0.0
    mf = mp = 0.0
    for r in e.rows:
        peak = lim.peak(r.precision)
        if r.phase != "optimizer" and r.flops > 0 and peak > 0:
            mf += r.flops
            mp += r.flops / peak
    if mp > 0:
        e.weighted_peak_flops = mf / mp
        if e.step_seconds > 0:
            e.model_mfu = (mf / world) / (e.step_seconds * e.weighted_peak_flops)
    if e.optimizer_flops > 0 and e.step_seconds > 0 and lim.peak(row_prec) > 0:
        e.optim_mfu = (e.optimizer_flops / world) / (e.step_seconds * lim.peak(row_prec))
    return e


def format_report(e: Estimate) -> str:
    out = [f"{'operation':30s} {'phase':9s} {'prec':>6s} {'compute (ms)':>14s} {'memory (ms)':>14s} "
           f"{'bound (ms)':>12s} {'limit':>10s}"]
    for r in e.rows:
        out.append(f"{r.name:30s} {r.phase:9s} {r.precision:>6s} {r.compute_seconds * 1e3:14.3f} "
                   f"{r.memory_seconds * 1e3:14.3f} {r.bound_seconds * 1e3:12.3f} {r.limit:>10s}")
    out.append(f"{'gradient_sync':30s} {'sync':9s} {'-':>6s} {'-':>14s} {'-':>14s} {e.sync_seconds * 1e3:12.3f} "
               f"{'sync':>10s}")
    out.append(f"phases: forward {e.forward_seconds * 1e3:.3f} | backward {e.backward_seconds * 1e3:.3f} | "
               f"optimizer {e.optimizer_seconds * 1e3:.3f} | sync {e.sync_seconds * 1e3:.3f} (ms)")
    out.append(f"step bound {e.step_seconds * 1e3:.3f} ms  ({e.run_seconds:.1f} s over {e.steps} steps)")
    out.append(f"at the bound: {e.tokens_per_second:.0f} tokens/s | model_mfu {e.model_mfu * 100:.1f}% | "
               f"optim_mfu {e.optim_mfu * 100:.1f}% | weighted peak {e.weighted_peak_flops / 1e12:.1f} TFLOP/s")
    return "\n".join(out) + "\n"


def report_json(e: Estimate) -> str:
    rows = []
    for r in e.rows:
        rows.append(dict(name=r.name, family=r.name.split("_")[0] if r.name.startswith("gemm") else r.name,
                         phase=r.phase, precision=r.precision, shape=e.shape, flops=r.flops, issued_flops=r.flops,
                         bytes=r.bytes, launches=r.launches, compute_seconds=r.compute_seconds,
                         memory_seconds=r.memory_seconds, bound_seconds=r.bound_seconds, ms=r.bound_seconds * 1e3,
                         limit=r.limit, gflops=(r.flops / r.bound_seconds / 1e9) if r.bound_seconds > 0 else 0.0,
                         work_ratio=1.0 if r.flops > 0 else 0.0, mfu=r.mfu))
    d = dict(schema="nanochat.roofline.v3", device=e.device, precision=e.precision, shape=e.shape, rows=rows,
             forward_seconds=e.forward_seconds, backward_seconds=e.backward_seconds, sync_seconds=e.sync_seconds,
             optimizer_seconds=e.optimizer_seconds, step_seconds=e.step_seconds, steps=e.steps,
             run_seconds=e.run_seconds, tokens_per_step=e.tokens_per_step, tokens_per_second=e.tokens_per_second,
             weighted_peak_flops=e.weighted_peak_flops, model_mfu=e.model_mfu, optim_mfu=e.optim_mfu,
             optimizer_flops=e.optimizer_flops)
    return json.dumps(d)
