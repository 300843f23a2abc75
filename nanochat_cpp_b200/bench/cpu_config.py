"""The CPU configuration: a tiny model trained for 20 steps without a GPU, loss trace and checkpoint round trip.

    python -m nanochat_cpp_b200.bench.cpu_config [--engine native|torch|both] [--steps 20]

4 layers, hidden 256, 4 heads (head_dim 64), vocabulary 4096, sequence 256, window pattern SSSL with short window
128, RoPE base 10000, batch 4, uniform random token ids from seed 0, Muon (5 Newton-Schulz steps, lr 0.02) on the
matrices and AdamW on embeddings / head. `native` is the C++ engine behind the C ABI, `torch` the PyTorch operator
path of the same package; `both` also reports how far apart their loss traces are (different random initial
weights are avoided by copying the PyTorch initialisation into the native model).
"""
from __future__ import annotations

import argparse
import json
import os
import tempfile
import time

import numpy as np
import torch

from ..config import Config
from ..cpu_engine import CpuModel, CpuOptimizer
from ..models import GPT
from ..optim import Optimizer, OptimizerConfig, SchedulerConfig

CFG = Config(num_layers=4, num_heads=4, num_kv_heads=4, hidden_dim=256, seq_len=256, vocab_size=4096,
             padded_vocab_size=4096, rope_base=10000.0, window_pattern="SSSL", short_window_override=128)
OPT = dict(unembedding_lr=0.004, embedding_lr=0.2, matrix_lr=0.02, scalar_lr=0.5, weight_decay=0.0, clip=1.0,
           adam_eps=1e-10, muon_ns_steps=5, muon_beta2=0.9)
SCHED = dict(num_iterations=20, warmup_steps=0, warmdown_ratio=0.65, final_lr_frac=0.0, weight_decay_base=0.0,
             muon_momentum_warmup_steps=400.0, muon_momentum_start=0.85, muon_momentum_peak=0.97,
             muon_momentum_final=0.90)


def batches(steps: int, batch: int = 4):
    rng = np.random.default_rng(0)
    for _ in range(steps):
        tok = rng.integers(0, CFG.vocab_size, (batch, CFG.seq_len + 1))
        yield tok[:, :-1].astype(np.int32), tok[:, 1:].astype(np.int32)


def run_torch(steps: int, perturb: float = 0.0):
    """`perturb` > 0 multiplies every initial weight by (1 + perturb * n), n ~ N(0, 1): the sensitivity probe."""
    torch.manual_seed(0)
    m = GPT(CFG, "cpu", torch.float32, seed=0)
    if perturb > 0.0:
        g = torch.Generator().manual_seed(1)
        m.params.master.mul_(1.0 + perturb * torch.randn(m.params.master.shape, generator=g))
        m.params.sync_compute()
    opt = Optimizer(m.params, OptimizerConfig(**OPT), SchedulerConfig(**{**SCHED, "num_iterations": steps}))
    losses, t0 = [], time.perf_counter()
    for k, (tok, tgt) in enumerate(batches(steps), start=1):
        m.zero_grad()
        losses.append(float(m.forward_backward(torch.from_numpy(tok).long(), torch.from_numpy(tgt).long())))
        opt.step(k)
    return m, losses, time.perf_counter() - t0


def run_native(steps: int, init_from: GPT = None):
    # the native engine derives the short window from seq_len: 256/4 rounded up to 128 = 128, as configured
    m = CpuModel(CFG, seed=0)
    if init_from is not None:
        fresh = GPT(CFG, "cpu", torch.float32, seed=0)
        for n in m.names():
            m.write(n, fresh.params.m(n).reshape(-1).numpy())
    opt = CpuOptimizer(m, **OPT, **{**SCHED, "num_iterations": steps})
    losses, t0 = [], time.perf_counter()
    for k, (tok, tgt) in enumerate(batches(steps), start=1):
        m.zero_grad()
        losses.append(m.forward_loss(tok, tgt))
        m.backward()
        opt.step(k)
    return m, losses, time.perf_counter() - t0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--engine", default="both", choices=["native", "torch", "both"])
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--sensitivity", type=float, default=0.0,
                    help="also run the torch engine from weights perturbed by this relative amount (e.g. 1e-7, one "
                         "fp32 rounding step) and report how far its loss trace moves: the scale below which two "
                         "fp32 engines cannot be told apart on this configuration")
    a = ap.parse_args()
    out = dict(config="cpu tiny: 4L/256/4h/vocab4096/seq256/batch4", steps=a.steps)
    tokens = a.steps * 4 * CFG.seq_len
    tm = None
    if a.engine in ("torch", "both"):
        tm, tl, tt = run_torch(a.steps)
        out["torch"] = dict(losses=[round(x, 6) for x in tl], seconds=round(tt, 2), tokens_per_s=round(tokens / tt, 1))
    if a.engine in ("native", "both"):
        nm, nl, nt = run_native(a.steps, init_from=tm)
        out["native"] = dict(losses=[round(x, 6) for x in nl], seconds=round(nt, 2),
                             tokens_per_s=round(tokens / nt, 1))
        with tempfile.TemporaryDirectory() as d:      # checkpoint round trip through the NCHKPT01 container
            path = os.path.join(d, "tiny.ckpt")
            nm.save(path)
            back = CpuModel(CFG, seed=1)
            back.load(path)
            same = all(np.array_equal(back.read(n), nm.read(n)) for n in nm.names())
            tok, tgt = next(batches(1))
            out["checkpoint_round_trip"] = dict(bit_identical=bool(same), bytes=os.path.getsize(path),
                                                loss_before=round(nm.forward_loss(tok, tgt), 6),
                                                loss_after=round(back.forward_loss(tok, tgt), 6))
    if a.sensitivity > 0.0 and tm is not None:
        _, pl, _ = run_torch(a.steps, perturb=a.sensitivity)
        out["sensitivity"] = dict(relative_perturbation=a.sensitivity, losses=[round(x, 6) for x in pl],
                                  max_loss_difference=float(max(abs(x - y) for x, y in zip(tl, pl))))
    if a.engine == "both":
        out["max_loss_difference"] = float(max(abs(x - y) for x, y in zip(out["torch"]["losses"],
                                                                          out["native"]["losses"])))
    print(json.dumps(out))


if __name__ == "__main__":
    main()
