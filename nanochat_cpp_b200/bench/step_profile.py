"""Per-operator breakdown of one training step (CUDA events around every operator call).

    python -m nanochat_cpp_b200.bench.step_profile --preset d20 --batch 32 [--out profile.txt]

Counterpart of the reference's traced per-family split (docs/performance-model.md:758-770).
"""
from __future__ import annotations

import argparse

import torch

from .. import ops
from ..config import preset
from ..data.synthetic import zipf_tokens
from ..train import TrainConfig, Trainer


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="d20")
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    cfg = preset(args.preset)
    tr = Trainer(cfg, TrainConfig(batch=args.batch, num_iterations=100, seed=0), device="cuda")
    rows = zipf_tokens(args.batch, cfg.seq_len, cfg.vocab_size, seed=1).cuda()
    mb = [(rows[:, :-1], rows[:, 1:])]
    for _ in range(3):
        tr.train_step(mb)
    torch.cuda.synchronize()
    a, b, c = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    with ops.profile() as prof:
        a.record()
        tr.model.zero_grad()
        loss = tr.model.forward_backward(*mb[0])
        b.record()
        tr.optimizer.step(4)
        c.record()
        table = prof.table()
    lines = [f"# {args.preset} batch {args.batch} x seq {cfg.seq_len}: fwd+bwd {a.elapsed_time(b):.2f} ms, "
             f"optimizer {b.elapsed_time(c):.2f} ms", f"{'operator':28s} {'ms':>10s} {'calls':>7s}"]
    total = 0.0
    for name, ms, n in table:
        lines.append(f"{name:28s} {ms:10.3f} {n:7d}")
        total += ms
    lines.append(f"{'sum of operators':28s} {total:10.3f}")
    text = "\n".join(lines)
    print(text)
    if args.out:
        open(args.out, "w").write(text + "\n")


if __name__ == "__main__":
    main()
