"""Smallest end-to-end use of the Python API: build a model, train a few steps on synthetic tokens, sample.

    python examples/hello_world.py            # CUDA when present, else the CPU path

Mirrors the reference's `examples/hello_world` (a dozen API calls: Config -> Model -> Optimizer -> steps -> generate).
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # run from a source tree
from nanochat_cpp_b200 import api


def main() -> None:
    cfg = api.Config(2, hidden_dim=128, num_heads=1, vocab_size=512, seq_len=64)
    model = api.Model(cfg, seed=0)
    opt = api.Optimizer(model, num_iterations=20)
    gen = torch.Generator().manual_seed(0)
    rows = torch.randint(0, cfg.vocab_size, (8, cfg.seq_len + 1), generator=gen)
    tokens, targets = rows[:, :-1], rows[:, 1:]
    for step in range(1, 21):
        loss = model.train_step(tokens, targets, opt, step=step)
        if step % 5 == 0:
            print(f"step {step:3d}  loss {float(loss):.4f}")
    out = model.generate([1, 2, 3], max_tokens=8, temperature=0.0)
    print("greedy continuation:", out[0].tokens)


if __name__ == "__main__":
    main()
