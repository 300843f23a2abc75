"""Checkpoint round trip across the three engines that share the `NCHKPT01` container:

  1. the PyTorch/CUDA model (`api.Model`) trains a few steps and saves;
  2. the native CPU engine (`cpu_engine.CpuModel`, C++ behind the C ABI) loads the file and scores the same batch;
  3. the file converts to a plain PyTorch `state_dict` and back without changing a byte of the weights.

    python examples/checkpoint_roundtrip.py [directory]

Mirrors the reference's `examples/checkpoint_roundtrip`.
"""
import os
import sys
import tempfile

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # run from a source tree
from nanochat_cpp_b200 import api
from nanochat_cpp_b200.cpu_engine import CpuModel
from nanochat_cpp_b200.train import convert


def main() -> None:
    out = sys.argv[1] if len(sys.argv) > 1 else tempfile.mkdtemp(prefix="nanochat_roundtrip_")
    os.makedirs(out, exist_ok=True)
    cfg = api.Config(2, hidden_dim=128, num_heads=1, vocab_size=512, seq_len=64)
    model = api.Model(cfg, seed=0, dtype="fp32")
    opt = api.Optimizer(model, num_iterations=10)
    rows = torch.randint(0, cfg.vocab_size, (4, cfg.seq_len + 1), generator=torch.Generator().manual_seed(1))
    tokens, targets = rows[:, :-1], rows[:, 1:]
    for step in range(1, 4):
        model.train_step(tokens, targets, opt, step=step)
    path = os.path.join(out, "model.ckpt")
    model.save(path)
    loss_torch = model.forward_loss(tokens, targets)

    native = CpuModel(cfg, seed=123)
    native.load(path)
    loss_native = native.forward_loss(tokens.numpy(), targets.numpy())
    print(f"loss  PyTorch path {loss_torch:.6f}   native CPU engine {loss_native:.6f}")
    assert abs(loss_torch - loss_native) < 2e-4

    pt = os.path.join(out, "model.pt")
    back = os.path.join(out, "model_back.ckpt")
    convert.container_to_torch(path, pt)
    convert.torch_to_container(pt, back, seq_len=cfg.seq_len)
    again = CpuModel(cfg, seed=5)
    again.load(back)
    for name in native.names():
        assert np.array_equal(native.read(name), again.read(name)), name
    print(f"round trip ok: {path} -> {pt} -> {back}")


if __name__ == "__main__":
    main()
