"""Checkpointing: canonical NCHKPT01 round trip with optimizer state (resume is bit-identical), and a file
written by the reference loads into a model built from its recorded configuration."""
import os

import torch

from nanochat_cpp_b200.config import Config
from nanochat_cpp_b200.optim import OptimizerConfig
from nanochat_cpp_b200.train import TrainConfig, Trainer
from nanochat_cpp_b200.train.checkpointer import load_checkpoint, save_checkpoint


def _cfg():
    return Config(num_layers=2, num_heads=4, num_kv_heads=2, hidden_dim=64, seq_len=16, vocab_size=96,
                  padded_vocab_size=128, rope_base=10000.0, window_pattern="SL")


def test_resume_is_exact(tmp_path):
    cfg = _cfg()
    g = torch.Generator().manual_seed(0)
    data = torch.randint(0, cfg.vocab_size, (6, 2, cfg.seq_len + 1), generator=g)
    tc = lambda: TrainConfig(batch=2, num_iterations=6, seed=4, dtype="fp32", optim=OptimizerConfig(adam_eps=1e-4))
    a = Trainer(cfg, tc(), device="cpu")
    for s in range(3):
        a.train_step([(data[s, :, :-1], data[s, :, 1:])])
    path = str(tmp_path / "ck.ckpt")
    save_checkpoint(path, a.model, a.optimizer, step=3, notes="unit test")
    for s in range(3, 6):
        a.train_step([(data[s, :, :-1], data[s, :, 1:])])
    b = Trainer(cfg, tc(), device="cpu")
    _, meta = load_checkpoint(path, b.model, b.optimizer)
    assert meta["step"] == 3 and meta["notes"] == ["unit test"] and meta["config"]["hidden_dim"] == 64
    b.step_count = 3
    for s in range(3, 6):
        b.train_step([(data[s, :, :-1], data[s, :, 1:])])
    assert torch.equal(a.model.params.master, b.model.params.master)


def test_reference_checkpoint_loads(data_dir):
    model, meta = load_checkpoint(os.path.join(data_dir, "sft_base_fixture.ckpt"))
    cfg = model.cfg
    tokens = torch.randint(0, cfg.vocab_size, (2, min(cfg.seq_len, 16)))
    loss = model.forward_loss(tokens, tokens)
    assert torch.isfinite(loss)
