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


def test_torch_state_dict_conversion_round_trip(tmp_path):
    import os
    import torch
    from nanochat_cpp_b200.config import Config
    from nanochat_cpp_b200.models import GPT
    from nanochat_cpp_b200.train.checkpointer import load_checkpoint
    from nanochat_cpp_b200.train.convert import container_to_torch, torch_to_container
    cfg = Config(num_layers=2, num_heads=2, num_kv_heads=1, hidden_dim=64, seq_len=32, vocab_size=100,
                 padded_vocab_size=128)
    m = GPT(cfg, "cpu", torch.float32, seed=1)
    pt, ck = os.path.join(tmp_path, "m.pt"), os.path.join(tmp_path, "m.ckpt")
    torch.save({"_orig_mod." + k: v.clone() for k, v in m.state_dict().items()}, pt)
    c = torch_to_container(pt, ck, seq_len=32, vocab_size=100)
    assert (c.num_heads, c.num_kv_heads, c.hidden_dim, c.vocab_size, c.padded_vocab_size) == (2, 1, 64, 100, 128)
    back, meta = load_checkpoint(ck)
    assert torch.equal(back.params.master, m.params.master) and "converted" in " ".join(meta["notes"])
    container_to_torch(ck, os.path.join(tmp_path, "m2.pt"))
    sd = torch.load(os.path.join(tmp_path, "m2.pt"))
    assert all(torch.equal(sd[k], v) for k, v in m.state_dict().items())


def test_attainment_join():
    from nanochat_cpp_b200.config import preset
    from nanochat_cpp_b200.perf.attain import attainment
    from nanochat_cpp_b200.perf.roofline import RooflinePlan
    rep = attainment({"linear_fwd": 40.0, "linear_wgrad": 80.0, "attention_bwd": 50.0, "rmsnorm_bwd": 5.0},
                     preset("d20"), RooflinePlan(batch=32))
    rows = {r["family"]: r for r in rep["rows"]}
    assert rep["schema"] == "nanochat.attainment.v1" and rows["gemm"]["measured_ms"] == 120.0
    assert 0 < rows["attention.backward"]["attainment"] < 1 and rep["step_measured_ms"] == 175.0
