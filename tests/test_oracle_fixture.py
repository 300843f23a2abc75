"""Upstream-PyTorch oracle: forward, backward and a 3-step optimizer trajectory.

`tests/data/debug_state.bin` was recorded from the upstream PyTorch nanochat model at
2 layers / hidden 32 / 8 heads / 2 kv heads / vocab 64 / seq 8 (fp32). Tolerances are the
reference's own (tests/oracle_test.cc:83-95): forward, backward, optimizer 1e-5; trajectory
loss 1e-5 and parameters 1e-4.
"""
import os

import numpy as np
import torch

from nanochat_cpp_b200.config import Config
from nanochat_cpp_b200.data.record_file import read_records
from nanochat_cpp_b200.models import GPT
from nanochat_cpp_b200.optim import Optimizer, OptimizerConfig, SchedulerConfig


def _load(data_dir, name):
    _, recs = read_records(os.path.join(data_dir, name))
    return recs


def _config(recs) -> Config:
    g = lambda k: int(recs["config/" + k][0])
    return Config(num_layers=g("layers"), num_heads=g("heads"), num_kv_heads=g("kv_heads"),
                  hidden_dim=g("embd"), seq_len=g("seq"), vocab_size=g("vocab"),
                  padded_vocab_size=g("padded_vocab"), rope_base=100000.0,
                  window_pattern=bytes(recs["config/window_pattern"]).decode())


def _model(recs, prefix="param/"):
    cfg = _config(recs)
    m = GPT(cfg, "cpu", torch.float32, init=False)
    m.load_state_dict({n: torch.from_numpy(np.array(recs[prefix + n])) for n in m.params.names()})
    return cfg, m


def test_forward_backward(data_dir):
    recs = _load(data_dir, "debug_state.bin")
    cfg, m = _model(recs)
    tokens = torch.from_numpy(np.array(recs["input/tokens"]))
    targets = torch.from_numpy(np.array(recs["input/targets"]))
    raw = m.logits(tokens)
    want = torch.from_numpy(np.array(recs["forward/raw_logits"]))[..., : cfg.vocab_size]
    assert (raw - want).abs().max().item() < 1e-5
    m.zero_grad()
    loss = m.forward_backward(tokens, targets)
    assert abs(loss.item() - float(recs["forward/loss"][0])) < 1e-5
    for n in m.params.names():
        want = torch.from_numpy(np.array(recs["grad/" + n])).view(m.params.g(n).shape)
        err = (m.params.g(n) - want).abs().max().item()
        assert err < 1e-5, (n, err)


def test_optimizer_trajectory(data_dir):
    recs = _load(data_dir, "debug_state.bin")
    cfg, m = _model(recs, "step/0/param/")
    tokens = torch.from_numpy(np.array(recs["input/tokens"]))
    targets = torch.from_numpy(np.array(recs["input/targets"]))
    o = lambda k: float(recs["config/opt/" + k][0])
    opt_cfg = OptimizerConfig(unembedding_lr=o("unembedding_lr"), embedding_lr=o("embedding_lr"),
                              matrix_lr=o("matrix_lr"), scalar_lr=o("scalar_lr"),
                              weight_decay=o("weight_decay"), clip=o("clip"), adam_eps=o("adam_eps"))
    sched = SchedulerConfig(num_iterations=0, warmup_steps=0, warmdown_ratio=0.0, final_lr_frac=0.0,
                            weight_decay_base=0.0, muon_momentum_warmup_steps=0.0, muon_momentum_start=0.95,
                            muon_momentum_peak=0.95, muon_momentum_final=0.95)
    opt = Optimizer(m.params, opt_cfg, sched)
    steps = int(recs["config/steps"][0])
    for k in range(1, steps + 1):
        m.zero_grad()
        m.forward_backward(tokens, targets)
        opt.step(k)
        loss = m.forward_loss(tokens, targets).item()
        assert abs(loss - float(recs[f"step/{k}/loss"][0])) < 1e-5, (k, loss)
        for n in m.params.names():
            want = torch.from_numpy(np.array(recs[f"step/{k}/param/{n}"])).view(m.params.m(n).shape)
            err = (m.params.m(n) - want).abs().max().item()
            assert err < 1e-4, (k, n, err)
