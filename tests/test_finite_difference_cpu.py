"""Finite-difference checks of the hand-written backward passes (no autograd anywhere in the framework)."""
import numpy as np
import torch

from nanochat_cpp_b200.config import Config
from nanochat_cpp_b200.cpu_engine import CpuModel
from nanochat_cpp_b200.models import GPT


def _cfg():
    return Config(num_layers=3, num_heads=2, num_kv_heads=1, hidden_dim=32, seq_len=24, vocab_size=40,
                  padded_vocab_size=64, window_pattern="SL", short_window_override=8)


PROBES = ["lm_head.weight", "transformer.wte.weight", "value_embeds.2.weight", "resid_lambdas", "x0_lambdas",
          "smear_gate.weight", "smear_lambda", "backout_lambda", "transformer.h.0.attn.c_q.weight",
          "transformer.h.1.attn.c_k.weight", "transformer.h.2.attn.c_v.weight", "transformer.h.0.attn.c_proj.weight",
          "transformer.h.2.attn.ve_gate.weight", "transformer.h.1.mlp.c_fc.weight", "transformer.h.2.mlp.c_proj.weight"]


def test_pytorch_path_backward_matches_central_differences():
    torch.manual_seed(0)
    cfg = _cfg()
    m = GPT(cfg, "cpu", torch.float32, seed=11)
    for spec in m.params.specs:   # zero-initialised projections would hide most gradients: move every weight a little
        m.params.m(spec.name).add_(0.05 * torch.randn(spec.shape))
    m.params.sync_compute()
    tok = torch.randint(0, cfg.vocab_size, (2, cfg.seq_len + 1))
    tokens, targets = tok[:, :-1], tok[:, 1:].clone()
    targets[0, 3] = -1                                       # an ignored target
    m.zero_grad()
    m.forward_backward(tokens, targets)
    rng = np.random.default_rng(0)
    checked = 0
    for name in PROBES:
        if name not in [s.name for s in m.params.specs]:
            continue
        w, g = m.params.m(name).view(-1), m.params.g(name).view(-1)
        nz = torch.nonzero(g.abs() > 1e-4).view(-1)
        for idx in (nz[rng.integers(0, len(nz))].item(),) if len(nz) else ():
            old = w[idx].item()
            eps = 2e-3 * max(1.0, abs(old))
            vals = []
            for sign in (+1, -1):
                w[idx] = old + sign * eps
                m.params.sync_compute()
                vals.append(float(m.forward_loss(tokens, targets)))
            w[idx] = old
            m.params.sync_compute()
            fd = (vals[0] - vals[1]) / (2 * eps)
            assert abs(fd - g[idx].item()) <= 3e-2 * max(abs(fd), abs(g[idx].item())) + 2e-4, (name, fd, g[idx].item())
            checked += 1
    assert checked >= 10


def test_native_engine_backward_matches_central_differences():
    cfg = _cfg()
    m = CpuModel(cfg, seed=11)
    rng = np.random.default_rng(1)
    for name in m.names():
        w = m.read(name)
        m.write(name, w + 0.05 * rng.standard_normal(w.shape).astype(np.float32))
    tok = rng.integers(0, cfg.vocab_size, size=(2, cfg.seq_len + 1)).astype(np.int32)
    tokens, targets = tok[:, :-1].copy(), tok[:, 1:].copy()
    targets[1, 5] = -1
    m.zero_grad()
    m.forward_loss(tokens, targets)
    m.backward()
    checked = 0
    for name in PROBES:
        if name not in m.names():
            continue
        w, g = m.read(name).reshape(-1), m.read(name, grad=True).reshape(-1)
        nz = np.nonzero(np.abs(g) > 1e-4)[0]
        if not len(nz):
            continue
        idx = int(nz[rng.integers(0, len(nz))])
        old = float(w[idx])
        eps = 2e-3 * max(1.0, abs(old))
        vals = []
        for sign in (+1, -1):
            w2 = w.copy()
            w2[idx] = old + sign * eps
            m.write(name, w2)
            vals.append(m.forward_loss(tokens, targets))
        m.write(name, w)
        fd = (vals[0] - vals[1]) / (2 * eps)
        assert abs(fd - g[idx]) <= 3e-2 * max(abs(fd), abs(g[idx])) + 2e-4, (name, fd, g[idx])
        checked += 1
    assert checked >= 10
