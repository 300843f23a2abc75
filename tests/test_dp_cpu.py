"""Data parallelism on CPU ranks (gloo): two ranks on half batches equal one rank on the whole batch."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from nanochat_cpp_b200.config import Config
from nanochat_cpp_b200.optim import OptimizerConfig
from nanochat_cpp_b200.train import TrainConfig, Trainer


def _cfg():
    return Config(num_layers=2, num_heads=4, num_kv_heads=2, hidden_dim=64, seq_len=16, vocab_size=96,
                  padded_vocab_size=128, rope_base=10000.0, window_pattern="SL")


def _opt():
    # a large Adam epsilon keeps parameters whose true gradient is zero from amplifying rounding noise
    # (the reference pins the same value for its oracle fixtures, tests/oracle_test.cc:89)
    return OptimizerConfig(adam_eps=1e-4)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _data(steps, batch, seq, vocab):
    g = torch.Generator().manual_seed(11)
    return torch.randint(0, vocab, (steps, batch, seq + 1), generator=g)


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from nanochat_cpp_b200.parallel.dp import DataParallel
    cfg = _cfg()
    tc = TrainConfig(batch=2, grad_accum=1, num_iterations=4, seed=5, dtype="fp32", optim=_opt())
    tr = Trainer(cfg, tc, device="cpu", dp=DataParallel(rank, world))
    data = _data(4, 4, cfg.seq_len, cfg.vocab_size)
    for step in range(4):
        rows = data[step, rank * 2:(rank + 1) * 2]
        tr.train_step([(rows[:, :-1], rows[:, 1:])])
    if rank == 0:
        torch.save(tr.model.params.master.clone(), out)
    dist.destroy_process_group()


def test_two_ranks_equal_one(tmp_path):
    cfg = _cfg()
    out = str(tmp_path / "dp.pt")
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    tc = TrainConfig(batch=4, grad_accum=1, num_iterations=4, seed=5, dtype="fp32", optim=_opt())
    tr = Trainer(cfg, tc, device="cpu")
    data = _data(4, 4, cfg.seq_len, cfg.vocab_size)
    for step in range(4):
        rows = data[step]
        tr.train_step([(rows[:, :-1], rows[:, 1:])])
    got = torch.load(out)
    want = tr.model.params.master
    assert (got - want).abs().max().item() < 1e-4
