"""The native in-process mesh runtime, its driver and the host collectives (CPU only)."""
import json
import multiprocessing as mp
import os

import numpy as np
import pytest

from nanochat_cpp_b200.config import Config
from nanochat_cpp_b200 import native_mesh as nm
from nanochat_cpp_b200.cpu_engine import CpuModel, CpuOptimizer


def tiny(seq=16):
    return Config(num_layers=2, num_heads=2, num_kv_heads=2, hidden_dim=32, seq_len=seq, vocab_size=64,
                  padded_vocab_size=64, window_pattern="SL")


def batch(rng, b, t, vocab=64):
    tok = rng.integers(0, vocab, size=(b, t + 1), dtype=np.int32)
    return tok[:, :-1].copy(), tok[:, 1:].copy()


@pytest.mark.parametrize("world,count", [(1, 5), (2, 7), (3, 2), (4, 1000), (8, 129)])
def test_memory_ring_all_reduce(world, count):
    rng = np.random.default_rng(world * 100 + count)
    rows = rng.standard_normal((world, count)).astype(np.float32)
    out = nm.memory_ring_all_reduce(rows)
    want = rows.astype(np.float64).sum(0)
    np.testing.assert_allclose(out[0], want, rtol=1e-5, atol=1e-5)
    for r in range(1, world):
        assert np.array_equal(out[r], out[0])  # every rank ends with the same bits


def test_ring_lost_message_times_out():
    rows = np.ones((4, 64), dtype=np.float32)
    with pytest.raises(RuntimeError, match="lost a peer"):
        nm.memory_ring_all_reduce(rows, drop_from=1, timeout_ms=300)


def _tcp_rank(rank, world, conn):
    ring = nm.TcpRing(rank, world)
    conn.send(ring.port)
    ring.connect(conn.recv())
    data = np.full(1000, float(rank + 1), dtype=np.float32)
    ring.all_reduce_sum(data)
    conn.send(data[:3].tolist() + [float(data.sum())])


def test_tcp_ring_all_reduce_across_processes():
    world = 3
    ctx = mp.get_context("spawn")
    pipes = [ctx.Pipe() for _ in range(world)]
    procs = [ctx.Process(target=_tcp_rank, args=(r, world, pipes[r][1])) for r in range(world)]
    for p in procs:
        p.start()
    ports = [pipes[r][0].recv() for r in range(world)]
    for r in range(world):
        pipes[r][0].send(ports)
    for r in range(world):
        assert pipes[r][0].poll(60)
        got = pipes[r][0].recv()
        assert got[:3] == [6.0, 6.0, 6.0] and got[3] == 6000.0
    for p in procs:
        p.join(30)
        assert p.exitcode == 0


def test_mesh_step_equals_single_replica_on_the_whole_batch():
    cfg = tiny()
    rng = np.random.default_rng(0)
    tok, tgt = batch(rng, 4, cfg.seq_len)
    rt = nm.NativeMeshRuntime(nm.Mesh(2), cfg, batch=4, seed=7)
    assert rt.world_size == 2 and len(rt.mesh) == 2
    one = nm.NativeMeshRuntime(nm.Mesh(1), cfg, batch=4, grad_accum=2, seed=7)
    for _ in range(3):
        l2 = rt.train_step(tok, tgt)
        l1 = one.train_step(tok, tgt)
        assert abs(l1 - l2) < 1e-5
    assert rt.step == 3
    assert rt.digest(0) == rt.digest(1)          # replicas stay bit-identical
    m = rt.metrics()
    assert len(m.loss) == 2 and m.grad_norm > 0 and m.step_seconds > 0
    names = rt.param_names()
    for i in (0, len(names) // 2, len(names) - 1):
        np.testing.assert_allclose(rt.read(0, i), one.read(0, i), rtol=2e-4, atol=2e-6)


def test_mesh_matches_the_engine_driven_by_hand():
    cfg = tiny()
    rng = np.random.default_rng(1)
    tok, tgt = batch(rng, 2, cfg.seq_len)
    rt = nm.NativeMeshRuntime(nm.Mesh(1), cfg, batch=2, seed=3)
    model = CpuModel(cfg, seed=3)
    opt = CpuOptimizer(model)
    for step in (1, 2):
        model.zero_grad()
        l_ref = model.forward_loss(tok, tgt)
        model.backward()
        opt.step(step)
        l = rt.train_step(tok, tgt)
        assert abs(l - l_ref) < 1e-6
    names = rt.param_names()
    for i, n in enumerate(names):
        assert np.array_equal(rt.read(0, i).reshape(-1), model.read(n).reshape(-1)), n


def test_mesh_save_load_resumes_bit_exact(tmp_path):
    cfg = tiny()
    rng = np.random.default_rng(2)
    batches = [batch(rng, 4, cfg.seq_len) for _ in range(4)]
    a = nm.NativeMeshRuntime(nm.Mesh(2), cfg, batch=4, seed=5)
    for tok, tgt in batches[:2]:
        a.train_step(tok, tgt)
    path = str(tmp_path / "mesh.ckpt")
    a.save(path)
    b = nm.NativeMeshRuntime(nm.Mesh(2), cfg, batch=4, seed=99)
    b.load(path)
    assert b.step == 2 and b.digest(0) == a.digest(0) and b.digest(1) == a.digest(0)
    for tok, tgt in batches[2:]:
        assert a.train_step(tok, tgt) == b.train_step(tok, tgt)
    assert a.digest(0) == b.digest(1)
    c = nm.NativeMeshRuntime(nm.Mesh(1), cfg, batch=4, seed=99)
    c.load_weights(path)
    assert c.step == 0                            # weights only: the schedule starts again
    # the file is the same container the GPU trainer reads
    import torch
    from nanochat_cpp_b200.optim import Optimizer, OptimizerConfig, SchedulerConfig
    from nanochat_cpp_b200.train.checkpointer import load_checkpoint
    gpt, meta = load_checkpoint(path)
    assert int(meta["step"]) == 2
    opt = Optimizer(gpt.params, OptimizerConfig(), SchedulerConfig(num_iterations=10))
    load_checkpoint(path, gpt, opt)
    assert opt.step_count == 2
    i = c.param_names().index("lm_head.weight")
    assert np.array_equal(gpt.state_dict()["lm_head.weight"].numpy(), c.read(0, i))


def test_mesh_lost_replica_fails_the_step_instead_of_hanging():
    cfg = tiny()
    rng = np.random.default_rng(3)
    tok, tgt = batch(rng, 4, cfg.seq_len)
    rt = nm.NativeMeshRuntime(nm.Mesh(2), cfg, batch=4, seed=5)
    rt.train_step(tok, tgt)
    rt.inject_drop(0, timeout_ms=300)
    with pytest.raises(RuntimeError, match="gradient reduce failed"):
        rt.train_step(tok, tgt)
    assert rt.step == 1


def test_mesh_train_run_driver(tmp_path):
    from nanochat_cpp_b200.post.sft import SftShard, save_sft_shard
    cfg = tiny()
    rng = np.random.default_rng(4)
    tok, tgt = batch(rng, 16, cfg.seq_len)
    shard = str(tmp_path / "rows.nchsft")
    save_sft_shard(shard, SftShard(tok, tgt))
    out = str(tmp_path / "run")
    base = dict(model=cfg, mesh_size=2, packed_rows_path=shard, batch=4, out_dir=out, peak_flops=1e12,
                optimizer=dict(num_iterations=5))        # one schedule for the split and the straight run
    s = nm.mesh_train_run(nm.MeshTrainConfig(num_iterations=3, save_every=2, **base))
    assert s.steps == 3 and not s.interrupted and os.path.exists(s.checkpoint) and s.last_loss > 0
    lines = [json.loads(l) for l in open(os.path.join(out, "metrics.jsonl"))]
    assert [l["step"] for l in lines] == [1, 2, 3]
    summary = json.load(open(os.path.join(out, "summary.json")))
    assert summary["final_step"] == 3 and summary["world_size"] == 2
    # resume continues the schedule and the data order: 3 + 2 steps == 5 steps in one go
    s2 = nm.mesh_train_run(nm.MeshTrainConfig(num_iterations=5, resume=True, **base))
    assert s2.steps == 2
    out_b = str(tmp_path / "run_b")
    s3 = nm.mesh_train_run(nm.MeshTrainConfig(num_iterations=5, **{**base, "out_dir": out_b}))
    assert s3.steps == 5 and abs(s3.last_loss - s2.last_loss) < 1e-6
