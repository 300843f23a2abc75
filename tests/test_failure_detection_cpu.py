"""Failure detection with failures made on the host: gloo ranks on CPU, a rank that leaves between steps, a rank
that raises, a rank that never joins, a collective that times out. No GPU is involved."""
import datetime
import os
import socket
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from nanochat_cpp_b200.parallel.health import Heartbeat, PeerLost, guarded_step


def _port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_heartbeat_states_with_a_local_store():
    store = dist.HashStore()
    a = Heartbeat(store, 0, 3, timeout_s=0.3)
    with pytest.raises(PeerLost, match="rank 1 is gone: never joined"):
        a.check()
    b, c = Heartbeat(store, 1, 3, timeout_s=0.3), Heartbeat(store, 2, 3, timeout_s=0.3)
    a.check()
    assert guarded_step(a, 1, lambda: 41 + 1) == 42 and a.peers()[0]["step"] == 1
    c.leave(4, "exception:ValueError")
    with pytest.raises(PeerLost, match="rank 2 is gone: exception:ValueError"):
        a.check()
    c.beat(5)
    time.sleep(0.4)
    a.beat(6)
    with pytest.raises(PeerLost, match="no heartbeat"):
        a.check()


def _worker(rank, world, port, q):
    os.environ["GLOO_SOCKET_IFNAME"] = "lo"
    store = dist.TCPStore("127.0.0.1", port, world, rank == 0, timeout=datetime.timedelta(seconds=20))
    dist.init_process_group("gloo", store=store, rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=3))
    hb = Heartbeat(store, rank, world, timeout_s=5.0)
    dist.barrier()
    done = 0
    try:
        for step in range(1, 6):
            if rank == 1 and step == 3:
                hb.leave(step - 1, "left")      # orderly exit between steps: nothing of this rank is in flight
                q.put((rank, "left", done))
                return

            def one_step():
                t = torch.ones(4) * (rank + 1)
                dist.all_reduce(t)
                return float(t[0])
            if rank == 0 and step == 3:
                time.sleep(0.5)                  # give the leaver time to publish
            guarded_step(hb, step, one_step)
            done = step
        q.put((rank, "finished", done))
    except PeerLost as e:
        q.put((rank, f"peer_lost:{e.rank}:{e.reason}", done))
    finally:
        if rank == 0:
            time.sleep(0.5)                      # keep the store alive until the peer has reported


def test_rank_leaving_between_steps_is_seen_before_the_next_collective():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict()
    for _ in range(2):
        r, what, done = q.get(timeout=120)
        got[r] = (what, done)
    for p in procs:
        p.join(timeout=60)
    assert got[1] == ("left", 2)
    assert got[0] == ("peer_lost:1:left", 2)     # rank 0 stopped before launching step 3's all-reduce


def _timeout_worker(rank, world, port, q):
    os.environ["GLOO_SOCKET_IFNAME"] = "lo"
    store = dist.TCPStore("127.0.0.1", port, world, rank == 0, timeout=datetime.timedelta(seconds=20))
    dist.init_process_group("gloo", store=store, rank=rank, world_size=world, timeout=datetime.timedelta(seconds=2))
    dist.barrier()
    if rank == 1:
        q.put((rank, "silent"))
        time.sleep(6)                            # a hung peer: alive but never joins the collective
        return
    try:
        t = torch.ones(2)
        dist.all_reduce(t)
        q.put((rank, "completed"))
    except Exception as e:
        q.put((rank, "collective_error:" + type(e).__name__))


def test_collective_with_a_silent_peer_ends_with_an_error_not_a_hang():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _port()
    procs = [ctx.Process(target=_timeout_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
    assert got[1] == "silent" and got[0].startswith("collective_error:")
