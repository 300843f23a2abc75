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


def test_launcher_stops_the_group_when_a_rank_fails_and_restarts_it(tmp_path):
    """Process-group supervision with plain Python children: the failing rank's exit code comes back, a rank that
    would run for a minute is stopped within seconds, a group that fails once succeeds on its second start, and a
    restart adds --resume for an existing checkpoint."""
    import sys
    import time
    from nanochat_cpp_b200.parallel import launcher
    py = sys.executable
    envs = launcher.rank_environments(2, 29671)
    assert envs[1]["RANK"] == "1" and envs[1]["NANOCHAT_WORLD_SIZE"] == "2" and envs[0]["MASTER_ADDR"] == "127.0.0.1"
    slow = [py, "-c", "import time; time.sleep(60)"]
    bad = [py, "-c", "import os, sys; sys.exit(3 if os.environ['RANK'] == '1' else 0)"]
    t0 = time.monotonic()
    res = launcher.run_group_once([slow, bad], envs, grace_s=2.0, first_rank_head_start_s=0.1)
    assert res.returncode == 3 and res.failed_rank == 1 and time.monotonic() - t0 < 20
    assert res.exit_codes[0] not in (None, 0)                      # rank 0 was stopped, not left running
    # a rank that never finishes: the deadline stops the group
    res = launcher.run_group_once([slow, slow], envs, grace_s=2.0, first_rank_head_start_s=0.1, timeout_s=1.0)
    assert res.returncode == 124 and res.failed_rank is None
    # fails on the first start, succeeds on the second (a marker file plays the checkpoint)
    marker = tmp_path / "ckpt"
    flaky = [py, "-c", f"import os, sys; p = {str(marker)!r}; ok = os.path.exists(p); open(p, 'w').close(); "
                       "sys.exit(0 if ok else 5)"]
    starts = []
    res = launcher.run_group(lambda attempt: (starts.append(attempt) or [flaky, [py, "-c", "pass"]]), envs,
                             max_restarts=2, grace_s=2.0, first_rank_head_start_s=0.1)
    assert res.returncode == 0 and res.starts == 2 and starts == [0, 1]
    argv = ["train", "--checkpoint", str(marker), "--batch", "4"]
    assert launcher.with_resume(argv, 0) == argv
    assert launcher.with_resume(argv, 1) == argv + ["--resume", str(marker)]
    assert launcher.with_resume(argv + ["--resume", "x"], 1) == argv + ["--resume", "x"]
