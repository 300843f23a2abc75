"""The process boundary: the resource sandbox applies and proves its limits, and the GPU queue hands out device sets
first in, first out, with cancellation and recovery from a lost worker. No GPU is involved: the queue's devices are
numbers, and its jobs are small Python commands that print what they were given."""
import json
import os
import subprocess
import sys
import threading
import time

import pytest

from nanochat_cpp_b200.process import gpu_queue as Q
from nanochat_cpp_b200.process import sandbox as S

PY = sys.executable


def _run_sandbox(args, **kw):
    return subprocess.run([PY, "-m", "nanochat_cpp_b200.process.sandbox"] + args, capture_output=True, text=True,
                          timeout=120, **kw)


@pytest.fixture
def profiles(tmp_path, monkeypatch):
    doc = {"version": 1, "profiles": {
        "small": {"cpus": 1, "mem_max": "1G", "pids": 64, "files": 256, "runtime": 30, "gpus": 0},
        "quick": {"cpus": 1, "mem_max": "1G", "pids": 64, "files": 256, "runtime": 1, "gpus": 0},
        "gpu-test": {"cpus": 1, "mem_max": "0", "pids": 64, "files": 256, "runtime": 20, "gpus": 1}}}
    path = tmp_path / "profiles.json"
    path.write_text(json.dumps(doc))
    monkeypatch.setenv("NANOCHAT_SANDBOX_PROFILES", str(path))
    monkeypatch.setenv("NANOCHAT_SANDBOX_LOG", str(tmp_path / "sandbox.log"))
    return path


def test_sandbox_exports_the_contract_and_applies_limits(profiles, tmp_path):
    code = ("import os, resource; print(os.environ['NANOCHAT_SANDBOX'], os.environ['NANOCHAT_SANDBOX_BACKEND'], "
            "len(os.sched_getaffinity(0)), resource.getrlimit(resource.RLIMIT_AS)[0], "
            "resource.getrlimit(resource.RLIMIT_NOFILE)[0], resource.getrlimit(resource.RLIMIT_CORE)[0], "
            "os.getpgrp() == os.getpid())")
    p = _run_sandbox(["--profile", "small", "--backend", "rlimit", "--", PY, "-c", code])
    assert p.returncode == 0, p.stderr
    name, backend, cpus, as_limit, files, core, own_group = p.stdout.split()
    assert (name, backend, cpus, files, core, own_group) == ("small", "rlimit", "1", "256", "0", "True")
    assert int(as_limit) == 1 << 30
    # the memory ceiling holds: 2 GB of zeros cannot be allocated under 1 GB of address space
    p = _run_sandbox(["--profile", "small", "--backend", "rlimit", "--", PY, "-c", "b = bytearray(2 << 30)"])
    assert p.returncode != 0 and "MemoryError" in p.stderr
    log = (tmp_path / "sandbox.log").read_text()
    assert "start profile=small" in log and "end profile=small" in log


def test_sandbox_wall_clock_stops_the_whole_process_group(profiles, tmp_path):
    marker = tmp_path / "grandchild.pid"
    code = (f"import subprocess, sys, time; p = subprocess.Popen([sys.executable, '-c', 'import time; time.sleep(60)']); "
            f"open({str(marker)!r}, 'w').write(str(p.pid)); time.sleep(60)")
    t0 = time.monotonic()
    p = _run_sandbox(["--profile", "quick", "--backend", "rlimit", "--", PY, "-c", code])
    assert p.returncode == S.EXIT_TIMEOUT and time.monotonic() - t0 < 20
    pid = int(marker.read_text())
    time.sleep(0.3)
    assert not Q.pid_alive(pid) or open(f"/proc/{pid}/stat").read().split()[2] == "Z"     # the grandchild went too


def test_verify_fails_outside_a_sandbox_and_unknown_profiles_are_refused(profiles, monkeypatch):
    monkeypatch.delenv("NANOCHAT_SANDBOX", raising=False)
    p = _run_sandbox(["verify"])
    assert p.returncode == S.EXIT_VERIFY and "NANOCHAT_SANDBOX is not set" in p.stdout
    p = _run_sandbox(["--profile", "nope", "--", "true"])
    assert p.returncode == S.EXIT_LAUNCH and "unknown sandbox profile" in p.stderr
    with pytest.raises(SystemExit):
        S.require_sandbox(enforce=True)
    monkeypatch.setenv("NANOCHAT_SANDBOX", "small")
    S.require_sandbox(enforce=True)


def test_device_sets_are_aligned_blocks():
    dev = list(range(8))
    assert Q.aligned_sets(dev, 2) == [[0, 1], [2, 3], [4, 5], [6, 7]]
    assert Q.aligned_sets(dev, 4) == [[0, 1, 2, 3], [4, 5, 6, 7]]
    assert Q.pick_set(dev, {0}, 2) == [2, 3] and Q.pick_set(dev, {0, 5}, 4) is None
    assert Q.pick_set(dev, set(), 8) == dev and Q.pick_set(dev, {3}, 8) is None


@pytest.fixture
def queue(tmp_path, monkeypatch, profiles):
    monkeypatch.setenv("NANOCHAT_GPUQ_DIR", str(tmp_path / "q"))
    base = Q.queue_base()
    return base, Q.open_db(base)


def _start_worker(base, devices):
    w = Q.Worker(devices, base, backend="rlimit")
    t = threading.Thread(target=w.serve, kwargs={"idle_exit": 0.0}, daemon=True)
    t.start()
    return w, t


PRINT_DEVICES = [PY, "-c", "import os, time; print('devices', os.environ['CUDA_VISIBLE_DEVICES'], "
                           "os.environ['NANOCHAT_SANDBOX']); time.sleep(0.6)"]


def test_queue_runs_disjoint_sets_side_by_side_and_keeps_order(queue):
    base, conn = queue
    a = Q.submit(conn, PRINT_DEVICES, gpus=1)
    b = Q.submit(conn, PRINT_DEVICES, gpus=1)
    c = Q.submit(conn, PRINT_DEVICES, gpus=4)
    d = Q.submit(conn, PRINT_DEVICES, gpus=2)
    with pytest.raises(ValueError):
        Q.submit(conn, PRINT_DEVICES, gpus=3)
    w, t = _start_worker(base, [0, 1, 2, 3])
    try:
        for j in (a, b, c, d):
            assert Q.wait_for(conn, j, timeout=60) == 0, Q.describe(Q.fetch(conn, j))
        ja, jb, jc, jd = (Q.fetch(conn, j) for j in (a, b, c, d))
        assert {ja["devices"], jb["devices"]} == {"0", "1"}                 # two 1-GPU jobs, different devices
        assert ja["started_ns"] < jb["ended_ns"] and jb["started_ns"] < ja["ended_ns"]      # at the same time
        assert jc["devices"] == "0,1,2,3" and jc["started_ns"] >= max(ja["ended_ns"], jb["ended_ns"])
        # the 2-GPU job fitted beside the 1-GPU jobs while the 4-GPU job waited: it overtook it, once
        assert jd["devices"] == "2,3" and jd["started_ns"] < jc["started_ns"] and jc["overtaken"] == 1
        assert "devices 0,1,2,3 gpu-test" in (base / "logs" / f"{c}.log").read_text()
    finally:
        w.stop.set()
        t.join(timeout=20)
    assert not Q.live_workers(conn) or all(not Q.pid_alive(x["pid"]) or x["id"] != w.id for x in Q.live_workers(conn))


def test_cancel_before_and_during_a_run(queue):
    base, conn = queue
    sleeper = [PY, "-c", "import time; print('started', flush=True); time.sleep(60)"]
    running = Q.submit(conn, sleeper, gpus=2)
    waiting = Q.submit(conn, sleeper, gpus=2)
    w, t = _start_worker(base, [0, 1])
    try:
        deadline = time.monotonic() + 30
        while Q.fetch(conn, running)["pid"] is None and time.monotonic() < deadline:
            time.sleep(0.05)
        assert Q.cancel(conn, waiting) == "cancelled"
        assert Q.cancel(conn, running) == "stopping"
        assert Q.wait_for(conn, running, timeout=30) != 0
        assert Q.fetch(conn, running)["state"] == "cancelled" and Q.fetch(conn, waiting)["state"] == "cancelled"
        assert Q.cancel(conn, running) == "cancelled"                      # a terminal state never changes
    finally:
        w.stop.set()
        t.join(timeout=20)


def test_a_lost_worker_is_reconciled(queue):
    base, conn = queue
    job = Q.submit(conn, PRINT_DEVICES, gpus=1)
    stale = Q.now_ns() - int(2 * Q.LEASE_SEC * 1e9)
    conn.execute("INSERT INTO workers VALUES ('w-dead', 999999, '0', ?)", (stale,))
    conn.execute("UPDATE jobs SET state = 'running', worker = 'w-dead', pid = NULL WHERE id = ?", (job,))
    later = Q.submit(conn, PRINT_DEVICES, gpus=1)
    w, t = _start_worker(base, [0])
    try:
        assert Q.wait_for(conn, later, timeout=60) == 0
        lost = Q.fetch(conn, job)
        assert lost["state"] == "failed" and lost["note"] == "worker lost"
    finally:
        w.stop.set()
        t.join(timeout=20)
    # a second worker refuses to start while one holds the lease
    w1, t1 = _start_worker(base, [0])
    time.sleep(0.5)
    try:
        assert Q.Worker([0], base).serve() == 1
    finally:
        w1.stop.set()
        t1.join(timeout=20)


def test_session_supervisor_runs_commands_one_at_a_time(tmp_path, monkeypatch, profiles):
    import io
    from nanochat_cpp_b200.process import supervisor as V
    monkeypatch.setenv("NANOCHAT_SESSION_DIR", str(tmp_path / "sessions"))
    rec = V.start("agent1", network="none", profile="small", worktree=str(tmp_path))
    try:
        assert rec["name"] == "agent1" and V.alive(rec["pid"])
        # a private network namespace when the kernel allows one; otherwise the record says why not
        assert rec["network"] == "none" or "refused" in rec["network_note"]
        st = V.status("agent1")[0]
        assert st["state"] == "live" and st["network_verified"]
        out = io.StringIO()
        rc = V.send("agent1", [PY, "-c", "import os, sys; print(os.environ['NANOCHAT_SESSION'], "
                                         "os.environ['NANOCHAT_SANDBOX'], os.getcwd()); sys.exit(3)"], out=out)
        assert rc == 3 and out.getvalue().split() == ["agent1", "small", str(tmp_path)]
        # two clients at once: the second command starts after the first has ended
        stamps = tmp_path / "stamps"
        code = (f"import time; f = open({str(stamps)!r}, 'a'); f.write('b'); f.flush(); time.sleep(0.5); "
                f"f.write('e'); f.close()")
        ts = [threading.Thread(target=V.send, args=("agent1", [PY, "-c", code]), kwargs={"out": io.StringIO()})
              for _ in range(2)]
        [t.start() for t in ts]
        [t.join(timeout=60) for t in ts]
        assert stamps.read_text() == "bebe"
        bad = io.StringIO()
        assert V.send("agent1", [], out=bad) == 125                        # an empty argv is refused, not run
    finally:
        assert V.stop("agent1")
    assert V.status("agent1")[0]["state"] == "idle"
    assert V.send("agent1", ["true"]) == 125
    with pytest.raises(ValueError):
        V.session_dir("../escape")


def test_lint_is_clean_and_catches_a_planted_finding(tmp_path):
    from nanochat_cpp_b200 import tools_cli as T
    assert T.lint_findings() == []
    (tmp_path / "tests").mkdir()
    (tmp_path / "profiles").mkdir()
    (tmp_path / "tests" / "test_x_gpu.py").write_text("def test_a():\n    pass\n")
    (tmp_path / "profiles" / "p.md").write_text("    ncu --set full -k regex:x python bench.py\n")
    (tmp_path / "broken.py").write_text("def f(:\n")
    found = " | ".join(T.lint_findings(str(tmp_path)))
    assert "without the gpu marker" in found and "without --clock-control none" in found and "does not compile" in found


def test_consistency_gates_pass_and_see_a_planted_gap(tmp_path):
    from nanochat_cpp_b200 import gates as G
    assert G.capi_findings() == [] and G.isolation_findings() == []
    names = G.header_functions()
    assert len(names) >= 68 and "nanochat_model_create" in names and "nanochat_generate_multi" in names
    fake = tmp_path / "capi.h"
    fake.write_text("int nanochat_init(void);\n/* int nanochat_commented_out(void); */\nint nanochat_not_there(int x);\n")
    assert G.header_functions(str(fake)) == ["nanochat_init", "nanochat_not_there"]
