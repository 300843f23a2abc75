#!/usr/bin/env python3
"""The GPU job queue: one worker owns the GPUs of a machine and hands them out in sets.

    python -m nanochat_cpp_b200.process.gpu_queue submit [--gpus N] [--profile P] [--wait] -- <cmd ...>
    python -m nanochat_cpp_b200.process.gpu_queue worker [--devices 0,1,2,3,4,5,6,7] [--idle-exit SEC]
    python -m nanochat_cpp_b200.process.gpu_queue list | status | cancel JOB | logs JOB | wait JOB | prune

A SQLite file holds the job records and their state machine (queued -> running -> done | failed | cancelled; a
terminal state never changes); plain files hold the logs. Clients only write records: the worker is the one process
that starts GPU work, so two jobs can never meet on a device.

An eight-GPU box is not one resource. A job asks for a set of 1, 2, 4 or 8 GPUs; the worker gives it an aligned set
(2 -> {0,1},{2,3},...; 4 -> {0..3},{4..7}: neighbours, so that a job's ranks share what the topology shares) through
`CUDA_VISIBLE_DEVICES`, and runs jobs on disjoint sets side by side. Order is first in, first out: the head of the
queue starts as soon as its set is free. A later job may start on idle devices while the head waits for a larger
set, but each job can be overtaken at most `MAX_OVERTAKE` times, after which the devices it needs are drained for it.

Every job runs under the resource sandbox (`sandbox.launch`) with the job's profile, in its own process group; cancel
and the wall clock stop exactly that group. The worker renews a lease every few seconds; a worker that starts finds
the running jobs of a worker whose lease ran out and marks them failed ("worker lost") after stopping what is left
of their process groups.

The reference serialises everything behind one device (python/nanochat_cpp/gpu_queue.py: a SQLite FIFO worker with
leases); the set allocation, alignment and bounded overtaking are what a multi-GPU node adds.
"""
from __future__ import annotations

import argparse
import json
import os
import secrets
import signal
import sqlite3
import subprocess
import sys
import threading
import time
from pathlib import Path

from . import sandbox

TERMINAL = ("done", "failed", "cancelled")
HEARTBEAT_SEC = 2.0
LEASE_SEC = 10.0
POLL_SEC = 0.1
MAX_QUEUE = 256
MAX_OVERTAKE = 4
LOG_KEEP_DAYS = 14


def queue_base() -> Path:
    base = os.environ.get("NANOCHAT_GPUQ_DIR")
    d = Path(base) if base else Path(os.environ.get("XDG_STATE_HOME", Path.home() / ".local" / "state")) / "nanochat" / "gpuq"
    d.mkdir(parents=True, exist_ok=True)
    (d / "logs").mkdir(exist_ok=True)
    return d


def open_db(base: Path | None = None) -> sqlite3.Connection:
    base = base or queue_base()
    conn = sqlite3.connect(base / "queue.db", timeout=30.0, isolation_level=None)
    conn.row_factory = sqlite3.Row
    conn.execute("PRAGMA journal_mode=WAL")
    conn.execute("""CREATE TABLE IF NOT EXISTS jobs (
        seq INTEGER PRIMARY KEY AUTOINCREMENT, id TEXT UNIQUE, state TEXT, command TEXT, cwd TEXT, profile TEXT,
        gpus INTEGER, devices TEXT, worker TEXT, pid INTEGER, exit_code INTEGER, note TEXT, overtaken INTEGER DEFAULT 0,
        cancel INTEGER DEFAULT 0, submitted_ns INTEGER, started_ns INTEGER, ended_ns INTEGER)""")
    conn.execute("""CREATE TABLE IF NOT EXISTS workers (
        id TEXT PRIMARY KEY, pid INTEGER, devices TEXT, heartbeat_ns INTEGER)""")
    return conn


def now_ns() -> int:
    return time.time_ns()


# ------------------------------------------------------------------------------------------------ records
def submit(conn, command: list, gpus: int = 1, profile: str = "gpu-test", cwd: str | None = None) -> str:
    if gpus not in (1, 2, 4, 8):
        raise ValueError("a job asks for 1, 2, 4 or 8 GPUs")
    depth = conn.execute("SELECT COUNT(*) FROM jobs WHERE state IN ('queued','running')").fetchone()[0]
    if depth >= MAX_QUEUE:
        raise RuntimeError(f"the queue is full ({depth} jobs)")
    sandbox.load_profile(profile)            # an unknown profile is refused at the door, not at start time
    job_id = time.strftime("%m%d-%H%M%S-") + secrets.token_hex(3)
    conn.execute("INSERT INTO jobs (id, state, command, cwd, profile, gpus, submitted_ns) VALUES (?,?,?,?,?,?,?)",
                 (job_id, "queued", json.dumps(command), cwd or os.getcwd(), profile, gpus, now_ns()))
    return job_id


def fetch(conn, job_id: str):
    return conn.execute("SELECT * FROM jobs WHERE id = ?", (job_id,)).fetchone()


def finish(conn, job_id: str, state: str, exit_code: int | None, note: str = "") -> None:
    conn.execute("UPDATE jobs SET state = ?, exit_code = ?, note = ?, ended_ns = ? WHERE id = ? AND state NOT IN "
                 "('done','failed','cancelled')", (state, exit_code, note, now_ns(), job_id))


def cancel(conn, job_id: str) -> str:
    """A queued job is cancelled here; a running one is flagged and its worker stops the process group."""
    conn.execute("BEGIN IMMEDIATE")
    try:
        job = fetch(conn, job_id)
        if job is None:
            return "unknown"
        if job["state"] == "queued":
            finish(conn, job_id, "cancelled", None, "cancelled before it started")
            return "cancelled"
        if job["state"] == "running":
            conn.execute("UPDATE jobs SET cancel = 1 WHERE id = ?", (job_id,))
            return "stopping"
        return job["state"]
    finally:
        conn.execute("COMMIT")


def live_workers(conn) -> list:
    horizon = now_ns() - int(LEASE_SEC * 1e9)
    return conn.execute("SELECT * FROM workers WHERE heartbeat_ns >= ?", (horizon,)).fetchall()


def pid_alive(pid: int) -> bool:
    try:
        os.kill(pid, 0)
        return True
    except ProcessLookupError:
        return False
    except PermissionError:
        return True


def reconcile(conn) -> list:
    """Jobs left `running` by a worker whose lease ran out: stop what is left of them and mark them failed."""
    horizon = now_ns() - int(LEASE_SEC * 1e9)
    lost = []
    for job in conn.execute("SELECT jobs.id, jobs.pid, workers.heartbeat_ns AS hb, workers.pid AS wpid FROM jobs "
                            "LEFT JOIN workers ON jobs.worker = workers.id WHERE jobs.state = 'running'").fetchall():
        if job["hb"] is not None and job["hb"] >= horizon and pid_alive(job["wpid"]):
            continue
        if job["pid"]:
            try:
                os.killpg(job["pid"], signal.SIGKILL)      # the job's own group: started by the sandbox with setsid
            except (ProcessLookupError, PermissionError):
                pass
        finish(conn, job["id"], "failed", None, "worker lost")
        lost.append(job["id"])
    conn.execute("DELETE FROM workers WHERE heartbeat_ns < ?", (horizon,))
    return lost


# ------------------------------------------------------------------------------------------------ device sets
def aligned_sets(devices: list, size: int) -> list:
    """The sets of `size` a job may get: consecutive, aligned blocks of the worker's device list."""
    return [devices[i:i + size] for i in range(0, len(devices) - size + 1, size)]


def pick_set(devices: list, busy: set, size: int):
    for s in aligned_sets(devices, size):
        if not busy.intersection(s):
            return s
    return None


def detect_devices() -> list:
    env = os.environ.get("NANOCHAT_GPUQ_DEVICES")
    if env:
        return [int(x) for x in env.split(",") if x.strip() != ""]
    try:
        out = subprocess.run(["nvidia-smi", "--query-gpu=index", "--format=csv,noheader"], capture_output=True,
                             text=True, timeout=30)
        return [int(x) for x in out.stdout.split()] if out.returncode == 0 else []
    except (OSError, subprocess.SubprocessError):
        return []


# ------------------------------------------------------------------------------------------------ worker
class Worker:
    def __init__(self, devices: list, base: Path | None = None, backend: str = "auto"):
        self.base = base or queue_base()
        self.devices = devices
        self.backend = backend
        self.id = "w-" + secrets.token_hex(4)
        self.running = {}             # job id -> dict(thread, proc, devices)
        self.lock = threading.Lock()
        self.stop = threading.Event()

    def _conn(self):
        return open_db(self.base)

    def _heartbeat_loop(self):
        conn = self._conn()
        while not self.stop.wait(HEARTBEAT_SEC):
            conn.execute("UPDATE workers SET heartbeat_ns = ? WHERE id = ?", (now_ns(), self.id))

    def _run_job(self, job, devices: list):
        conn = self._conn()
        log = open(self.base / "logs" / f"{job['id']}.log", "ab", buffering=0)
        env = dict(os.environ, CUDA_VISIBLE_DEVICES=",".join(str(d) for d in devices), NANOCHAT_GPUQ_JOB=job["id"],
                   NANOCHAT_GPUQ_GPUS=str(len(devices)))

        def started(proc):
            with self.lock:
                self.running[job["id"]]["proc"] = proc
            conn.execute("UPDATE jobs SET pid = ? WHERE id = ?", (proc.pid, job["id"]))

        cwd = job["cwd"] if os.path.isdir(job["cwd"]) else None
        old = os.getcwd()
        try:
            # the sandbox starts the job in its own session; cwd is per process, so pass it through `env -C`-less
            # means: a small wrapper that changes directory first
            argv = json.loads(job["command"])
            if cwd:
                argv = [sys.executable, "-c", "import os,sys;os.chdir(sys.argv[1]);os.execvp(sys.argv[2],sys.argv[2:])",
                        cwd] + argv
            rc = sandbox.launch(job["profile"], argv, self.backend, env=env, stdout=log, stderr=subprocess.STDOUT,
                                on_start=started)
        except Exception as e:      # a job must never take the worker down
            rc = sandbox.EXIT_LAUNCH
            log.write(f"[gpuq] launch failed: {e}\n".encode())
        finally:
            os.chdir(old) if os.getcwd() != old else None
            log.close()
        cancelled = bool(fetch(conn, job["id"])["cancel"])
        state = "cancelled" if cancelled else ("done" if rc == 0 else "failed")
        note = {sandbox.EXIT_TIMEOUT: "wall clock of the profile", sandbox.EXIT_VERIFY: "sandbox limits not applied",
                sandbox.EXIT_LAUNCH: "could not start"}.get(rc, "")
        finish(conn, job["id"], state, rc, "cancelled while running" if cancelled else note)
        with self.lock:
            self.running.pop(job["id"], None)

    def _busy(self) -> set:
        with self.lock:
            return {d for j in self.running.values() for d in j["devices"]}

    def _claim(self, conn):
        """The next job to start and its device set, or None. FIFO with bounded overtaking."""
        queued = conn.execute("SELECT * FROM jobs WHERE state = 'queued' ORDER BY seq").fetchall()
        busy = self._busy()
        blocked = []          # jobs ahead that could not start
        for job in queued:
            if job["gpus"] > len(self.devices):
                finish(conn, job["id"], "failed", None, f"asks for {job['gpus']} GPUs, the worker has {len(self.devices)}")
                continue
            if any(b["overtaken"] >= MAX_OVERTAKE for b in blocked):
                return None   # someone ahead has waited long enough: drain for it
            devs = pick_set(self.devices, busy, job["gpus"])
            if devs is None:
                blocked.append(job)
                continue
            conn.execute("BEGIN IMMEDIATE")
            try:
                cur = conn.execute("UPDATE jobs SET state = 'running', worker = ?, devices = ?, started_ns = ? WHERE id = ? "
                                   "AND state = 'queued'", (self.id, ",".join(map(str, devs)), now_ns(), job["id"]))
                if cur.rowcount == 1:
                    for b in blocked:
                        conn.execute("UPDATE jobs SET overtaken = overtaken + 1 WHERE id = ?", (b["id"],))
            finally:
                conn.execute("COMMIT")
            if cur.rowcount == 1:
                return job, devs
        return None

    def _apply_cancels(self, conn):
        for row in conn.execute("SELECT id FROM jobs WHERE state = 'running' AND cancel = 1 AND worker = ?", (self.id,)):
            with self.lock:
                entry = self.running.get(row["id"])
            if entry and entry.get("proc") is not None and not entry.get("stopping"):
                entry["stopping"] = True
                threading.Thread(target=sandbox.terminate_group, args=(entry["proc"], 2.0), daemon=True).start()

    def serve(self, idle_exit: float = 0.0) -> int:
        conn = self._conn()
        others = [w for w in live_workers(conn) if pid_alive(w["pid"])]
        if others:
            print(f"gpuq: worker {others[0]['id']} (pid {others[0]['pid']}) already owns the GPUs", file=sys.stderr)
            return 1
        reconcile(conn)
        conn.execute("INSERT OR REPLACE INTO workers VALUES (?,?,?,?)",
                     (self.id, os.getpid(), ",".join(map(str, self.devices)), now_ns()))
        threading.Thread(target=self._heartbeat_loop, daemon=True).start()
        idle_since = time.monotonic()
        try:
            while not self.stop.is_set():
                self._apply_cancels(conn)
                claimed = self._claim(conn)
                if claimed is not None:
                    job, devs = claimed
                    t = threading.Thread(target=self._run_job, args=(job, devs), daemon=True)
                    with self.lock:
                        self.running[job["id"]] = {"thread": t, "proc": None, "devices": devs}
                    t.start()
                    idle_since = time.monotonic()
                    continue
                with self.lock:
                    active = bool(self.running)
                if active:
                    idle_since = time.monotonic()
                elif idle_exit > 0 and time.monotonic() - idle_since > idle_exit:
                    break
                time.sleep(POLL_SEC)
        finally:
            self.stop.set()
            with self.lock:
                entries = list(self.running.values())
            for e in entries:              # a stopping worker takes its jobs with it, by their own groups
                if e.get("proc") is not None:
                    sandbox.terminate_group(e["proc"], 2.0)
            for e in entries:
                e["thread"].join(timeout=10)
            conn.execute("DELETE FROM workers WHERE id = ?", (self.id,))
        return 0


# ------------------------------------------------------------------------------------------------ client verbs
def wait_for(conn, job_id: str, timeout: float = 0.0, follow=None) -> int:
    """Block until the job is terminal; returns its exit code (1 when it has none)."""
    base = queue_base()
    offset, start = 0, time.monotonic()
    while True:
        job = fetch(conn, job_id)
        if follow is not None:
            path = base / "logs" / f"{job_id}.log"
            if path.exists():
                with open(path, "rb") as f:
                    f.seek(offset)
                    chunk = f.read()
                    offset += len(chunk)
                    follow.write(chunk.decode(errors="replace"))
                    follow.flush()
        if job is None:
            return 2
        if job["state"] in TERMINAL:
            return job["exit_code"] if job["exit_code"] is not None else (0 if job["state"] == "done" else 1)
        if timeout > 0 and time.monotonic() - start > timeout:
            return 3
        time.sleep(POLL_SEC)


def prune_logs(conn, base: Path, keep_days: float = LOG_KEEP_DAYS) -> int:
    horizon = time.time() - keep_days * 86400
    live = {r["id"] for r in conn.execute("SELECT id FROM jobs WHERE state IN ('queued','running')")}
    removed = 0
    for p in (base / "logs").glob("*.log"):
        if p.stem not in live and p.stat().st_mtime < horizon:
            p.unlink()
            removed += 1
    return removed


def describe(job) -> dict:
    d = {k: job[k] for k in job.keys()}
    d["command"] = json.loads(d["command"])
    return d


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="gpuq", description="GPU job queue")
    sub = ap.add_subparsers(dest="verb", required=True)
    s = sub.add_parser("submit")
    s.add_argument("--gpus", type=int, default=1)
    s.add_argument("--profile", default="gpu-test")
    s.add_argument("--wait", action="store_true")
    s.add_argument("cmd", nargs=argparse.REMAINDER)
    w = sub.add_parser("worker")
    w.add_argument("--devices", default="")
    w.add_argument("--idle-exit", type=float, default=0.0)
    w.add_argument("--backend", default="auto")
    for name in ("cancel", "logs", "wait", "status"):
        p = sub.add_parser(name)
        p.add_argument("job", nargs="?" if name == "status" else None)
    sub.add_parser("list")
    pr = sub.add_parser("prune")
    pr.add_argument("--keep-days", type=float, default=LOG_KEEP_DAYS)
    a = ap.parse_args(argv)
    base = queue_base()
    conn = open_db(base)
    if a.verb == "submit":
        cmd = a.cmd[1:] if a.cmd[:1] == ["--"] else a.cmd
        if not cmd:
            ap.error("no command")
        try:
            job_id = submit(conn, cmd, a.gpus, a.profile)
        except (ValueError, RuntimeError, KeyError) as e:
            print(f"gpuq: {e}", file=sys.stderr)
            return 2
        print(job_id)
        if not live_workers(conn):
            print("gpuq: no worker is running; start one with `gpuq worker`", file=sys.stderr)
        return wait_for(conn, job_id, follow=sys.stdout) if a.wait else 0
    if a.verb == "worker":
        devices = [int(x) for x in a.devices.split(",") if x.strip()] if a.devices else detect_devices()
        if not devices:
            print("gpuq: no GPUs found (name them with --devices)", file=sys.stderr)
            return 1
        worker = Worker(devices, base, a.backend)
        signal.signal(signal.SIGTERM, lambda *_: worker.stop.set())
        return worker.serve(a.idle_exit)
    if a.verb == "cancel":
        print(cancel(conn, a.job))
        return 0
    if a.verb == "wait":
        return wait_for(conn, a.job)
    if a.verb == "logs":
        path = base / "logs" / f"{a.job}.log"
        sys.stdout.write(path.read_text(errors="replace") if path.exists() else "")
        return 0
    if a.verb == "list":
        for job in conn.execute("SELECT * FROM jobs ORDER BY seq DESC LIMIT 40"):
            print(f"{job['id']}  {job['state']:<9}  gpus={job['gpus']} devices={job['devices'] or '-':<15} "
                  f"rc={job['exit_code']}  {' '.join(json.loads(job['command']))[:60]}")
        return 0
    if a.verb == "status":
        if a.job:
            job = fetch(conn, a.job)
            print(json.dumps(describe(job) if job else {"error": "unknown job"}, indent=1))
            return 0 if job else 2
        workers = [dict(id=w["id"], pid=w["pid"], devices=w["devices"]) for w in live_workers(conn)]
        counts = {r["state"]: r["n"] for r in conn.execute("SELECT state, COUNT(*) AS n FROM jobs GROUP BY state")}
        print(json.dumps({"workers": workers, "jobs": counts}, indent=1))
        return 0
    if a.verb == "prune":
        print(f"removed {prune_logs(conn, base, a.keep_days)} logs")
        return 0
    return 2


if __name__ == "__main__":
    sys.exit(main())
