#!/usr/bin/env python3
"""Sessions and their supervisor: a named, long-lived context that commands are sent into, one at a time.

    python -m nanochat_cpp_b200.process.supervisor start  --name NAME [--network host|none] [--profile P]
    python -m nanochat_cpp_b200.process.supervisor send   --name NAME -- <cmd ...>
    python -m nanochat_cpp_b200.process.supervisor status [--name NAME] [--json]
    python -m nanochat_cpp_b200.process.supervisor stop   --name NAME

A session is a record on disk (name, network setting, default sandbox profile, working tree, the supervisor's pid and
its namespace identifiers) plus, while it is live, one supervisor process. The supervisor (`hold`) owns whatever the
session isolates and runs every command as its own child, so containment comes from inheritance: with
`--network none` it enters a private user + network namespace before serving (loopback only), and every command it
starts is inside that namespace without needing the privilege to make one. When the kernel refuses the namespace
(an unprivileged container, as here) the session records `network: host (private namespace refused: ...)` instead of
pretending; `status` reads the namespace identifier of the live supervisor back from /proc and compares it with the
caller's, so the record cannot claim an isolation the process does not have.

The wire is newline-delimited JSON over a unix socket in the session directory. A request is
{"argv": [...], "cwd": "...", "env": {...}, "profile": "..."}; the reply is a sequence of
{"stream": "out", "data": "..."} frames and one {"exit": N} frame, or {"error": "..."} and {"exit": 125}. One command
runs at a time: a second client waits for the first to finish (builds and GPU jobs of one session do not overlap).
Commands run under the resource sandbox with the session's profile.

The reference splits this into session.py (record + systemd slice) and supervisor.py (hold / send over NDJSON, one
namespace per session); this is the same protocol without systemd.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import signal
import socket
import subprocess
import sys
import threading
import time
from pathlib import Path

from . import sandbox

CLONE_NEWUSER, CLONE_NEWNET = 0x10000000, 0x40000000


def session_root() -> Path:
    base = os.environ.get("NANOCHAT_SESSION_DIR")
    d = Path(base) if base else Path(os.environ.get("XDG_STATE_HOME", Path.home() / ".local" / "state")) / "nanochat" / "sessions"
    d.mkdir(parents=True, exist_ok=True)
    return d


def session_dir(name: str) -> Path:
    if not name or any(c in name for c in "/\\ \t\n") or name.startswith("."):
        raise ValueError(f"bad session name '{name}'")
    return session_root() / name


def read_record(name: str) -> dict | None:
    try:
        return json.loads((session_dir(name) / "session.json").read_text())
    except (OSError, ValueError):
        return None


def write_record(name: str, record: dict) -> None:
    d = session_dir(name)
    d.mkdir(parents=True, exist_ok=True)
    tmp = d / "session.json.tmp"
    tmp.write_text(json.dumps(record, indent=1, sort_keys=True))
    os.replace(tmp, d / "session.json")


def net_namespace(pid="self") -> str:
    try:
        return os.readlink(f"/proc/{pid}/ns/net")
    except OSError:
        return ""


def enter_private_network() -> str:
    """Unshare user + network namespaces for this process. Returns '' on success, else the reason it was refused."""
    uid, gid = os.getuid(), os.getgid()
    libc = ctypes.CDLL(None, use_errno=True)
    if libc.unshare(CLONE_NEWUSER | CLONE_NEWNET) != 0:
        return os.strerror(ctypes.get_errno())
    try:       # map the caller to itself inside the namespace so files keep their owner
        Path("/proc/self/setgroups").write_text("deny")
        Path("/proc/self/uid_map").write_text(f"{uid} {uid} 1")
        Path("/proc/self/gid_map").write_text(f"{gid} {gid} 1")
    except OSError:
        pass
    return ""


def alive(pid) -> bool:
    if not pid:
        return False
    try:
        os.kill(int(pid), 0)
        return True
    except (ProcessLookupError, ValueError):
        return False
    except PermissionError:
        return True


# ------------------------------------------------------------------------------------------------ hold (server)
def _serve_one(conn: socket.socket, record: dict, lock: threading.Lock) -> None:
    f = conn.makefile("rwb", buffering=0)

    def frame(obj):
        try:
            f.write((json.dumps(obj) + "\n").encode())
        except OSError:
            pass
    try:
        line = f.readline()
        req = json.loads(line)
        argv = req["argv"]
        if not isinstance(argv, list) or not argv:
            raise ValueError("argv must be a non-empty list")
    except (ValueError, KeyError, TypeError) as e:
        frame({"error": f"bad request: {e}"})
        frame({"exit": 125})
        conn.close()
        return
    if req.get("control") == "stop":
        frame({"exit": 0})
        conn.close()
        os.kill(os.getpid(), signal.SIGTERM)
        return
    with lock:                      # one command at a time
        env = dict(os.environ)
        env.update({str(k): str(v) for k, v in (req.get("env") or {}).items()})
        env["NANOCHAT_SESSION"] = record["name"]
        profile = req.get("profile") or record["profile"]
        cwd = req.get("cwd") or record["worktree"]
        r, w = os.pipe()
        done = {}

        def run():
            wrapped = [sys.executable, "-c", "import os,sys;os.chdir(sys.argv[1]);os.execvp(sys.argv[2],sys.argv[2:])",
                       cwd] + argv
            with os.fdopen(w, "wb", buffering=0) as out:
                done["rc"] = sandbox.launch(profile, wrapped, "auto", env=env, stdout=out, stderr=subprocess.STDOUT)
        t = threading.Thread(target=run, daemon=True)
        t.start()
        with os.fdopen(r, "rb", buffering=0) as src:
            while True:
                chunk = src.read(65536)
                if not chunk:
                    break
                frame({"stream": "out", "data": chunk.decode(errors="replace")})
        t.join()
        frame({"exit": int(done.get("rc", 125))})
    conn.close()


def hold(name: str, network: str, profile: str, worktree: str, ready_fd: int | None = None) -> int:
    d = session_dir(name)
    d.mkdir(parents=True, exist_ok=True)
    note = ""
    if network == "none":
        refused = enter_private_network()
        if refused:
            network, note = "host", f"private namespace refused: {refused}"
    sock_path = d / "supervisor.sock"
    if sock_path.exists():
        sock_path.unlink()
    server = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    server.bind(str(sock_path))
    server.listen(8)
    record = dict(name=name, network=network, network_note=note, profile=profile, worktree=worktree, pid=os.getpid(),
                  net_ns=net_namespace(), socket=str(sock_path), started=time.strftime("%Y-%m-%dT%H:%M:%S"))
    write_record(name, record)
    if ready_fd is not None:
        os.write(ready_fd, b"ready\n")
        os.close(ready_fd)
    lock = threading.Lock()
    stop = threading.Event()
    signal.signal(signal.SIGTERM, lambda *_: stop.set())
    server.settimeout(0.2)
    try:
        while not stop.is_set():
            try:
                conn, _ = server.accept()
            except socket.timeout:
                continue
            except OSError:
                break
            threading.Thread(target=_serve_one, args=(conn, record, lock), daemon=True).start()
    finally:
        server.close()
        try:
            sock_path.unlink()
        except OSError:
            pass
        record.update(pid=None, stopped=time.strftime("%Y-%m-%dT%H:%M:%S"))
        write_record(name, record)
    return 0


# ------------------------------------------------------------------------------------------------ client side
def start(name: str, network: str = "host", profile: str = "cpu-test", worktree: str | None = None) -> dict:
    rec = read_record(name)
    if rec and alive(rec.get("pid")):
        return rec
    r, w = os.pipe()
    os.set_inheritable(w, True)
    cmd = [sys.executable, "-m", "nanochat_cpp_b200.process.supervisor", "hold", "--name", name, "--network", network,
           "--profile", profile, "--worktree", worktree or os.getcwd(), "--ready-fd", str(w)]
    subprocess.Popen(cmd, pass_fds=(w,), start_new_session=True, stdin=subprocess.DEVNULL,
                     stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    os.close(w)
    with os.fdopen(r, "rb") as f:
        if not f.readline():
            raise RuntimeError("the supervisor did not come up")
    return read_record(name)


def send(name: str, argv: list, cwd: str | None = None, env: dict | None = None, profile: str | None = None,
         out=None, control: str | None = None) -> int:
    rec = read_record(name)
    if not rec or not alive(rec.get("pid")):
        print(f"session '{name}' has no live supervisor (start it first)", file=sys.stderr)
        return 125
    s = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    s.connect(rec["socket"])
    f = s.makefile("rwb", buffering=0)
    req = {"argv": argv, "cwd": cwd, "env": env or {}, "profile": profile}
    if control:
        req["control"] = control
    f.write((json.dumps(req) + "\n").encode())
    out = out or sys.stdout
    rc = 125
    for line in f:
        msg = json.loads(line)
        if "stream" in msg:
            out.write(msg["data"])
            out.flush()
        elif "error" in msg:
            print(msg["error"], file=sys.stderr)
        elif "exit" in msg:
            rc = int(msg["exit"])
            break
    s.close()
    return rc


def status(name: str | None = None) -> list:
    names = [name] if name else sorted(p.name for p in session_root().iterdir() if (p / "session.json").exists())
    out = []
    for n in names:
        rec = read_record(n)
        if rec is None:
            continue
        live = alive(rec.get("pid"))
        seen = net_namespace(rec["pid"]) if live else ""
        rec["state"] = "live" if live else "idle"
        # read back: a session that says `none` must really sit in a namespace other than the caller's
        rec["network_verified"] = (not live) or (rec["network"] == "host") or (seen != "" and seen != net_namespace())
        out.append(rec)
    return out


def stop(name: str) -> bool:
    rec = read_record(name)
    if not rec or not alive(rec.get("pid")):
        return False
    send(name, ["true"], control="stop", out=open(os.devnull, "w"))
    deadline = time.monotonic() + 10
    while alive(rec["pid"]) and time.monotonic() < deadline:
        time.sleep(0.05)
    if alive(rec["pid"]):
        os.kill(int(rec["pid"]), signal.SIGTERM)      # the exact pid from the session's own record
    return True


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="session")
    sub = ap.add_subparsers(dest="verb", required=True)
    for verb in ("start", "hold"):
        p = sub.add_parser(verb)
        p.add_argument("--name", required=True)
        p.add_argument("--network", default="host", choices=["host", "none"])
        p.add_argument("--profile", default="cpu-test")
        p.add_argument("--worktree", default=os.getcwd())
        if verb == "hold":
            p.add_argument("--ready-fd", type=int, default=None)
    p = sub.add_parser("send")
    p.add_argument("--name", required=True)
    p.add_argument("--profile", default=None)
    p.add_argument("cmd", nargs=argparse.REMAINDER)
    p = sub.add_parser("status")
    p.add_argument("--name", default=None)
    p.add_argument("--json", action="store_true")
    p = sub.add_parser("stop")
    p.add_argument("--name", required=True)
    a = ap.parse_args(argv)
    if a.verb == "hold":
        return hold(a.name, a.network, a.profile, a.worktree, a.ready_fd)
    if a.verb == "start":
        rec = start(a.name, a.network, a.profile, a.worktree)
        print(json.dumps(rec, indent=1))
        return 0
    if a.verb == "send":
        cmd = a.cmd[1:] if a.cmd[:1] == ["--"] else a.cmd
        if not cmd:
            ap.error("no command")
        return send(a.name, cmd, cwd=os.getcwd(), profile=a.profile)
    if a.verb == "status":
        rows = status(a.name)
        if a.json:
            print(json.dumps(rows, indent=1))
        else:
            for r in rows:
                print(f"{r['name']:<16} {r['state']:<5} network={r['network']} profile={r['profile']} pid={r.get('pid')}")
        return 0
    if a.verb == "stop":
        print("stopped" if stop(a.name) else "not running")
        return 0
    return 2


if __name__ == "__main__":
    sys.exit(main())
