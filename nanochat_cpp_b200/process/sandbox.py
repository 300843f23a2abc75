#!/usr/bin/env python3
"""The resource sandbox: start a job under a named budget and make the job able to prove it.

    python -m nanochat_cpp_b200.process.sandbox [--profile NAME] [--backend auto|cgroup|rlimit|none] -- <cmd ...>
    python -m nanochat_cpp_b200.process.sandbox verify            (inside a sandbox: read the limits back)

A profile (`profiles.json` beside this file) names CPUs, a memory ceiling, a process count, an open-file count, a wall
clock and a GPU count. The launcher applies what the machine allows:

  cgroup   a child cgroup (v2) of the launcher's own with memory.max / pids.max / cpu.max, when that directory is
           writable (a delegated subtree; no root, no systemd needed);
  rlimit   hard rlimits (address space for profiles with a memory ceiling, open files, core = 0, CPU seconds =
           wall clock x CPUs) and a CPU affinity mask: always available;
  none     nothing but the environment contract (for a machine where limits are applied from outside).

In every backend the job runs in its own session and process group; the launcher enforces the wall clock itself
(SIGTERM to the group, SIGKILL after a grace period, exit code 124) and exports the contract the binaries check:
`NANOCHAT_SANDBOX=<profile>`, `NANOCHAT_SANDBOX_BACKEND`, `NANOCHAT_SANDBOX_CPUS`, and `OMP_NUM_THREADS`. GPU profiles
carry no address-space limit: a CUDA context reserves far more virtual memory than it uses.

`verify` is a separate process on purpose: it runs inside the budget, before the job, and reads back what its own
process got (rlimits, affinity, cgroup files, the sentinel). A budget that was silently not applied fails here
(exit 126) instead of letting an unbounded run pass as a bounded one.

The reference does this with systemd user scopes and cgroup v2 (python/nanochat_cpp/sandbox.py, tools/sandbox/
profiles.json) and makes every binary refuse to start without the `NANOCHAT_SANDBOX` sentinel
(include/nanochat/sandbox.h). The sentinel contract is kept; systemd is not assumed.
"""
from __future__ import annotations

import argparse
import json
import os
import resource
import signal
import subprocess
import sys
import time
from pathlib import Path

EXIT_TIMEOUT, EXIT_LAUNCH, EXIT_VERIFY = 124, 125, 126
KILL_GRACE_SEC = 5.0


def profiles_file() -> Path:
    return Path(os.environ.get("NANOCHAT_SANDBOX_PROFILES", Path(__file__).with_name("profiles.json")))


def load_profile(name: str) -> dict:
    doc = json.loads(profiles_file().read_text())
    if name not in doc["profiles"]:
        raise KeyError(f"unknown sandbox profile '{name}' (known: {', '.join(sorted(doc['profiles']))})")
    return dict(doc["profiles"][name], name=name)


def parse_bytes(text) -> int:
    text = str(text).strip().upper()
    mult = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30, "T": 1 << 40}
    if text and text[-1] in mult:
        return int(float(text[:-1]) * mult[text[-1]])
    return int(text or 0)


def log_path() -> Path:
    base = os.environ.get("NANOCHAT_SANDBOX_LOG")
    if base:
        return Path(base)
    state = Path(os.environ.get("XDG_STATE_HOME", Path.home() / ".local" / "state")) / "nanochat"
    state.mkdir(parents=True, exist_ok=True)
    return state / "sandbox.log"


def _log(line: str) -> None:
    try:
        with open(log_path(), "a") as f:
            f.write(time.strftime("%Y-%m-%dT%H:%M:%S ") + line + "\n")
    except OSError:
        pass


# ------------------------------------------------------------------------------------------------ cgroup backend
def own_cgroup_dir() -> Path | None:
    try:
        for line in Path("/proc/self/cgroup").read_text().splitlines():
            if line.startswith("0::"):
                d = Path("/sys/fs/cgroup") / line[3:].lstrip("/")
                return d if (d / "cgroup.procs").exists() else None
    except OSError:
        pass
    return None


def cgroup_usable() -> bool:
    d = own_cgroup_dir()
    return d is not None and os.access(d, os.W_OK) and (d / "cgroup.subtree_control").exists()


def make_cgroup(profile: dict) -> Path:
    parent = own_cgroup_dir()
    d = parent / f"nanochat-{profile['name']}-{os.getpid()}"
    d.mkdir()
    mem = parse_bytes(profile.get("mem_max", 0))
    if mem > 0:
        (d / "memory.max").write_text(str(mem))
    if int(profile.get("pids", 0)) > 0:
        (d / "pids.max").write_text(str(int(profile["pids"])))
    if int(profile.get("cpus", 0)) > 0:
        (d / "cpu.max").write_text(f"{int(profile['cpus']) * 100000} 100000")
    return d


# ------------------------------------------------------------------------------------------------ rlimit backend
def affinity_for(cpus: int) -> list:
    have = sorted(os.sched_getaffinity(0))
    return have[:cpus] if 0 < cpus < len(have) else have


def apply_rlimits(profile: dict) -> None:
    """Runs in the child between fork and exec."""
    def cap(kind, value):
        soft, hard = resource.getrlimit(kind)
        value = value if hard == resource.RLIM_INFINITY else min(value, hard)
        resource.setrlimit(kind, (value, value))
    mem = parse_bytes(profile.get("mem_max", 0))
    if mem > 0 and int(profile.get("gpus", 0)) == 0:
        cap(resource.RLIMIT_AS, mem)
    if int(profile.get("files", 0)) > 0:
        cap(resource.RLIMIT_NOFILE, int(profile["files"]))
    cap(resource.RLIMIT_CORE, 0)
    runtime, cpus = int(profile.get("runtime", 0)), max(1, int(profile.get("cpus", 1)))
    if runtime > 0:
        cap(resource.RLIMIT_CPU, runtime * cpus)
    os.sched_setaffinity(0, affinity_for(int(profile.get("cpus", 0))))


# ------------------------------------------------------------------------------------------------ launch
def sandbox_env(profile: dict, backend: str, base: dict | None = None) -> dict:
    env = dict(os.environ if base is None else base)
    cpus = len(affinity_for(int(profile.get("cpus", 0))))
    env.update(NANOCHAT_SANDBOX=profile["name"], NANOCHAT_SANDBOX_BACKEND=backend, NANOCHAT_SANDBOX_CPUS=str(cpus),
               NANOCHAT_SANDBOX_PROFILE_JSON=json.dumps(profile, sort_keys=True))
    env.setdefault("OMP_NUM_THREADS", str(cpus))
    return env


def terminate_group(proc: subprocess.Popen, grace: float = KILL_GRACE_SEC) -> None:
    """SIGTERM to the job's own process group (the launcher started it with setsid), SIGKILL after `grace`."""
    try:
        os.killpg(proc.pid, signal.SIGTERM)
    except ProcessLookupError:
        return
    deadline = time.monotonic() + grace
    while time.monotonic() < deadline:
        if proc.poll() is not None:
            break
        time.sleep(0.05)
    try:
        os.killpg(proc.pid, signal.SIGKILL)      # also reaps grandchildren that ignored SIGTERM
    except ProcessLookupError:
        pass


def launch(profile_name: str, argv: list, backend: str = "auto", env: dict | None = None, stdout=None, stderr=None,
           verify_first: bool = True, on_start=None) -> int:
    """Run `argv` under the profile; returns its exit code (124 on the wall clock, 125 / 126 on launch / verify)."""
    try:
        profile = load_profile(profile_name)
    except (KeyError, OSError, ValueError) as e:
        print(f"sandbox: {e}", file=sys.stderr)
        return EXIT_LAUNCH
    if backend == "auto":
        backend = "cgroup" if cgroup_usable() else "rlimit"
    cg = None
    if backend == "cgroup":
        try:
            cg = make_cgroup(profile)
        except OSError as e:
            print(f"sandbox: cgroup backend unavailable ({e}); using rlimits", file=sys.stderr)
            backend = "rlimit"
    child_env = sandbox_env(profile, backend, env)

    def preexec():
        os.setsid()
        if cg is not None:
            (cg / "cgroup.procs").write_text(str(os.getpid()))
        if backend != "none":
            apply_rlimits(profile)

    def run(cmd, **kw):
        return subprocess.Popen(cmd, env=child_env, preexec_fn=preexec, **kw)

    try:
        if verify_first and backend != "none":
            v = run([sys.executable, "-m", "nanochat_cpp_b200.process.sandbox", "verify"], stdout=subprocess.PIPE,
                    stderr=subprocess.STDOUT, text=True)
            out, _ = v.communicate(timeout=60)
            if v.returncode != 0:
                print("sandbox: the limits were not applied:\n" + out, file=sys.stderr)
                _log(f"verify-failed profile={profile['name']} backend={backend}")
                return EXIT_VERIFY
        started = time.monotonic()
        try:
            proc = run(argv, stdout=stdout, stderr=stderr)
        except OSError as e:
            print(f"sandbox: cannot start {argv[0]}: {e}", file=sys.stderr)
            return EXIT_LAUNCH
        if on_start is not None:
            on_start(proc)
        _log(f"start profile={profile['name']} backend={backend} pid={proc.pid} cmd={' '.join(argv)[:200]}")
        runtime = int(profile.get("runtime", 0))
        try:
            rc = proc.wait(timeout=runtime if runtime > 0 else None)
        except subprocess.TimeoutExpired:
            terminate_group(proc)
            proc.wait()
            rc = EXIT_TIMEOUT
        except KeyboardInterrupt:
            terminate_group(proc)
            proc.wait()
            rc = 130
        _log(f"end profile={profile['name']} pid={proc.pid} rc={rc} seconds={time.monotonic() - started:.1f}")
        return rc if rc >= 0 else 128 - rc
    finally:
        if cg is not None:
            try:
                cg.rmdir()
            except OSError:
                pass


# ------------------------------------------------------------------------------------------------ verify
def verify() -> int:
    """Inside the sandbox: every limit of the profile must be visible on this very process."""
    problems = []
    name = os.environ.get("NANOCHAT_SANDBOX", "")
    if not name:
        problems.append("NANOCHAT_SANDBOX is not set")
    try:
        profile = json.loads(os.environ.get("NANOCHAT_SANDBOX_PROFILE_JSON", ""))
    except ValueError:
        profile = None
        problems.append("no profile in the environment")
    backend = os.environ.get("NANOCHAT_SANDBOX_BACKEND", "")
    if profile is not None and backend in ("rlimit", "cgroup"):
        mem = parse_bytes(profile.get("mem_max", 0))
        if backend == "rlimit" and mem > 0 and int(profile.get("gpus", 0)) == 0:
            if resource.getrlimit(resource.RLIMIT_AS)[0] not in range(1, mem + 1):
                problems.append("address-space limit missing")
        if int(profile.get("files", 0)) > 0 and resource.getrlimit(resource.RLIMIT_NOFILE)[0] > int(profile["files"]):
            problems.append("open-file limit missing")
        if resource.getrlimit(resource.RLIMIT_CORE)[0] != 0:
            problems.append("core dumps not disabled")
        want = int(profile.get("cpus", 0))
        if 0 < want < (os.cpu_count() or 1) and len(os.sched_getaffinity(0)) > want:
            problems.append(f"affinity mask has {len(os.sched_getaffinity(0))} CPUs, profile allows {want}")
        if os.getsid(0) != os.getpid() and os.getpgrp() != os.getpid():
            problems.append("not in a process group of its own")
        if backend == "cgroup":
            d = own_cgroup_dir()
            if d is None or "nanochat-" not in d.name:
                problems.append("not inside a nanochat cgroup")
            elif mem > 0 and (d / "memory.max").read_text().strip() != str(mem):
                problems.append("memory.max differs from the profile")
    for p in problems:
        print("sandbox verify:", p)
    if not problems:
        print(f"sandbox verify: ok profile={name} backend={backend} cpus={len(os.sched_getaffinity(0))}")
    return 0 if not problems else EXIT_VERIFY


def require_sandbox(enforce: bool | None = None) -> None:
    """What a program calls first: refuse to run outside a sandbox when enforcement is on
    (`NANOCHAT_SANDBOX_ENFORCE=1`). The native CLI applies the same rule."""
    if enforce is None:
        enforce = os.environ.get("NANOCHAT_SANDBOX_ENFORCE") == "1"
    if enforce and not os.environ.get("NANOCHAT_SANDBOX"):
        raise SystemExit("refusing to run outside the sandbox: start through `nanochat run <profile> -- ...` "
                         "(NANOCHAT_SANDBOX is not set)")


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv[:1] == ["verify"]:
        return verify()
    if argv[:1] == ["launch"]:
        argv = argv[1:]
    ap = argparse.ArgumentParser(prog="sandbox", description="run a command under a resource profile")
    ap.add_argument("--profile", default="cpu-test")
    ap.add_argument("--backend", default="auto", choices=["auto", "cgroup", "rlimit", "none"])
    ap.add_argument("--no-verify", action="store_true")
    ap.add_argument("cmd", nargs=argparse.REMAINDER)
    a = ap.parse_args(argv)
    cmd = a.cmd[1:] if a.cmd[:1] == ["--"] else a.cmd
    if not cmd:
        ap.error("no command")
    return launch(a.profile, cmd, a.backend, verify_first=not a.no_verify)


if __name__ == "__main__":
    sys.exit(main())
