"""Process-group supervision for the `dist` launcher: start one child per rank, stop the whole group as soon as one
rank fails, optionally start it again from the last checkpoint.

The reference's launcher kills the group when a rank dies and recovery is a restart from the last checkpoint plus the
data-cursor sidecar (python/nanochat_cpp/cli.py cmd_dist; src/train.cc:735-738). Here the same policy is one function
over explicit argument lists, so it is tested on CPU with plain Python children: a rank that exits with an error, a
rank that never finishes, a group that succeeds on its second start.

Only the processes started here are ever signalled, by their own PIDs.
"""
from __future__ import annotations

import os
import subprocess
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence


@dataclass
class GroupResult:
    returncode: int                      # 0, or the exit code of the first rank that failed
    failed_rank: Optional[int] = None    # rank whose failure stopped the group
    starts: int = 1                      # how many times the group was started
    exit_codes: List[Optional[int]] = field(default_factory=list)   # of the last start, by rank


def _stop(procs: Sequence[subprocess.Popen], grace_s: float) -> None:
    """Terminate, then kill, the children that are still running (exact PIDs of our own children)."""
    for p in procs:
        if p.poll() is None:
            p.terminate()
    deadline = time.monotonic() + grace_s
    for p in procs:
        if p.poll() is None:
            try:
                p.wait(timeout=max(0.0, deadline - time.monotonic()))
            except subprocess.TimeoutExpired:
                p.kill()
                p.wait()


def run_group_once(commands: Sequence[Sequence[str]], envs: Sequence[Dict[str, str]], *, poll_s: float = 0.2,
                   grace_s: float = 5.0, first_rank_head_start_s: float = 0.5,
                   timeout_s: Optional[float] = None) -> GroupResult:
    """Start commands[r] with envs[r] for every rank r (rank 0 first: it hosts the rendezvous), then watch them.
    The first non-zero exit stops every other rank; so does `timeout_s` (exit code 124, no failed rank)."""
    procs: List[subprocess.Popen] = []
    try:
        for r, (cmd, env) in enumerate(zip(commands, envs)):
            procs.append(subprocess.Popen(list(cmd), env=dict(env)))
            if r == 0 and len(commands) > 1:
                time.sleep(first_rank_head_start_s)
        t0 = time.monotonic()
        while True:
            codes = [p.poll() for p in procs]
            bad = next((r for r, c in enumerate(codes) if c not in (None, 0)), None)
            if bad is not None:
                _stop(procs, grace_s)
                return GroupResult(int(codes[bad]), bad, 1, [p.poll() for p in procs])
            if all(c == 0 for c in codes):
                return GroupResult(0, None, 1, codes)
            if timeout_s is not None and time.monotonic() - t0 > timeout_s:
                _stop(procs, grace_s)
                return GroupResult(124, None, 1, [p.poll() for p in procs])
            time.sleep(poll_s)
    finally:
        _stop(procs, grace_s)


def run_group(make_commands: Callable[[int], Sequence[Sequence[str]]], envs: Sequence[Dict[str, str]], *,
              max_restarts: int = 0, **kw) -> GroupResult:
    """`make_commands(attempt)` returns the per-rank argument lists of start number `attempt` (0-based), so a restart
    can add `--resume <checkpoint>`. The group is started again after a failure, at most `max_restarts` times."""
    attempt = 0
    while True:
        res = run_group_once(make_commands(attempt), envs, **kw)
        res.starts = attempt + 1
        if res.returncode == 0 or attempt >= max_restarts:
            return res
        attempt += 1


def rank_environments(world_size: int, master_port: int, base: Optional[Dict[str, str]] = None) -> List[Dict[str, str]]:
    """The torch and NANOCHAT_* environment contract of each rank on one node (rendezvous on 127.0.0.1)."""
    base = dict(os.environ if base is None else base)
    out = []
    for r in range(world_size):
        out.append(dict(base, RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(world_size), MASTER_ADDR="127.0.0.1",
                        MASTER_PORT=str(master_port), NANOCHAT_RANK=str(r), NANOCHAT_WORLD_SIZE=str(world_size),
                        NANOCHAT_MASTER_ADDR="127.0.0.1", NANOCHAT_MASTER_PORT=str(master_port)))
    return out


def with_resume(argv: Sequence[str], attempt: int) -> List[str]:
    """On a restart, a `train` / `sft` command that names `--checkpoint X` and no `--resume` continues from X if it
    exists (the checkpoint carries the step, the optimizer state and the data cursor)."""
    argv = list(argv)
    if attempt == 0 or "--resume" in argv or "--checkpoint" not in argv:
        return argv
    ckpt = argv[argv.index("--checkpoint") + 1] if argv.index("--checkpoint") + 1 < len(argv) else ""
    if ckpt and os.path.exists(ckpt):
        argv += ["--resume", ckpt]
    return argv
