"""Failure detection between training steps, on the host.

Every rank publishes a heartbeat (its step and a wall-clock stamp) in the job's key-value store and, before it
launches the next step, checks its peers: a peer that announced it is leaving, or whose heartbeat is older than
the timeout, raises `PeerLost` here BEFORE any collective or flag-waiting kernel is launched for the new step, so
no GPU work is ever left waiting for a rank that is gone. The device-side counterpart is the bounded wait of the
communication kernels (a status word instead of a hang); a short process-group timeout covers a peer that dies
inside a collective. The reference has only the rendezvous accept timeout and the collective timeout of its TCP
transport (src/rendezvous.cc:105-133, src/distributed.h `timeout_ms`); elastic recovery here is: detect, stop
cleanly, resume the surviving world size from the last canonical checkpoint (which is world-size independent).
"""
from __future__ import annotations

import time
from typing import List, Optional


class PeerLost(RuntimeError):
    def __init__(self, rank: int, reason: str):
        super().__init__(f"rank {rank} is gone: {reason}")
        self.rank, self.reason = rank, reason


class Heartbeat:
    """`store` is a torch.distributed store (TCPStore / FileStore / HashStore) shared by all ranks."""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 30.0, prefix: str = "hb"):
        self.store, self.rank, self.world, self.timeout_s, self.prefix = store, rank, world, timeout_s, prefix
        self.beat(0)

    def _key(self, rank: int) -> str:
        return f"{self.prefix}/{rank}"

    def beat(self, step: int) -> None:
        self.store.set(self._key(self.rank), f"{step}:{time.time():.3f}:alive")

    def leave(self, step: int, reason: str = "left") -> None:
        """Announce an orderly exit (between steps, with nothing of this rank in flight)."""
        self.store.set(self._key(self.rank), f"{step}:{time.time():.3f}:{reason}")

    def peers(self) -> List[dict]:
        out = []
        for r in range(self.world):
            if not self.store.check([self._key(r)]):      # `get` would block until the store's own timeout
                out.append(dict(rank=r, step=-1, age=float("inf"), state="missing"))
                continue
            raw = self.store.get(self._key(r)).decode()
            step, stamp, state = raw.split(":", 2)
            out.append(dict(rank=r, step=int(step), age=time.time() - float(stamp), state=state))
        return out

    def check(self, step: Optional[int] = None) -> None:
        """Raises PeerLost when a peer left, never appeared, or stopped beating. With `step`, a peer more than one
        step behind AND silent for the timeout counts as lost too."""
        for p in self.peers():
            if p["rank"] == self.rank:
                continue
            if p["state"] == "missing":
                raise PeerLost(p["rank"], "never joined")
            if p["state"] != "alive":
                raise PeerLost(p["rank"], p["state"])
            if p["age"] > self.timeout_s:
                raise PeerLost(p["rank"], f"no heartbeat for {p['age']:.1f} s (step {p['step']})")


def guarded_step(hb: Heartbeat, step: int, fn):
    """Check the peers, run one step, publish the heartbeat. The check comes first so that a lost peer is found
    before this rank launches work that would wait for it."""
    hb.check(step)
    out = fn()
    hb.beat(step)
    return out
