"""`MeshRuntime`: a data-parallel trainer behind one object, driven from a single client process.

The reference's mesh runtime (src/mesh_runtime.cc:112-318, python/nanochat_cpp/runtime.py) runs one host thread
per replica inside one process and sums gradients through a host staging buffer. Here a replica is a process
that owns one GPU (or a CPU replica with the `gloo` backend): the client keeps a pipe to each, `train_step`
splits the global batch by rows across replicas, replicas run the owner-sharded data-parallel step of
`parallel.DataParallel`, and replica 0 answers queries (loss, metrics, parameters, digest, checkpoints). The mesh
is rank 1 with the single axis "data", as in the reference (include/nanochat/mesh.h).
"""
from __future__ import annotations

import os
import socket
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch
import torch.multiprocessing as mp

from .config import Config
from .train.loop import TrainConfig


@dataclass
class MeshSpec:
    devices: Sequence[str]
    axis_names: Sequence[str] = ("data",)

    @property
    def world(self) -> int:
        return len(self.devices)


def fnv1a64(data: bytes, h: int = 0xCBF29CE484222325) -> int:
    for chunk in (data[i:i + (1 << 20)] for i in range(0, len(data), 1 << 20)):
        for b in chunk:
            h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


def _digest(master: torch.Tensor) -> int:
    """FNV-1a over the fp32 master weights; folded per 4 KiB block so large models stay cheap to hash."""
    raw = master.detach().to("cpu", torch.float32).contiguous().numpy().view(np.uint8)
    if raw.size <= (1 << 22):
        return fnv1a64(raw.tobytes())
    blocks = raw[: raw.size // 4096 * 4096].reshape(-1, 4096).astype(np.uint64)
    weights = (np.arange(4096, dtype=np.uint64) * np.uint64(0x9E3779B97F4A7C15)) | np.uint64(1)
    folded = (blocks * weights).sum(axis=1, dtype=np.uint64)
    return fnv1a64(folded.tobytes() + raw[raw.size // 4096 * 4096:].tobytes())


def _replica(rank: int, world: int, device: str, port: int, cfg: Config, tc: TrainConfig, conn) -> None:
    import torch.distributed as dist
    from .parallel import DataParallel
    from .train.loop import Trainer
    dev = torch.device(device)
    dp = None
    if world > 1:
        if dev.type == "cuda":
            torch.cuda.set_device(dev)
        dist.init_process_group("nccl" if dev.type == "cuda" else "gloo", init_method=f"tcp://127.0.0.1:{port}",
                                rank=rank, world_size=world)
        dp = DataParallel(rank, world, transport=os.environ.get("NANOCHAT_DP_TRANSPORT",
                                                                "fused" if dev.type == "cuda" else "nccl"),
                          device=dev)
    trainer = Trainer(cfg, tc, device=dev, dp=dp)
    t_last, tokens_last = time.perf_counter(), 0
    last_loss = float("nan")
    while True:
        cmd, arg = conn.recv()
        try:
            if cmd == "train_step":
                tok, tgt = arg                                   # this replica's rows [accum, B, T]
                micro = [(torch.as_tensor(tok[a], device=dev).long(), torch.as_tensor(tgt[a], device=dev).long())
                         for a in range(tok.shape[0])]
                loss = trainer.train_step(micro)
                if dp is not None:
                    loss = loss.clone().float()
                    dist.all_reduce(loss)
                    loss = loss / world
                last_loss = float(loss)
                tokens_last += tok.size * world
                conn.send(("ok", last_loss))
            elif cmd == "metrics":
                now = time.perf_counter()
                out = dict(step=trainer.step_count, loss=last_loss, grad_norm=trainer.optimizer.grad_norm(),
                           tokens_per_second=tokens_last / max(now - t_last, 1e-9), world_size=world)
                t_last, tokens_last = now, 0
                conn.send(("ok", out))
            elif cmd == "digest":
                from .train.checkpointer import _gather_master
                conn.send(("ok", _digest(_gather_master(trainer.model, dp))))
            elif cmd == "param":
                from .train.checkpointer import _gather_master
                s = next(s for s in trainer.model.params.specs if s.name == arg)
                m = _gather_master(trainer.model, dp)
                conn.send(("ok", m[s.offset:s.offset + s.count].view(s.shape).cpu().numpy()))
            elif cmd == "param_names":
                conn.send(("ok", [(s.name, tuple(s.shape)) for s in trainer.model.params.specs]))
            elif cmd == "save":
                trainer.save(arg)
                conn.send(("ok", None))
            elif cmd == "load":
                conn.send(("ok", trainer.resume(arg)))
            elif cmd == "load_weights":
                from .train.checkpointer import load_checkpoint
                load_checkpoint(arg, trainer.model)
                conn.send(("ok", None))
            elif cmd == "close":
                conn.send(("ok", None))
                break
            else:
                conn.send(("error", f"unknown command {cmd}"))
        except Exception as e:  # the replica stays alive; the client raises
            conn.send(("error", f"{type(e).__name__}: {e}"))
    if world > 1:
        dist.destroy_process_group()


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class MeshRuntime:
    def __init__(self, cfg: Config, devices: Sequence[str] = ("cpu",), tc: Optional[TrainConfig] = None):
        self.cfg, self.spec = cfg, MeshSpec(list(devices))
        self.tc = tc or TrainConfig(dtype="bf16" if str(devices[0]).startswith("cuda") else "fp32")
        ctx = mp.get_context("spawn")
        port = _free_port()
        self._conns, self._procs = [], []
        for r, d in enumerate(self.spec.devices):
            parent, child = ctx.Pipe()
            p = ctx.Process(target=_replica, args=(r, self.spec.world, d, port, cfg, self.tc, child), daemon=True)
            p.start()
            self._conns.append(parent)
            self._procs.append(p)

    def _all(self, cmd, args=None):
        for i, c in enumerate(self._conns):
            c.send((cmd, args[i] if isinstance(args, list) else args))
        out = [c.recv() for c in self._conns]
        for status, val in out:
            if status != "ok":
                raise RuntimeError(val)
        return [v for _, v in out]

    def train_step(self, tokens, targets) -> float:
        """`tokens`, `targets`: [global_batch, T] (or [accum, global_batch, T]); rows are split evenly by replica."""
        tok, tgt = np.asarray(tokens), np.asarray(targets)
        if tok.ndim == 2:
            tok, tgt = tok[None], tgt[None]
        w = self.spec.world
        if tok.shape[1] % w:
            raise ValueError(f"global batch {tok.shape[1]} is not a multiple of the {w} replicas")
        per = tok.shape[1] // w
        parts = [(tok[:, r * per:(r + 1) * per], tgt[:, r * per:(r + 1) * per]) for r in range(w)]
        return self._all("train_step", parts)[0]

    def metrics(self) -> dict:
        return self._all("metrics")[0]

    def digest(self) -> int:
        return self._all("digest")[0]

    def param_names(self):
        return self._all("param_names")[0]

    def param(self, name: str) -> np.ndarray:
        return self._all("param", name)[0]

    def save(self, path: str) -> None:
        self._all("save", path)

    def load(self, path: str) -> int:
        return self._all("load", path)[0]

    def load_weights(self, path: str) -> None:
        self._all("load_weights", path)

    def step(self) -> int:
        return self.metrics()["step"]

    def close(self) -> None:
        if self._conns:
            try:
                self._all("close")
            finally:
                for p in self._procs:
                    p.join(timeout=30)
                self._conns, self._procs = [], []

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
