"""ctypes binding of the native in-process mesh runtime, its training driver and the host collectives
(`include/nanochat/capi.h`: `nanochat_mesh_*`, `nanochat_runtime_*`, `nanochat_mesh_train_run`, `ncb_tcp_*`;
implemented in `csrc/host/mesh.cc`, `collective.cc`, `capi_mesh.cc`).

The client surface follows the reference's `python/nanochat_cpp/runtime.py` (`MeshRuntime`, `MeshTrainConfig`) for the
CPU engine: one process, one model replica per mesh position, gradients reduced by a ring inside the process. The
GPU counterpart (one process per GPU) is `nanochat_cpp_b200.runtime.MeshRuntime`.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np

from .config import Config
from .cpu_engine import _ConfigC, _OptimC, _ParamC, _i32, _l
from .data.native import last_error


class _MetricsC(C.Structure):
    _fields_ = [("device_count", C.c_int), ("loss", C.POINTER(C.c_float)), ("grad_norm", C.c_float),
                ("step_seconds", C.c_float)]


class _DataC(C.Structure):
    _fields_ = [("parquet", C.POINTER(C.c_char_p)), ("parquet_count", C.c_int), ("tokenizer_path", C.c_char_p),
                ("packed_rows_path", C.c_char_p), ("data_seed", C.c_uint64)]


class _RunC(C.Structure):
    _fields_ = [("batch", C.c_int), ("grad_accum", C.c_int), ("seq", C.c_int), ("seed", C.c_uint64),
                ("num_iterations", C.c_int), ("log_every", C.c_int), ("save_every", C.c_int), ("resume", C.c_int)]


class _OutputC(C.Structure):
    _fields_ = [("out_dir", C.c_char_p), ("checkpoint_path", C.c_char_p)]


class _TrainC(C.Structure):
    _fields_ = [("model", _ConfigC), ("mesh", C.c_void_p), ("preset", C.c_char_p), ("optimizer", C.POINTER(_OptimC)),
                ("warm_start_path", C.c_char_p), ("flops_per_token", C.c_double), ("peak_flops", C.c_double),
                ("data", _DataC), ("run", _RunC), ("output", _OutputC)]


class _SummaryC(C.Structure):
    _fields_ = [("steps", C.c_int), ("interrupted", C.c_int), ("mean_loss", C.c_double), ("steady_mfu", C.c_double),
                ("checkpoint", C.c_char * 4096)]


_ready = False


def _m():
    global _ready
    L = _l()
    if not _ready:
        L.nanochat_mesh_create.restype = C.c_void_p
        L.nanochat_mesh_create.argtypes = [C.c_void_p, C.c_int]
        L.nanochat_mesh_free.argtypes = [C.c_void_p]
        L.nanochat_mesh_size.argtypes = [C.c_void_p]
        L.nanochat_runtime_create.restype = C.c_void_p
        L.nanochat_runtime_create.argtypes = [C.c_void_p, C.POINTER(_ConfigC), C.POINTER(_OptimC), C.c_int, C.c_int,
                                              C.c_int, C.c_uint64]
        L.nanochat_runtime_free.argtypes = [C.c_void_p]
        L.nanochat_runtime_world_size.argtypes = [C.c_void_p]
        L.nanochat_runtime_train_step.restype = C.c_float
        L.nanochat_runtime_train_step.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        L.nanochat_runtime_metrics.argtypes = [C.c_void_p, C.POINTER(_MetricsC)]
        L.nanochat_runtime_param_count.argtypes = [C.c_void_p, C.c_int]
        L.nanochat_runtime_param_info.argtypes = [C.c_void_p, C.c_int, C.c_int, C.POINTER(_ParamC)]
        L.nanochat_runtime_param_read.restype = C.c_int64
        L.nanochat_runtime_param_read.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_int64,
                                                  C.c_void_p]
        L.nanochat_runtime_param_digest.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_uint64)]
        for f in (L.nanochat_runtime_save, L.nanochat_runtime_load, L.nanochat_runtime_load_weights):
            f.argtypes = [C.c_void_p, C.c_char_p]
        L.nanochat_runtime_step.argtypes = [C.c_void_p]
        L.ncb_runtime_inject_drop.argtypes = [C.c_void_p, C.c_int, C.c_int]
        L.nanochat_mesh_train_run.restype = C.c_float
        L.nanochat_mesh_train_run.argtypes = [C.POINTER(_TrainC), C.POINTER(_SummaryC)]
        L.ncb_tcp_create.restype = C.c_void_p
        L.ncb_tcp_create.argtypes = [C.c_int, C.c_int]
        L.ncb_tcp_port.argtypes = [C.c_void_p]
        L.ncb_tcp_connect.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        L.ncb_tcp_all_reduce_sum.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int]
        L.ncb_tcp_free.argtypes = [C.c_void_p]
        L.ncb_memory_ring_all_reduce.argtypes = [C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_int]
        _ready = True
    return L


def _config_c(cfg: Config) -> _ConfigC:
    return _ConfigC(cfg.num_layers, cfg.num_heads, cfg.num_kv_heads, cfg.hidden_dim, cfg.seq_len, cfg.vocab_size,
                    cfg.padded_vocab_size, cfg.rope_base, cfg.window_pattern.encode(), int(cfg.value_embedding))


def _optim_c(fields: Optional[dict], preset: str = "default") -> _OptimC:
    c = _OptimC()
    if _l().nanochat_optim_config_preset(preset.encode(), C.byref(c)) != 0:
        raise ValueError(last_error() or f"unknown optimizer preset {preset!r}")
    for k, v in (fields or {}).items():
        setattr(c, k, v)
    return c


class Mesh:
    """A rank-1 "data" mesh over `count` positions (device indices default to 0, 1, ...)."""

    def __init__(self, count: int = 1, indices: Optional[Sequence[int]] = None):
        arr = _i32(indices) if indices is not None else None
        self._h = _m().nanochat_mesh_create(arr.ctypes.data if arr is not None else None, count)

    def __len__(self) -> int:
        return int(_m().nanochat_mesh_size(self._h))

    def __del__(self):
        if getattr(self, "_h", None):
            _m().nanochat_mesh_free(self._h)
            self._h = None


@dataclass
class MeshMetrics:
    loss: List[float]
    grad_norm: float
    step_seconds: float


class NativeMeshRuntime:
    """One model replica per mesh position inside this process (CPU engine)."""

    def __init__(self, mesh: Mesh, cfg: Config, batch: int, grad_accum: int = 1, seq: int = 0, seed: int = 42,
                 optim: Optional[dict] = None):
        self.mesh, self.cfg = mesh, cfg
        self.batch, self.seq = batch, seq or cfg.seq_len
        c, o = _config_c(cfg), _optim_c(optim)
        self._h = _m().nanochat_runtime_create(mesh._h, C.byref(c), C.byref(o), batch, grad_accum, seq, seed)
        if not self._h:
            raise RuntimeError(last_error() or "nanochat_runtime_create failed")

    @property
    def world_size(self) -> int:
        return int(_m().nanochat_runtime_world_size(self._h))

    @property
    def step(self) -> int:
        return int(_m().nanochat_runtime_step(self._h))

    def train_step(self, tokens, targets) -> float:
        t, g = _i32(tokens), _i32(targets)
        if t.shape != (self.batch, self.seq) or g.shape != t.shape:
            raise ValueError(f"expected [{self.batch}, {self.seq}] tokens and targets")
        before = self.step
        loss = float(_m().nanochat_runtime_train_step(self._h, t.ctypes.data, g.ctypes.data))
        if self.step == before:
            raise RuntimeError(last_error() or "nanochat_runtime_train_step failed")
        return loss

    def metrics(self) -> MeshMetrics:
        m = _MetricsC()
        _m().nanochat_runtime_metrics(self._h, C.byref(m))
        return MeshMetrics([float(m.loss[i]) for i in range(m.device_count)], float(m.grad_norm),
                           float(m.step_seconds))

    def param_names(self, replica: int = 0) -> List[str]:
        info, out = _ParamC(), []
        for i in range(_m().nanochat_runtime_param_count(self._h, replica)):
            _m().nanochat_runtime_param_info(self._h, replica, i, C.byref(info))
            out.append(info.name.decode())
        return out

    def read(self, replica: int, index: int, grad: bool = False) -> np.ndarray:
        info = _ParamC()
        if not _m().nanochat_runtime_param_info(self._h, replica, index, C.byref(info)):
            raise IndexError("bad replica or parameter index")
        out = np.empty(info.count, dtype=np.float32)
        n = _m().nanochat_runtime_param_read(self._h, replica, index, int(grad), 0, info.count, out.ctypes.data)
        if n != info.count:
            raise RuntimeError("short parameter read")
        return out.reshape(info.rows, info.cols) if info.rows > 0 and info.cols > 0 else out

    def digest(self, replica: int = 0) -> int:
        out = C.c_uint64()
        if _m().nanochat_runtime_param_digest(self._h, replica, C.byref(out)) != 0:
            raise IndexError(last_error() or "bad replica index")
        return int(out.value)

    def save(self, path: str) -> None:
        _m().nanochat_runtime_save(self._h, path.encode())

    def load(self, path: str) -> None:
        _m().nanochat_runtime_load(self._h, path.encode())

    def load_weights(self, path: str) -> None:
        _m().nanochat_runtime_load_weights(self._h, path.encode())

    def inject_drop(self, sender: int, timeout_ms: int = 500) -> None:
        """Failure-detection hook: the next step loses one ring message from `sender`; the step then raises."""
        _m().ncb_runtime_inject_drop(self._h, sender, timeout_ms)

    def __del__(self):
        if getattr(self, "_h", None):
            _m().nanochat_runtime_free(self._h)
            self._h = None


@dataclass
class MeshTrainConfig:
    model: Config
    mesh_size: int = 1
    preset: str = "default"
    optimizer: Optional[dict] = None
    warm_start_path: str = ""
    flops_per_token: float = 0.0
    peak_flops: float = 0.0
    parquet: List[str] = field(default_factory=list)
    tokenizer_path: str = ""
    packed_rows_path: str = ""
    data_seed: int = 0
    batch: int = 8
    grad_accum: int = 1
    seq: int = 0
    seed: int = 42
    num_iterations: int = 10
    log_every: int = 0
    save_every: int = 0
    resume: bool = False
    out_dir: str = "."
    checkpoint_path: str = ""


@dataclass
class MeshTrainSummary:
    last_loss: float
    steps: int
    interrupted: bool
    mean_loss: float
    steady_mfu: float
    checkpoint: str


def mesh_train_run(cfg: MeshTrainConfig) -> MeshTrainSummary:
    """Runs one job of the native driver (step loop, metrics.jsonl, summary.json, checkpoints, resume)."""
    mesh = Mesh(cfg.mesh_size)
    c = _TrainC()
    c.model = _config_c(cfg.model)
    c.mesh = mesh._h
    c.preset = cfg.preset.encode()
    opt = _optim_c(cfg.optimizer, cfg.preset) if cfg.optimizer is not None else None
    c.optimizer = C.pointer(opt) if opt is not None else None
    c.warm_start_path = cfg.warm_start_path.encode()
    c.flops_per_token, c.peak_flops = cfg.flops_per_token, cfg.peak_flops
    paths = (C.c_char_p * max(1, len(cfg.parquet)))(*[p.encode() for p in cfg.parquet])
    c.data = _DataC(C.cast(paths, C.POINTER(C.c_char_p)), len(cfg.parquet), cfg.tokenizer_path.encode(),
                    cfg.packed_rows_path.encode(), cfg.data_seed)
    c.run = _RunC(cfg.batch, cfg.grad_accum, cfg.seq, cfg.seed, cfg.num_iterations, cfg.log_every, cfg.save_every,
                  int(cfg.resume))
    c.output = _OutputC(cfg.out_dir.encode(), cfg.checkpoint_path.encode())
    s = _SummaryC()
    last = float(_m().nanochat_mesh_train_run(C.byref(c), C.byref(s)))
    if s.steps == 0 and last == 0.0:
        raise RuntimeError(last_error() or "nanochat_mesh_train_run failed")
    return MeshTrainSummary(last, s.steps, bool(s.interrupted), s.mean_loss, s.steady_mfu, s.checkpoint.decode())


class TcpRing:
    """One rank of a multi-process CPU job: TCP over 127.0.0.1, ring all-reduce. Exchange `port` between the ranks
    (a file, a pipe, a store), then `connect(ports)`."""

    def __init__(self, rank: int, world: int):
        self.rank, self.world = rank, world
        self._h = _m().ncb_tcp_create(rank, world)
        if not self._h:
            raise RuntimeError(last_error() or "ncb_tcp_create failed")

    @property
    def port(self) -> int:
        return int(_m().ncb_tcp_port(self._h))

    def connect(self, ports: Sequence[int], timeout_ms: int = 10000) -> None:
        arr = _i32(ports)
        if _m().ncb_tcp_connect(self._h, arr.ctypes.data, len(arr), timeout_ms) != 0:
            raise RuntimeError(last_error() or "ncb_tcp_connect failed")

    def all_reduce_sum(self, data: np.ndarray, timeout_ms: int = 60000) -> None:
        assert data.dtype == np.float32 and data.flags.c_contiguous
        if _m().ncb_tcp_all_reduce_sum(self._h, data.ctypes.data, data.size, timeout_ms) != 0:
            raise RuntimeError(last_error() or "ring all-reduce failed")

    def __del__(self):
        if getattr(self, "_h", None):
            _m().ncb_tcp_free(self._h)
            self._h = None


def memory_ring_all_reduce(rows: np.ndarray, drop_from: int = -1, timeout_ms: int = 60000) -> np.ndarray:
    """`world` threads reduce the rows of `rows` [world, count] with the ring over in-process mailboxes; returns the
    reduced rows (all equal). `drop_from` loses one message of that rank (the call then raises after the timeout)."""
    out = np.ascontiguousarray(rows, dtype=np.float32).copy()
    if _m().ncb_memory_ring_all_reduce(out.ctypes.data, out.shape[0], out.shape[1], drop_from, timeout_ms) != 0:
        raise RuntimeError(last_error() or "ring all-reduce failed")
    return out
