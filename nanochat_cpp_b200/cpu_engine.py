"""ctypes binding of the native engines behind the C ABI (the model / optimizer / generate / score part of
`include/nanochat/capi.h`). By default a model lives in the C++ CPU engine (`csrc/host/engine.cc`): useful on
machines without a GPU and as an oracle that shares no code with the PyTorch path. After `select_device("cuda:0")`
the same calls create and drive a model in the C++ GPU engine (`csrc/gpu/gpu_engine.cc`, the sm_100a kernels without
Python or PyTorch in the loop), which is what the native command line and hosts in other languages use."""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from .config import Config
from .data.native import last_error, lib


class _ConfigC(C.Structure):
    _fields_ = [("num_layers", C.c_int), ("num_heads", C.c_int), ("num_kv_heads", C.c_int), ("hidden_dim", C.c_int),
                ("seq_len", C.c_int), ("vocab_size", C.c_int), ("padded_vocab_size", C.c_int),
                ("rope_base", C.c_float), ("window_pattern", C.c_char_p), ("value_embedding", C.c_int)]


class _ParamC(C.Structure):
    _fields_ = [("name", C.c_char_p), ("value", C.c_void_p), ("grad", C.c_void_p), ("count", C.c_int64),
                ("rows", C.c_int), ("cols", C.c_int)]


class _OptimC(C.Structure):
    _fields_ = [(n, C.c_float) for n in ("unembedding_lr", "embedding_lr", "matrix_lr", "scalar_lr", "weight_decay")] + \
               [("muon_ns_steps", C.c_int)] + [(n, C.c_float) for n in ("muon_beta2", "adam_eps", "clip")] + \
               [("num_iterations", C.c_int), ("warmup_steps", C.c_int)] + \
               [(n, C.c_float) for n in ("warmdown_ratio", "final_lr_frac", "weight_decay_base",
                                         "muon_momentum_warmup_steps", "muon_momentum_start", "muon_momentum_peak",
                                         "muon_momentum_final")]


class _GenC(C.Structure):
    _fields_ = [("num_samples", C.c_int), ("max_tokens", C.c_int), ("temperature", C.c_float), ("top_k", C.c_int),
                ("seed", C.c_uint64), ("stop_id", C.c_int), ("bos_id", C.c_int), ("stop_ids", C.POINTER(C.c_int))]


class _SeqC(C.Structure):
    _fields_ = [("count", C.c_int), ("tokens", C.POINTER(C.c_int)), ("mask", C.POINTER(C.c_uint8)),
                ("lengths", C.POINTER(C.c_int)), ("offsets", C.POINTER(C.c_int))]


class _FocusC(C.Structure):
    _fields_ = [("position", C.c_int), ("ids", C.POINTER(C.c_int)), ("count", C.c_int)]


class _ScoreC(C.Structure):
    _fields_ = [("nll", C.POINTER(C.c_float)), ("argmax", C.POINTER(C.c_int)), ("focus_logits", C.POINTER(C.c_float))]


_ready = False


def _l():
    global _ready
    L = lib()
    if not _ready:
        L.nanochat_model_create.restype = C.c_void_p
        L.nanochat_model_create.argtypes = [C.POINTER(_ConfigC), C.c_uint64]
        L.nanochat_model_free.argtypes = [C.c_void_p]
        L.nanochat_forward_loss.restype = C.c_float
        L.nanochat_forward_loss.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        L.nanochat_backward.argtypes = [C.c_void_p]
        L.nanochat_backward_accumulate.argtypes = [C.c_void_p, C.c_float]
        L.nanochat_backward_weighted.argtypes = [C.c_void_p, C.c_void_p, C.c_float]
        L.nanochat_zero_grad.argtypes = [C.c_void_p]
        L.nanochat_param_count.argtypes = [C.c_void_p]
        L.nanochat_param_info.argtypes = [C.c_void_p, C.c_int, C.POINTER(_ParamC)]
        for f in (L.nanochat_param_read, L.nanochat_param_write):
            f.restype = C.c_int64
            f.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int64, C.c_int64, C.c_void_p]
        L.nanochat_save.argtypes = [C.c_void_p, C.c_char_p]
        L.nanochat_load.argtypes = [C.c_void_p, C.c_char_p]
        L.nanochat_optim_create.restype = C.c_void_p
        L.nanochat_optim_create.argtypes = [C.c_void_p, C.POINTER(_OptimC)]
        L.nanochat_optim_step.argtypes = [C.c_void_p, C.c_int]
        L.nanochat_optim_grad_norm.restype = C.c_float
        L.nanochat_optim_grad_norm.argtypes = [C.c_void_p]
        L.nanochat_optim_free.argtypes = [C.c_void_p]
        L.nanochat_optim_config_preset.argtypes = [C.c_char_p, C.POINTER(_OptimC)]
        L.nanochat_rl_step.restype = C.c_float
        L.nanochat_rl_step.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                       C.c_int, C.c_int, C.c_int]
        L.nanochat_generate.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.POINTER(_GenC), C.POINTER(_SeqC)]
        L.nanochat_score_batch.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                           C.c_void_p]
        _ready = True
    return L


def select_device(name: str = "cpu") -> None:
    """"cpu", "cuda" or "cuda:N": the engine that models created afterwards live in (process-wide)."""
    L = _l()
    L.nanochat_select_device.argtypes = [C.c_char_p]
    if L.nanochat_select_device(name.encode()) != 0:
        raise RuntimeError(last_error() or f"cannot select device {name!r}")


def backend() -> str:
    L = _l()
    L.nanochat_backend.restype = C.c_char_p
    return L.nanochat_backend().decode()


def device_count() -> int:
    return int(_l().nanochat_device_count())


def _i32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a), dtype=np.int32)


class CpuModel:
    def __init__(self, cfg: Config, seed: int = 0):
        self.cfg = cfg
        c = _ConfigC(cfg.num_layers, cfg.num_heads, cfg.num_kv_heads, cfg.hidden_dim, cfg.seq_len, cfg.vocab_size,
                     cfg.padded_vocab_size, cfg.rope_base, cfg.window_pattern.encode(), int(cfg.value_embedding))
        self._h = _l().nanochat_model_create(C.byref(c), seed)
        if not self._h:
            raise RuntimeError(last_error() or "nanochat_model_create failed")
        self._index: Dict[str, Tuple[int, int, int, int]] = {}
        info = _ParamC()
        for i in range(_l().nanochat_param_count(self._h)):
            _l().nanochat_param_info(self._h, i, C.byref(info))
            self._index[info.name.decode()] = (i, info.count, info.rows, info.cols)

    def names(self) -> List[str]:
        return list(self._index)

    def read(self, name: str, grad: bool = False) -> np.ndarray:
        i, n, _, _ = self._index[name]
        out = np.empty(n, dtype=np.float32)
        _l().nanochat_param_read(self._h, i, int(grad), 0, n, out.ctypes.data)
        return out

    def write(self, name: str, values) -> None:
        i, n, _, _ = self._index[name]
        v = np.ascontiguousarray(np.asarray(values, dtype=np.float32).reshape(-1))
        assert v.size == n, (name, v.size, n)
        _l().nanochat_param_write(self._h, i, 0, 0, n, v.ctypes.data)

    def forward_loss(self, tokens, targets) -> float:
        t, g = _i32(tokens), _i32(targets)
        return float(_l().nanochat_forward_loss(self._h, t.ctypes.data, g.ctypes.data, t.shape[0], t.shape[1]))

    def backward(self, scale: float = 1.0, row_weights=None) -> None:
        if row_weights is not None:
            w = np.ascontiguousarray(np.asarray(row_weights, dtype=np.float32).reshape(-1))
            _l().nanochat_backward_weighted(self._h, w.ctypes.data, scale)
        elif scale == 1.0:
            _l().nanochat_backward(self._h)
        else:
            _l().nanochat_backward_accumulate(self._h, scale)

    def zero_grad(self) -> None:
        _l().nanochat_zero_grad(self._h)

    def train_step(self, tokens, targets, optimizer: "CpuOptimizer" = None) -> float:
        """zero_grad + forward + backward (+ one optimizer step): `nanochat_train_step`."""
        t, g = _i32(tokens), _i32(targets)
        L = _l()
        L.nanochat_train_step.restype = C.c_float
        L.nanochat_train_step.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        return float(L.nanochat_train_step(self._h, optimizer._h if optimizer is not None else None, t.ctypes.data,
                                           g.ctypes.data, t.shape[0], t.shape[1]))

    def device_status(self) -> int:
        L = _l()
        L.ncb_model_device_status.argtypes = [C.c_void_p]
        return int(L.ncb_model_device_status(self._h))

    def activation(self, name: str, layer: int = -1) -> np.ndarray:
        """fp32 copy of an activation the last forward kept on a CUDA device (`ncb_model_read_activation`)."""
        L = _l()
        L.ncb_model_read_activation.restype = C.c_int64
        L.ncb_model_read_activation.argtypes = [C.c_void_p, C.c_char_p, C.c_int, C.c_void_p, C.c_int64]
        n = L.ncb_model_read_activation(self._h, name.encode(), layer, None, 0)
        if n < 0:
            raise KeyError(name)
        out = np.empty(n, dtype=np.float32)
        L.ncb_model_read_activation(self._h, name.encode(), layer, out.ctypes.data, n)
        return out

    def launch_count(self) -> int:
        L = _l()
        L.ncb_model_launch_count.restype = C.c_int64
        L.ncb_model_launch_count.argtypes = [C.c_void_p]
        return int(L.ncb_model_launch_count(self._h))

    def save(self, path: str) -> None:
        _l().nanochat_save(self._h, path.encode())

    def load(self, path: str) -> None:
        _l().nanochat_load(self._h, path.encode())

    def generate(self, prompt: Sequence[int], *, num_samples=1, max_tokens=16, temperature=0.0, top_k=0, seed=0,
                 stop_id=-1, bos_id=-1):
        p = _i32(prompt)
        g = _GenC(num_samples, max_tokens, temperature, top_k, seed, stop_id, bos_id, None)
        out = _SeqC()
        _l().nanochat_generate(self._h, p.ctypes.data, p.size, C.byref(g), C.byref(out))
        rows = []
        for r in range(out.count):
            a, n = out.offsets[r], out.lengths[r]
            rows.append(([out.tokens[a + k] for k in range(n)], [out.mask[a + k] for k in range(n)]))
        return rows

    def score(self, tokens, lengths=None, focus=None):
        t = _i32(tokens)
        B, T = t.shape
        ln = _i32(lengths) if lengths is not None else None
        keep, fc = [], None
        if focus is not None:
            fc = (_FocusC * B)()
            for b in range(B):
                if focus[b] is None:
                    fc[b] = _FocusC(-1, None, 0)
                else:
                    ids = _i32(focus[b][1])
                    keep.append(ids)
                    fc[b] = _FocusC(int(focus[b][0]), ids.ctypes.data_as(C.POINTER(C.c_int)), ids.size)
        res = (_ScoreC * B)()
        _l().nanochat_score_batch(self._h, t.ctypes.data, B, T, ln.ctypes.data if ln is not None else None,
                                  C.cast(fc, C.c_void_p) if fc is not None else None, C.cast(res, C.c_void_p))
        out = []
        for b in range(B):
            nf = 0 if focus is None or focus[b] is None else len(focus[b][1])
            out.append(([res[b].nll[p] for p in range(T)], [res[b].argmax[p] for p in range(T)],
                        [res[b].focus_logits[k] for k in range(nf)]))
        return out

    def __del__(self):
        if getattr(self, "_h", None) and _l is not None:      # module globals may be gone at interpreter exit
            _l().nanochat_model_free(self._h)
            self._h = None


NativeModel = CpuModel      # the same handle drives the GPU engine once a CUDA device is selected


class CpuOptimizer:
    def __init__(self, model: CpuModel, **fields):
        c = _OptimC()
        _l().nanochat_optim_config_preset(b"default", C.byref(c))
        for k, v in fields.items():
            setattr(c, k, v)
        self.model = model
        self._h = _l().nanochat_optim_create(model._h, C.byref(c))

    def step(self, step: int) -> None:
        _l().nanochat_optim_step(self._h, step)

    def grad_norm(self) -> float:
        return float(_l().nanochat_optim_grad_norm(self._h))

    def rl_step(self, tokens, targets, advantages, num_passes: int, examples_per_rank: int, step: int) -> float:
        t, g = _i32(tokens), _i32(targets)
        a = np.ascontiguousarray(np.asarray(advantages, dtype=np.float32))
        return float(_l().nanochat_rl_step(self.model._h, self._h, t.ctypes.data, g.ctypes.data, a.ctypes.data,
                                           t.shape[0], t.shape[1], num_passes, examples_per_rank, step))

    def __del__(self):
        if getattr(self, "_h", None) and _l is not None:
            _l().nanochat_optim_free(self._h)
            self._h = None


NativeOptimizer = CpuOptimizer
