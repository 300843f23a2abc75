"""The user-facing Python API, with the names and call shapes of the reference's `nanochat_cpp` package
(python/nanochat_cpp/api.py): `Config`, `Tokenizer`, `Model`, `Optimizer`, `TokenData`, `Trainer`, `Evaluator`,
`no_grad`, `evaluate`, `model_flags`. The objects wrap this package's engine (models.GPT, optim.Optimizer, the
native tokenizer and loader) instead of a C handle; on a GPU every operator runs the sm_100a kernels.
"""
from __future__ import annotations

import glob
import os
from dataclasses import dataclass
from typing import Iterable, List, Optional, Sequence

import numpy as np
import torch

from . import config as _config
from .data import native as _native
from .models import GPT
from .optim import Optimizer as _Optimizer
from .optim import OptimizerConfig, SchedulerConfig

ASPECT_RATIO = 64
HEAD_DIM = 128
PAD_VOCAB_TO = 64


class Config(_config.Config):
    """`Config(depth)` derives hidden = depth * aspect_ratio rounded up to a multiple of head_dim and
    heads = hidden / head_dim (reference api.py:269-310); every field can be given explicitly."""

    def __init__(self, depth: Optional[int] = None, *, num_layers: Optional[int] = None,
                 num_heads: Optional[int] = None, num_kv_heads: Optional[int] = None,
                 hidden_dim: Optional[int] = None, seq_len: int = 2048, vocab_size: int = 32768,
                 padded_vocab_size: Optional[int] = None, rope_base: float = 100000.0, window_pattern: str = "SSSL",
                 aspect_ratio: int = ASPECT_RATIO, head_dim: int = HEAD_DIM, value_embedding: bool = True,
                 short_window_override: int = 0):
        if num_layers is None:
            num_layers = int(depth) if depth is not None else 12
        if hidden_dim is None:
            hidden_dim = (num_layers * aspect_ratio + head_dim - 1) // head_dim * head_dim
        if num_heads is None:
            num_heads = max(1, hidden_dim // head_dim)
        if num_kv_heads is None:
            num_kv_heads = num_heads
        if padded_vocab_size is None:
            padded_vocab_size = (vocab_size + PAD_VOCAB_TO - 1) // PAD_VOCAB_TO * PAD_VOCAB_TO
        super().__init__(num_layers=int(num_layers), num_heads=int(num_heads), num_kv_heads=int(num_kv_heads),
                         hidden_dim=int(hidden_dim), seq_len=int(seq_len), vocab_size=int(vocab_size),
                         padded_vocab_size=int(padded_vocab_size), rope_base=float(rope_base),
                         window_pattern=str(window_pattern), value_embedding=bool(value_embedding),
                         short_window_override=int(short_window_override))


def model_flags(config: Optional[_config.Config] = None) -> List[str]:
    """The command-line flags that describe `config` (for `python -m nanochat_cpp_b200.cli ...`)."""
    c = config or Config()
    out = ["--layers", str(c.num_layers), "--heads", str(c.num_heads), "--kv-heads", str(c.num_kv_heads),
           "--hidden", str(c.hidden_dim), "--seq", str(c.seq_len), "--vocab", str(c.vocab_size),
           "--padded-vocab", str(c.padded_vocab_size), "--rope-base", repr(float(c.rope_base)),
           "--window-pattern", c.window_pattern]
    if not c.value_embedding:
        out.append("--no-value-embedding")
    return out


class Tokenizer:
    def __init__(self, inner: _native.Tokenizer):
        self._t = inner

    @classmethod
    def load(cls, path) -> "Tokenizer":
        return cls(_native.Tokenizer.load(os.fspath(path)))

    @property
    def vocab_size(self) -> int:
        return self._t.vocab_size

    def encode_special(self, name: str) -> int:
        return self._t.special_id(name)

    def get_bos_token_id(self) -> int:
        return self._t.bos_id

    def encode(self, text, prepend: int = -1, append: int = -1):
        if isinstance(text, str):
            return self._t.encode(text, prepend=prepend, append=append)
        return [self._t.encode(t, prepend=prepend, append=append) for t in text]

    def decode(self, ids) -> str:
        return self._t.decode(list(ids))

    @property
    def handle(self):
        return self._t


def tokenizer(path) -> Tokenizer:
    return Tokenizer.load(path)


@dataclass
class ParamView:
    name: str
    shape: tuple
    value: torch.Tensor
    grad: torch.Tensor

    @property
    def is_matrix(self) -> bool:
        return len(self.shape) == 2


@dataclass
class GeneratedRow:
    tokens: List[int]
    mask: List[int]


@dataclass
class ScoreReport:
    nll: List[List[float]]
    argmax: List[List[int]]
    focus_logits: List[List[float]]


def _default_device():
    return torch.device("cuda") if torch.cuda.is_available() else torch.device("cpu")


def _ids(x, device) -> torch.Tensor:
    return torch.as_tensor(np.asarray(x), device=device).long()


class Model:
    def __init__(self, config: _config.Config, device=None, seed: int = 0, dtype: Optional[str] = None):
        self.device = torch.device(device) if device is not None else _default_device()
        dt = {"bf16": torch.bfloat16, "fp32": torch.float32, None: torch.bfloat16 if self.device.type == "cuda"
              else torch.float32}[dtype]
        self.config = config
        self.gpt = GPT(config, self.device, dt, seed=seed)
        self._batch = None
        self._grad_enabled = True

    @classmethod
    def from_checkpoint(cls, path, device=None) -> "Model":
        from .train.checkpointer import load_checkpoint
        dev = torch.device(device) if device is not None else _default_device()
        gpt, _ = load_checkpoint(os.fspath(path), device=dev,
                                 dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32)
        m = cls.__new__(cls)
        m.device, m.config, m.gpt, m._batch, m._grad_enabled = dev, gpt.cfg, gpt, None, True
        return m

    def _shape(self, tokens, batch, seq):
        t = _ids(tokens, self.device)
        if t.dim() == 1:
            t = t.view(batch if batch else -1, seq if seq else self.config.seq_len)
        return t

    def forward_loss(self, tokens, targets, batch: Optional[int] = None, seq: Optional[int] = None) -> float:
        tok, tgt = self._shape(tokens, batch, seq), self._shape(targets, batch, seq)
        self._batch = (tok, tgt)
        return float(self.gpt.forward_loss(tok, tgt))

    def _backward(self, scale: float, row_weights=None, divisor=None) -> None:
        if self._batch is None:
            raise RuntimeError("backward() needs a forward_loss() call first")
        if not self._grad_enabled:
            raise RuntimeError("backward() inside no_grad()")
        tok, tgt = self._batch
        self.gpt.forward_backward(tok, tgt, grad_scale=scale, row_weights=row_weights, divisor=divisor)

    def backward(self) -> None:
        self._backward(1.0)

    def backward_accumulate(self, scale: float = 1.0) -> None:
        self._backward(float(scale))

    def backward_weighted(self, row_weights, scale: float = 1.0) -> None:
        """Gradient of sum(row_weights * nll) * scale / valid_targets (the RL step's backward)."""
        w = torch.as_tensor(np.asarray(row_weights, dtype=np.float32), device=self.device).reshape(-1)
        valid = int((self._batch[1] != -1).sum().item())
        self._backward(1.0, row_weights=w, divisor=valid / float(scale) if scale else None)

    def train_step(self, tokens, targets, optimizer=None, batch=None, seq=None, step: Optional[int] = None) -> float:
        tok, tgt = self._shape(tokens, batch, seq), self._shape(targets, batch, seq)
        self.gpt.zero_grad()
        loss = float(self.gpt.forward_backward(tok, tgt))
        if optimizer is not None:
            optimizer.step(step if step is not None else optimizer.steps_done + 1)
        return loss

    def zero_grad(self) -> None:
        self.gpt.zero_grad()

    def param_count(self) -> int:
        return len(self.gpt.params.specs)

    def param_total(self) -> int:
        return self.gpt.num_params()

    @property
    def dtype(self) -> str:
        return "bf16" if self.gpt.dtype == torch.bfloat16 else "fp32"

    def params(self) -> List[ParamView]:
        P = self.gpt.params
        return [ParamView(s.name, tuple(s.shape), P.m(s.name), P.g(s.name)) for s in P.specs]

    def save(self, path) -> None:
        from .train.checkpointer import save_checkpoint
        save_checkpoint(os.fspath(path), self.gpt)

    def load(self, path) -> None:
        from .train.checkpointer import load_checkpoint
        load_checkpoint(os.fspath(path), self.gpt)

    def generate(self, prompt, max_tokens: int = 256, temperature: float = 1.0, top_k: int = 0, seed: int = 0,
                 num_samples: int = 1, stop_id: int = -1, bos_id: int = -1) -> List[GeneratedRow]:
        from .inference import GenerateParams, InferenceEngine, generate
        if not hasattr(self, "_engine"):
            self._engine = InferenceEngine(self.gpt)
        rows = generate(self._engine, list(prompt), GenerateParams(num_samples=num_samples, max_tokens=max_tokens,
                                                                   temperature=temperature, top_k=top_k, seed=seed,
                                                                   stop_id=stop_id, bos_id=bos_id))
        return [GeneratedRow(r.tokens, r.mask) for r in rows]

    def no_grad(self):
        return no_grad(self)


class Optimizer:
    """`Optimizer(model, matrix_lr=..., warmup_steps=..., num_iterations=...)`: optimizer and schedule fields in one
    keyword list, as the reference's flat `nanochat_optim_config`."""

    def __init__(self, model: Model, **fields):
        oc, sc = OptimizerConfig(), SchedulerConfig()
        for k, v in fields.items():
            if hasattr(oc, k):
                setattr(oc, k, type(getattr(oc, k))(v))
            elif hasattr(sc, k):
                setattr(sc, k, type(getattr(sc, k))(v))
            else:
                raise TypeError(f"unknown optimizer field {k!r}")
        self.num_iterations = sc.num_iterations
        self.model = model
        self.inner = _Optimizer(model.gpt.params, oc, sc)
        self.steps_done = 0

    def step(self, step: int) -> None:
        self.inner.step(int(step))
        self.steps_done = int(step)

    def grad_norm(self) -> float:
        return self.inner.grad_norm()

    def zero_grad(self) -> None:
        self.model.zero_grad()


def _expand(patterns) -> List[str]:
    if isinstance(patterns, (str, os.PathLike)):
        patterns = [patterns]
    out: List[str] = []
    for p in patterns:
        hits = sorted(glob.glob(os.fspath(p)))
        out.extend(hits if hits else [os.fspath(p)])
    return out


class TokenData:
    """Packed (tokens, targets) batches from parquet shards (BOS-aligned best-fit packing in the native loader)."""

    def __init__(self, parquet, tokenizer: Tokenizer, seq_len: int, batch: int = 1, text_column: str = "text",
                 buffer_docs: int = 1000, rank: int = 0, world: int = 1):
        self._paths, self._tok, self._seq, self._batch = _expand(parquet), tokenizer, int(seq_len), int(batch)
        self._kw = dict(text_column=text_column, buffer_docs=buffer_docs, rank=rank, world=world)
        self._open()

    def _open(self):
        self._loader = _native.DataLoader.from_parquet(self._paths, self._tok.handle, self._batch, self._seq,
                                                       **self._kw)

    def reset(self) -> None:
        self._open()

    def rebatch(self, batch: int) -> "TokenData":
        return TokenData(self._paths, self._tok, self._seq, batch, **self._kw)

    def next(self):
        return self._loader.next()

    def token_bytes(self) -> np.ndarray:
        from .eval import token_bytes_table
        return token_bytes_table(self._tok.handle)


class Trainer:
    """Iterating yields `(step, mean micro-batch loss)`; one optimizer step per iteration (reference api.py:966)."""

    def __init__(self, model: Model, data: TokenData, batch: Optional[int] = None, total_batch: Optional[int] = None,
                 warmup_steps: Optional[int] = None, num_iterations: Optional[int] = None,
                 optimizer: Optional[Optimizer] = None, grad_accum: Optional[int] = None,
                 optimizer_config: Optional[dict] = None, scheduler_config: Optional[dict] = None):
        if batch is not None and int(batch) != data._batch:
            data = data.rebatch(int(batch))
        self.model, self.data, self.batch, self.seq = model, data, data._batch, data._seq
        if grad_accum is None:
            grad_accum = max(1, int(total_batch) // (self.batch * self.seq)) if total_batch else 1
        self.grad_accum = max(1, int(grad_accum))
        self.num_iterations = int(num_iterations or getattr(optimizer, "num_iterations", 0) or 1)
        if optimizer is None:
            opts = dict(optimizer_config or {})
            opts.update(scheduler_config or {})
            if warmup_steps is not None:
                opts["warmup_steps"] = int(warmup_steps)
            opts.setdefault("num_iterations", self.num_iterations)
            optimizer = Optimizer(model, **opts)
        self.optimizer = optimizer
        self._step = 0

    def __iter__(self):
        return self

    def __len__(self) -> int:
        return self.num_iterations

    def __next__(self):
        if self._step >= self.num_iterations:
            raise StopIteration
        step = self._step + 1
        self.model.zero_grad()
        total = 0.0
        for _ in range(self.grad_accum):
            tok, tgt = self.data.next()
            dev = self.model.device
            total += float(self.model.gpt.forward_backward(_ids(tok, dev), _ids(tgt, dev),
                                                           grad_scale=1.0 / self.grad_accum))
        self.optimizer.step(step)
        self._step = step
        return step, total / self.grad_accum

    def save(self, path) -> None:
        from .train.checkpointer import save_checkpoint
        save_checkpoint(os.fspath(path), self.model.gpt, self.optimizer.inner, step=self._step)


class Evaluator:
    def __init__(self, model: Model):
        self.model = model

    def bpb(self, data: TokenData, steps: int) -> float:
        from .eval import eval_bpb
        return eval_bpb(self.model.gpt, data, steps, data.token_bytes())

    def score(self, tokens, lengths=None, focus=None) -> ScoreReport:
        from .eval import score_batch
        res = score_batch(self.model.gpt, tokens, lengths, focus)
        return ScoreReport([r.nll for r in res], [r.argmax for r in res], [r.focus_logits for r in res])

    def generate(self, prompt, **kwargs) -> List[GeneratedRow]:
        return self.model.generate(prompt, **kwargs)


class _NoGrad:
    def __init__(self, model: Optional[Model] = None):
        self.model = model

    def __enter__(self):
        if self.model is not None:
            self._prev, self.model._grad_enabled = self.model._grad_enabled, False
        return self

    def __exit__(self, *exc):
        if self.model is not None:
            self.model._grad_enabled = self._prev
        return False


def no_grad(model: Optional[Model] = None) -> _NoGrad:
    return _NoGrad(model)


def evaluate(model: Model, parquet, tokenizer: Tokenizer, tokens: Optional[int] = None, batch: int = 1,
             steps: Optional[int] = None) -> float:
    """Bits per byte of `model` on parquet shards; `tokens` is the token budget (steps = tokens / (batch * seq))."""
    seq = model.config.seq_len
    data = TokenData(parquet, tokenizer, seq, batch)
    n = steps or max(1, int(tokens or batch * seq) // (batch * seq))
    return Evaluator(model).bpb(data, n)
