"""Policy-gradient step and the persistent worker that serves it over a line protocol.

`rl_step` is the reference's `RlStep` (`src/rl.cc`): zero the gradients, forward the rollout rows, backward with
per-position weights (the advantages) and the divisor `valid * num_passes * examples_per_rank` in place of the
valid-target count, then one optimizer step. With no valid target only the loss is returned.

`RlWorker` keeps model and optimizer alive between steps and speaks the reference's pipe protocol
(`src/rl_worker.h:15-67`): one ASCII line per message, first word the type, then `key=value` fields; lists are
comma separated; floats use `%.9g`. Requests: `rollout`, `advantage`, `save`, `ping`, `quit`; a failing
request answers `<type> ok=0 error=<message with _ for blanks>` and leaves the step counter alone.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, TextIO

import numpy as np
import torch

from ..models import GPT
from ..optim import Optimizer


@dataclass
class RlStepResult:
    loss: float
    grad_norm: float
    valid_targets: int
    divisor: int


@torch.no_grad()
def rl_step(model: GPT, optimizer: Optional[Optimizer], tokens, targets, advantages, num_passes: int,
            examples_per_rank: int, step: int) -> RlStepResult:
    if num_passes <= 0 or examples_per_rank <= 0:
        raise ValueError("rl_step: num_passes and examples_per_rank must be positive")
    dev = model.device
    tok = torch.as_tensor(np.asarray(tokens), device=dev).long()
    tgt = torch.as_tensor(np.asarray(targets), device=dev).long()
    adv = torch.as_tensor(np.asarray(advantages, dtype=np.float32), device=dev).reshape(-1)
    if tok.dim() != 2 or tok.shape != tgt.shape or adv.numel() != tok.numel():
        raise ValueError("rl_step: tokens, targets and advantages must share one [batch, seq] shape")
    valid = int((tgt != -1).sum().item())
    model.zero_grad()
    if valid == 0:
        return RlStepResult(float(model.forward_loss(tok, tgt)), 0.0, 0, 0)
    divisor = valid * num_passes * examples_per_rank
    loss = model.forward_backward(tok, tgt, row_weights=adv, divisor=float(divisor))
    gn = 0.0
    if optimizer is not None:
        optimizer.step(step)
        gn = optimizer.grad_norm()
    return RlStepResult(float(loss), gn, valid, divisor)


def _fields(words: Sequence[str]) -> Dict[str, str]:
    out = {}
    for w in words:
        if "=" in w:
            k, v = w.split("=", 1)
            out[k] = v
    return out


def _ints(text: str) -> List[int]:
    return [int(x) for x in text.split(",")] if text else []


def _floats(text: str) -> List[float]:
    return [float(x) for x in text.split(",")] if text else []


class RlWorker:
    """Holds the policy and its optimizer across steps; `serve` answers protocol lines until `quit` or EOF."""

    def __init__(self, model: GPT, optimizer: Optional[Optimizer], step: int = 0, engine=None):
        self.model, self.optimizer = model, optimizer
        self.step = step          # completed optimizer steps; the next step is step + 1
        self._engine = engine

    # -- requests -----------------------------------------------------------------------------------------
    def advantage(self, tokens, targets, advantages, batch: int, seq: int, num_passes: int,
                  examples_per_rank: int) -> RlStepResult:
        if batch <= 0 or seq <= 0:
            raise ValueError("batch and seq must be positive")
        n = batch * seq
        if len(tokens) != n or len(targets) != n or len(advantages) != n:
            raise ValueError(f"every list must hold batch*seq = {n} entries")
        res = rl_step(self.model, self.optimizer, np.asarray(tokens, dtype=np.int64).reshape(batch, seq),
                      np.asarray(targets, dtype=np.int64).reshape(batch, seq), advantages, num_passes,
                      examples_per_rank, self.step + 1)
        if res.valid_targets > 0:
            self.step += 1
        return res

    def rollout(self, prompts: Sequence[int], num_prompts: int, prompt_len: int, *, num_samples: int = 1,
                max_tokens: int = 16, temperature: float = 1.0, top_k: int = 0, seed: int = 0,
                stop_ids: Sequence[int] = (), bos_id: int = -1):
        from ..inference import GenerateParams, InferenceEngine, generate_multi
        if num_prompts <= 0 or prompt_len <= 0 or len(prompts) != num_prompts * prompt_len:
            raise ValueError("prompts must hold num_prompts * prompt_len ids")
        if self._engine is None:
            self._engine = InferenceEngine(self.model, use_cuda_graph=False)
        p = torch.as_tensor(np.asarray(prompts, dtype=np.int64).reshape(num_prompts, prompt_len))
        params = GenerateParams(max_tokens=max_tokens, temperature=temperature, top_k=top_k, seed=seed,
                                stop_ids=tuple(stop_ids), bos_id=bos_id, num_samples=num_samples)
        return generate_multi(self._engine, p, params)

    def save(self, path: str) -> None:
        from ..train.checkpointer import save_checkpoint
        save_checkpoint(path, self.model, self.optimizer, step=self.step, stage="rl")

    # -- protocol -----------------------------------------------------------------------------------------
    def handle(self, line: str) -> str:
        words = line.strip().split(" ")
        kind = words[0] if words and words[0] else "unknown"
        try:
            f = _fields(words[1:])
            if kind == "ping":
                return "pong ok=1"
            if kind == "quit":
                return "quit ok=1"
            if kind == "save":
                if "path" not in f:
                    raise ValueError("save needs path=")
                self.save(f["path"])
                return "save ok=1"
            if kind == "advantage":
                res = self.advantage(_ints(f.get("tokens", "")), _ints(f.get("targets", "")),
                                     _floats(f.get("advantages", "")), int(f["batch"]), int(f["seq"]),
                                     int(f["num_passes"]), int(f["examples_per_rank"]))
                return (f"advantage ok=1 step={self.step} loss={res.loss:.9g} grad_norm={res.grad_norm:.9g} "
                        f"valid_targets={res.valid_targets}")
            if kind == "rollout":
                stop = _ints(f.get("stop_ids", ""))
                if "stop_id" in f and int(f["stop_id"]) >= 0:
                    stop.append(int(f["stop_id"]))
                rows = self.rollout(_ints(f.get("prompts", "")), int(f["num_prompts"]), int(f["prompt_len"]),
                                    num_samples=int(f.get("num_samples", 1)), max_tokens=int(f["max_tokens"]),
                                    temperature=float(f.get("temperature", 1.0)), top_k=int(f.get("top_k", 0)),
                                    seed=int(f.get("seed", 0)), stop_ids=stop, bos_id=int(f.get("bos_id", -1)))
                lengths = ",".join(str(len(r.tokens)) for r in rows)
                masks = ",".join(str(int(m)) for r in rows for m in r.mask)
                toks = ",".join(str(int(t)) for r in rows for t in r.tokens)
                return (f"rollout ok=1 num_prompts={f['num_prompts']} num_samples={f.get('num_samples', 1)} "
                        f"rows={len(rows)} lengths={lengths} masks={masks} tokens={toks}")
            raise ValueError(f"unknown message type {kind}")
        except Exception as e:  # a failing request leaves the worker alive
            msg = "_".join(str(e).split()) or type(e).__name__
            return f"{kind} ok=0 error={msg}"

    def serve(self, inp: TextIO, out: TextIO) -> int:
        for line in inp:
            if not line.strip():
                continue
            reply = self.handle(line)
            out.write(reply + "\n")
            out.flush()
            if reply.startswith("quit ok=1"):
                break
        return 0
