"""Evaluation: bits per byte over a loader, per-position scoring, bits per byte over packed SFT rows.

Semantics follow the reference (`src/eval.cc:26-85` EvalBpb, `:87-204` ScoreBatch, `:206-300`
EvaluatePackedRows): losses are natural-log cross entropies of the soft-capped logits over the unpadded
vocabulary; a target of -1 is ignored; a target whose byte length is 0 (special tokens) counts neither nats
nor bytes; bpb = sum(nats) / (ln 2 * sum(bytes)).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..config import LOGIT_SOFTCAP
from ..models import GPT


def token_bytes_table(tokenizer) -> np.ndarray:
    """Byte length of every token id; special tokens count 0 (they are markup, not text)."""
    n = tokenizer.vocab_size
    specials = set()
    for name in ("<|bos|>", "<|user_start|>", "<|user_end|>", "<|assistant_start|>", "<|assistant_end|>",
                 "<|python_start|>", "<|python_end|>", "<|output_start|>", "<|output_end|>"):
        sid = tokenizer.special_id(name)
        if sid >= 0:
            specials.add(sid)
    out = np.zeros(n, dtype=np.int32)
    for i in range(n):
        if i not in specials:
            out[i] = len(tokenizer.decode_bytes([i]))
    return out


@torch.no_grad()
def eval_bpb(model: GPT, loader, steps: int, token_bytes: Optional[np.ndarray] = None) -> float:
    """Bits per byte over `steps` batches of `loader` (anything with `next() -> (tokens, targets)` int arrays).
    Without a byte table every valid target counts one byte (the result is then bits per token)."""
    if steps <= 0:
        return math.inf
    dev = model.device
    table = None if token_bytes is None else torch.as_tensor(np.asarray(token_bytes), dtype=torch.int64, device=dev)
    nats = torch.zeros((), dtype=torch.float64, device=dev)
    nbytes = torch.zeros((), dtype=torch.int64, device=dev)
    for _ in range(steps):
        try:
            tok, tgt = loader.next()
        except StopIteration:
            break
        tokens = torch.as_tensor(np.asarray(tok), device=dev).long()
        targets = torch.as_tensor(np.asarray(tgt), device=dev).long()
        _, rows = model.forward_loss(tokens, targets, return_rows=True)
        t = targets.reshape(-1)
        valid = t >= 0
        if table is None:
            b = valid.to(torch.int64)
        else:
            safe = t.clamp(0, table.numel() - 1)
            b = torch.where(valid & (t < table.numel()), table[safe], torch.zeros_like(safe))
        use = b > 0
        nats += (rows.reshape(-1).double() * use).sum()
        nbytes += b.sum()
    total = int(nbytes.item())
    if total == 0:
        return math.inf
    return float(nats.item() / (math.log(2.0) * total))


@dataclass
class ScoreResult:
    nll: List[float] = field(default_factory=list)        # [seq]; position p scores token p+1; 0 past length-1
    argmax: List[int] = field(default_factory=list)       # [seq]; -1 past length-1
    focus_logits: List[float] = field(default_factory=list)


@torch.no_grad()
def score_batch(model: GPT, tokens, lengths: Optional[Sequence[int]] = None,
                focus: Optional[Sequence[Optional[tuple]]] = None) -> List[ScoreResult]:
    """Per-position negative log-likelihood and greedy prediction for every row of `tokens` [B, T].

    `focus[b] = (position, ids)` additionally returns the soft-capped logits of `ids` at `position` (used by
    multiple-choice tasks to compare answer letters); ids outside the vocabulary give 0."""
    dev = model.device
    tokens = torch.as_tensor(np.asarray(tokens), device=dev).long()
    B, T = tokens.shape
    if lengths is None:
        lens = torch.full((B,), T, dtype=torch.long, device=dev)
    else:
        lens = torch.as_tensor(np.asarray(lengths), device=dev).long().clamp(0, T)
    pos = torch.arange(T, device=dev)[None, :]
    has_next = (pos + 1) < lens[:, None]
    targets = torch.full((B, T), -1, dtype=torch.long, device=dev)
    targets[:, :-1] = tokens[:, 1:]
    targets = torch.where(has_next, targets, torch.full_like(targets, -1))
    _, rows = model.forward_loss(tokens, targets, return_rows=True)
    nll = torch.where(has_next, rows.view(B, T).float(), torch.zeros((), device=dev)).cpu()
    logits = model.logits(tokens)                                   # [B, T, vocab] fp32, before the soft cap
    arg = torch.where(has_next, logits.argmax(-1), torch.full((B, T), -1, dtype=torch.long, device=dev)).cpu()
    out = []
    for b in range(B):
        r = ScoreResult(nll=nll[b].tolist(), argmax=arg[b].tolist())
        if focus is not None and focus[b] is not None:
            p, ids = focus[b]
            if 0 <= p < T and len(ids) > 0:
                V = logits.shape[-1]
                row = logits[b, p].cpu()
                row = LOGIT_SOFTCAP * torch.tanh(row / LOGIT_SOFTCAP)
                r.focus_logits = [float(row[i]) if 0 <= i < V else 0.0 for i in ids]
        out.append(r)
    return out


@dataclass
class PackedBpb:
    bpb: float = math.inf
    valid_targets: int = 0
    target_bytes: int = 0


@torch.no_grad()
def evaluate_packed_rows(model: GPT, tokens: np.ndarray, targets: np.ndarray, token_bytes: np.ndarray,
                         device_batch: int, eval_steps: int) -> PackedBpb:
    """Bits per byte over the first `eval_steps * device_batch` packed rows ([rows, seq] arrays; -1 = masked)."""
    if device_batch <= 0 or eval_steps <= 0:
        raise ValueError("device_batch and eval_steps must be positive")
    rows, seq = tokens.shape
    if eval_steps * device_batch > rows:
        raise ValueError(f"the validation shard holds {rows} rows, fewer than the {eval_steps * device_batch} that "
                         "eval_steps * device_batch reads in one pass")
    dev = model.device
    table = np.asarray(token_bytes)
    nats, nbytes, nvalid = 0.0, 0, 0
    for s in range(eval_steps):
        sl = slice(s * device_batch, (s + 1) * device_batch)
        tg = targets[sl]
        valid = int((tg >= 0).sum())
        if valid == 0:
            continue
        if int(tg.max()) >= table.size:
            raise ValueError(f"the shard targets token {int(tg.max())}, which the token-byte table does not cover")
        loss = model.forward_loss(torch.as_tensor(np.array(tokens[sl]), device=dev).long(),
                                  torch.as_tensor(np.array(tg), device=dev).long())
        loss = float(loss)
        if not math.isfinite(loss):
            raise FloatingPointError(f"the model returned a non-finite loss for evaluation step {s}")
        nats += loss * valid
        b = table[np.clip(tg, 0, None)] * (tg >= 0)
        nbytes += int(np.clip(b, 0, None).sum())
        nvalid += valid
    if nbytes <= 0:
        raise ValueError("the packed validation rows hold no valid target bytes")
    return PackedBpb(bpb=nats / (math.log(2.0) * nbytes), valid_targets=nvalid, target_bytes=nbytes)
