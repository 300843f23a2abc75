"""SFT data: a deterministic task mixture and the BOS-aligned best-fit packer.

The packer is the reference's (python/nanochat_cpp/sft_data.py `PackedRowStream`, itself a restatement of
upstream's `sft_data_generator_bos_bestfit`): a buffer of `buffer_size` rendered conversations; a row of
`seq_len + 1` tokens takes, again and again, the longest buffered conversation that still fits; when none fits
the rest of the row is padded with BOS (SFT never crops a conversation); conversations longer than a row are
skipped. Targets are the next token where the mask is 1 and -1 elsewhere, including the padding.
"""
from __future__ import annotations

import random
from typing import Callable, List, Optional, Sequence, Tuple

import numpy as np


class TaskMixture:
    """Several tasks shuffled together with a fixed seed; list a task twice to oversample it."""

    def __init__(self, tasks: Sequence, seed: int = 42):
        self.tasks = list(tasks)
        self.index_map = [(t, i) for t, task in enumerate(self.tasks) for i in range(len(task))]
        random.Random(seed).shuffle(self.index_map)

    def __len__(self) -> int:
        return len(self.index_map)

    def __getitem__(self, index: int) -> dict:
        t, i = self.index_map[index]
        return self.tasks[t][i]


class PackedRowStream:
    """One epoch of packed rows; counters (`rows`, `iterations`, `consumed`, `epoch`, `progress`, `last_step`) can
    be read after each row."""

    def __init__(self, conversations, tokenizer, seq_len: int, render: Optional[Callable] = None, *,
                 buffer_size: int = 100, render_max_tokens: int = 2048, batch: int = 1, num_iterations: int = 0,
                 rank: int = 0, world_size: int = 1):
        if len(conversations) <= 0:
            raise ValueError("the SFT conversation list is empty")
        if seq_len < 1 or buffer_size < 1 or world_size < 1 or batch < 1:
            raise ValueError("seq_len, buffer_size, world_size and batch must be positive")
        if not 0 <= rank < len(conversations):
            raise ValueError(f"rank {rank} is outside the dataset ({len(conversations)})")
        if render is None:
            from .render import render_conversation
            render = lambda c, t: render_conversation(c, t, max_tokens=render_max_tokens)  # noqa: E731
        self._conv, self._tok, self._render = conversations, tokenizer, render
        self._n, self._seq, self._cap = len(conversations), int(seq_len), int(seq_len) + 1
        bos = getattr(tokenizer, "get_bos_token_id", None)
        self._bos = bos() if bos else tokenizer.bos_id
        self._buffer_size, self._batch, self._iters_total, self._world = buffer_size, batch, num_iterations, world_size
        self._buffer: List[Tuple[List[int], List[int]]] = []
        self._cursor = self.consumed = int(rank)
        self.epoch, self.iterations, self.rows = 1, 0, 0
        self._in_batch, self._stall, self._done = 0, 0, False
        self.approx_progress = self.progress = 0.0
        self.last_step = False

    def __iter__(self):
        return self

    def __next__(self):
        if self._done:
            raise StopIteration
        row = self._next_row()
        self.rows += 1
        self._in_batch += 1
        if self._in_batch >= self._batch:
            self._in_batch = 0
            self.iterations += 1
            self.approx_progress = (self.iterations / self._iters_total if self._iters_total > 0
                                    else self.consumed / self._n)
            self.progress = max(self.progress, self.approx_progress)
            self.last_step = self.consumed >= self._n or 0 < self._iters_total <= self.iterations
            self._done = self.last_step
        return row

    def _refill(self) -> None:
        while len(self._buffer) < self._buffer_size:
            ids, mask = self._render(self._conv[self._cursor], self._tok)
            self._cursor += self._world
            if self._cursor >= self._n:
                self._cursor %= self._n
                self.epoch += 1
            if len(ids) > self._cap:
                self._stall += 1
                if self._stall >= self._n:
                    raise ValueError(f"no conversation fits one row of {self._cap} tokens")
                continue
            self._stall = 0
            self._buffer.append((list(ids), list(mask)))

    def _next_row(self):
        row: List[int] = []
        keep: List[int] = []
        content = self._cap
        while len(row) < self._cap:
            self._refill()
            room = self._cap - len(row)
            best, best_len = -1, 0
            for i, (ids, _) in enumerate(self._buffer):
                if best_len < len(ids) <= room:
                    best, best_len = i, len(ids)
            if best < 0:
                content = len(row)
                row += [self._bos] * room
                keep += [0] * room
                break
            ids, mask = self._buffer.pop(best)
            row += ids
            keep += mask
            self.consumed += self._world
        inputs = row[:self._seq]
        targets = [t if k else -1 for t, k in zip(row[1:self._cap], keep[1:self._cap])]
        for pos in range(max(content - 1, 0), self._seq):
            targets[pos] = -1
        return inputs, targets


def pack_rows(conversations, tokenizer, seq_len: int, render=None, **kw):
    """All rows of one epoch as (tokens, targets) int32 arrays of shape [rows, seq_len]."""
    rows = list(PackedRowStream(conversations, tokenizer, seq_len, render, **kw))
    tok = np.array([r[0] for r in rows], dtype=np.int32).reshape(len(rows), seq_len)
    tgt = np.array([r[1] for r in rows], dtype=np.int32).reshape(len(rows), seq_len)
    return tok, tgt
