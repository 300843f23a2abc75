"""Synthetic token streams for benchmarks: Zipf(s) over the vocabulary with a BOS every `seq` tokens."""
from __future__ import annotations

import numpy as np
import torch


def zipf_tokens(n_rows: int, seq: int, vocab: int, seed: int = 0, s: float = 1.1, bos_id: int = 0) -> torch.Tensor:
    """[n_rows, seq + 1] int32 rows on the CPU (pinned when CUDA is available): column 0 is BOS, the rest is
    Zipf(s)-distributed over [1, vocab). Inputs are row[:-1], targets row[1:]."""
    rng = np.random.default_rng(seed)
    ranks = np.arange(1, vocab, dtype=np.float64)
    p = ranks ** (-s)
    cdf = np.cumsum(p / p.sum())
    u = rng.random((n_rows, seq + 1))
    ids = (np.searchsorted(cdf, u) + 1).astype(np.int32)
    ids = np.minimum(ids, vocab - 1)
    ids[:, 0] = bos_id
    t = torch.from_numpy(ids)
    if torch.cuda.is_available():
        t = t.pin_memory()
    return t
