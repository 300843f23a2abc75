"""Model hyper-parameters and their derived dimensions.

Behavioural parity with the reference `include/nanochat/config.h:13-107`:
same defaults (12 layers / 6 heads / hidden 768 / seq 2048 / vocab 32768 /
rope base 1e5 / window pattern "SSSL" / value embeddings on), same derived
quantities (`head_dim`, `kv_dim`, `mlp_dim = 4*hidden`, alternating value
embeddings with the last layer always carrying one, short window = a quarter
of the context rounded up to a 128-token tile, last layer always full
context) and the same validation rules.

One addition: `short_window_override` lets a benchmark configuration state a
short window explicitly (the reference derives it from `seq_len` only).
"""
from __future__ import annotations

import dataclasses
import math
from dataclasses import dataclass

RMS_EPS = 1.1920929e-07  # reference src/ops.h:28 (float epsilon)
LOGIT_SOFTCAP = 15.0  # reference src/ops.h:29
QK_SCALE = 1.2  # reference src/ops.h:30
VE_GATE_CHANNELS = 12  # reference src/ops.h:31
SMEAR_CHANNELS = 24  # reference src/ops.h:32


@dataclass
class Config:
    num_layers: int = 12
    num_heads: int = 6
    num_kv_heads: int = 6
    hidden_dim: int = 768
    seq_len: int = 2048
    vocab_size: int = 32768
    padded_vocab_size: int = 32768
    rope_base: float = 100000.0
    window_pattern: str = "SSSL"
    value_embedding: bool = True
    short_window_override: int = 0  # 0 = derive from seq_len

    # ---- derived -----------------------------------------------------
    @property
    def head_dim(self) -> int:
        return self.hidden_dim // self.num_heads

    @property
    def query_dim(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_kv_heads * self.head_dim

    @property
    def mlp_dim(self) -> int:
        return 4 * self.hidden_dim

    @property
    def backout_layer(self) -> int:
        # reference src/model.cc:207
        return self.num_layers // 2

    def has_value_embedding(self, layer: int) -> bool:
        if not self.value_embedding:
            return False
        return layer % 2 == (self.num_layers - 1) % 2

    @property
    def short_window(self) -> int:
        if self.short_window_override > 0:
            return self.short_window_override
        return ((self.seq_len // 4 + 127) // 128) * 128

    def window_left(self, layer: int) -> int:
        """Left extent of the window of `layer`; -1 means full context."""
        if layer >= self.num_layers - 1:
            return -1
        if not self.window_pattern:
            return -1
        kind = self.window_pattern[layer % len(self.window_pattern)]
        return self.short_window if kind == "S" else -1

    def effective_window(self, layer: int, tokens: int) -> int:
        left = self.window_left(layer)
        return tokens if left < 0 else min(left, tokens)

    def validate(self) -> None:
        c = self
        if min(c.num_layers, c.num_heads, c.num_kv_heads, c.hidden_dim, c.seq_len,
               c.vocab_size, c.padded_vocab_size) <= 0:
            raise ValueError("model dimensions and vocabulary sizes must be positive")
        if c.hidden_dim < SMEAR_CHANNELS:
            raise ValueError("hidden_dim must be at least 24 for the smear and value gates")
        if c.hidden_dim % c.num_heads != 0:
            raise ValueError("hidden_dim must be divisible by num_heads")
        if c.num_heads % c.num_kv_heads != 0:
            raise ValueError("num_heads must be divisible by num_kv_heads")
        if c.head_dim % 2 != 0:
            raise ValueError("head_dim must be even for rotary embeddings")
        if c.padded_vocab_size < c.vocab_size:
            raise ValueError("padded_vocab_size must be >= vocab_size")
        if not (c.rope_base > 0.0) or not math.isfinite(c.rope_base):
            raise ValueError("rope_base must be finite and positive")
        for kind in c.window_pattern:
            if kind not in "SL":
                raise ValueError("window_pattern can contain only 'S' and 'L'")

    def replace(self, **kw) -> "Config":
        return dataclasses.replace(self, **kw)

    def to_dict(self) -> dict:
        return dataclasses.asdict(self)

    @classmethod
    def from_depth(cls, depth: int, *, seq_len: int = 2048, vocab_size: int = 32768,
                   head_dim: int = 128, **kw) -> "Config":
        """`depth -> hidden = depth*64` rounded up to a multiple of `head_dim`,
        vocab padded to 64 (reference python/nanochat_cpp/api.py `Config`)."""
        hidden = ((depth * 64 + head_dim - 1) // head_dim) * head_dim
        heads = hidden // head_dim
        padded = ((vocab_size + 63) // 64) * 64
        return cls(num_layers=depth, num_heads=heads, num_kv_heads=kw.pop("num_kv_heads", heads),
                   hidden_dim=hidden, seq_len=seq_len, vocab_size=vocab_size,
                   padded_vocab_size=padded, **kw)


def preset(name: str) -> Config:
    """Named configurations used by the benchmarks and tests."""
    if name == "tiny":  # CPU reference config: 4 layers, hidden 256, 4 heads of 64
        return Config(num_layers=4, num_heads=4, num_kv_heads=4, hidden_dim=256, seq_len=256,
                      vocab_size=4096, padded_vocab_size=4096, rope_base=10000.0)
    if name == "d12":
        return Config(num_layers=12, num_heads=6, num_kv_heads=6, hidden_dim=768, seq_len=2048,
                      vocab_size=32768, padded_vocab_size=32768, short_window_override=1024)
    if name == "d20":
        return Config(num_layers=20, num_heads=10, num_kv_heads=10, hidden_dim=1280, seq_len=2048,
                      vocab_size=65536, padded_vocab_size=65536, short_window_override=1024)
    if name == "d20-h100":  # shape of the reference's published 1xH100 run
        return Config(num_layers=20, num_heads=10, num_kv_heads=5, hidden_dim=1280, seq_len=1024,
                      vocab_size=32768, padded_vocab_size=32768, window_pattern="SSL")
    if name == "d26":
        return Config(num_layers=26, num_heads=13, num_kv_heads=13, hidden_dim=1664, seq_len=2048,
                      vocab_size=65536, padded_vocab_size=65536, short_window_override=1024)
    raise KeyError(f"unknown preset {name!r}")
