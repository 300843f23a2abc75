"""A tiktoken encoding built from an NCTOKEN1 artefact.

The artefact stores the split pattern, the merge list (pairs of token ids, in merge order) and the special tokens;
token ids 0..255 are the bytes, merge k makes id 256 + k. tiktoken wants `mergeable_ranks`, a map from each token's
byte string to its id: built here by replaying the merges. With it `tiktoken.Encoding` produces the same ids as the
native tokenizer (checked in the tests), which gives callers tiktoken's multi-threaded batch encoder for the same
vocabulary. `TiktokenTokenizer` has the method names upstream nanochat's tokenizer interface uses
(`get_vocab_size`, `get_bos_token_id`, `encode_special`, `encode(text, prepend, append)`, `decode`).
Counterpart of the reference's python/nanochat_cpp_bridge/reference_data.py.
"""
from __future__ import annotations

import dataclasses
import struct
from pathlib import Path
from typing import Dict, List, Sequence, Tuple

from .extras import need


@dataclasses.dataclass
class Artefact:
    pattern: str
    merges: List[Tuple[int, int]]
    specials: Dict[str, int]

    @property
    def vocab_size(self) -> int:
        return max([256 + len(self.merges)] + [i + 1 for i in self.specials.values()])


def read_nctoken1(path) -> Artefact:
    data = Path(path).read_bytes()
    if data[:8] != b"NCTOKEN1":
        raise ValueError(f"{path}: not an NCTOKEN1 artefact")
    off = 8

    def u32() -> int:
        nonlocal off
        if off + 4 > len(data):
            raise ValueError(f"{path}: truncated")
        (v,) = struct.unpack_from("<I", data, off)
        off += 4
        return v

    def text() -> str:
        nonlocal off
        n = u32()
        if off + n > len(data):
            raise ValueError(f"{path}: truncated")
        s = data[off:off + n].decode("utf-8")
        off += n
        return s
    if u32() != 1:
        raise ValueError(f"{path}: unsupported version")
    pattern = text()
    merges = [(u32(), u32()) for _ in range(u32())]
    specials = {}
    for _ in range(u32()):
        name = text()
        specials[name] = u32()
    return Artefact(pattern, merges, specials)


def token_bytes(art: Artefact) -> List[bytes]:
    table = [bytes([b]) for b in range(256)]
    for a, b in art.merges:
        if a >= len(table) or b >= len(table):
            raise ValueError("merge refers to a token that does not exist yet")
        table.append(table[a] + table[b])
    return table


def mergeable_ranks(art: Artefact) -> Dict[bytes, int]:
    ranks = {}
    for i, t in enumerate(token_bytes(art)):
        if t in ranks:
            raise ValueError(f"tokens {ranks[t]} and {i} have the same bytes; tiktoken needs distinct ones")
        ranks[t] = i
    return ranks


def build_encoding(art: Artefact, name: str = "nanochat"):
    tiktoken = need("tiktoken", "building a tiktoken encoding")
    return tiktoken.Encoding(name=name, pat_str=art.pattern, mergeable_ranks=mergeable_ranks(art),
                             special_tokens=dict(art.specials))


class TiktokenTokenizer:
    def __init__(self, art: Artefact):
        self.artefact = art
        self.enc = build_encoding(art)
        self._lengths = [len(t) for t in token_bytes(art)]

    @classmethod
    def load(cls, path) -> "TiktokenTokenizer":
        return cls(read_nctoken1(path))

    def get_vocab_size(self) -> int:
        return self.artefact.vocab_size

    def get_bos_token_id(self) -> int:
        return self.artefact.specials["<|bos|>"]

    def encode_special(self, name: str) -> int:
        return self.artefact.specials[name]

    def _affix(self, v):
        return None if v is None else (v if isinstance(v, int) else self.encode_special(v))

    def encode(self, text, prepend=None, append=None, num_threads: int = 1):
        """One string -> ids; a list of strings -> a list of id lists (tiktoken's thread pool). `prepend` / `append`:
        a token id or the name of a special token."""
        pre, app = self._affix(prepend), self._affix(append)

        def wrap(ids):
            return ([pre] if pre is not None else []) + list(ids) + ([app] if app is not None else [])
        if isinstance(text, str):
            return wrap(self.enc.encode_ordinary(text))
        return [wrap(ids) for ids in self.enc.encode_ordinary_batch(list(text), num_threads=num_threads)]

    def decode(self, ids: Sequence[int]) -> str:
        return self.enc.decode(list(ids))

    def token_byte_lengths(self) -> List[int]:
        """Bytes per token id (0 for special tokens): what bits-per-byte evaluation divides by."""
        out = self._lengths + [0] * (self.get_vocab_size() - len(self._lengths))
        return out
