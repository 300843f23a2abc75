"""ctypes bindings of the native host runtime (`libnanochat_core.so`): tokenizer, BPE trainer, data loader,
checkpoint container, parquet reader, sampler. The library is built in-tree by `nanochat_cpp_b200.build`."""
from __future__ import annotations

import ctypes as C
import os
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

_HERE = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_PATH = os.path.join(_HERE, "libnanochat_core.so")
_lib = None


class Record(C.Structure):
    pass


Record._fields_ = [("name", C.c_char_p), ("dtype", C.c_int32), ("ndim", C.c_int32), ("dims", C.POINTER(C.c_int64)),
                   ("data", C.c_void_p), ("bytes", C.c_int64), ("attribute_count", C.c_int64),
                   ("attributes", C.POINTER(Record))]


class ConfigC(C.Structure):
    _fields_ = [("num_layers", C.c_int), ("num_heads", C.c_int), ("num_kv_heads", C.c_int), ("hidden_dim", C.c_int),
                ("seq_len", C.c_int), ("vocab_size", C.c_int), ("padded_vocab_size", C.c_int),
                ("rope_base", C.c_float), ("window_pattern", C.c_char_p), ("value_embedding", C.c_int)]


class MetadataC(C.Structure):
    _fields_ = [("schema", C.c_int32), ("stage", C.c_int32), ("step", C.c_int64), ("world_size", C.c_int64),
                ("precision", C.c_int32), ("config_json", C.c_char_p), ("tokenizer_id", C.c_char_p),
                ("git_revision", C.c_char_p), ("created_utc", C.c_char_p), ("notes", C.POINTER(C.c_char_p)),
                ("note_count", C.c_int32)]


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_PATH):
            from .. import build
            build.build_core()
        L = C.CDLL(_PATH)
        L.nanochat_last_error.restype = C.c_char_p
        L.nanochat_version.restype = C.c_char_p
        L.nanochat_tokenizer_load.restype = C.c_void_p
        L.nanochat_tokenizer_load.argtypes = [C.c_char_p]
        L.nanochat_tokenizer_free.argtypes = [C.c_void_p]
        L.ncb_encode_n.argtypes = [C.c_void_p, C.c_char_p, C.c_int64, C.c_int, C.c_int, C.c_void_p, C.c_int]
        L.nanochat_decode.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_char_p, C.c_int]
        L.ncb_tokenizer_vocab_size.argtypes = [C.c_void_p]
        L.ncb_tokenizer_special_id.argtypes = [C.c_void_p, C.c_char_p]
        L.ncb_tokenizer_save.argtypes = [C.c_void_p, C.c_char_p]
        L.ncb_tokenizer_train.restype = C.c_void_p
        L.ncb_tokenizer_train.argtypes = [C.c_char_p, C.c_char_p, C.c_char_p, C.c_int, C.c_int64, C.c_int64]
        L.ncb_split_pattern.argtypes = [C.c_char_p, C.c_int64, C.c_void_p, C.c_int]
        for name in ("ncb_loader_from_documents", "ncb_loader_from_text", "ncb_loader_zipf", "nanochat_loader_create"):
            getattr(L, name).restype = C.c_void_p
        L.ncb_loader_from_documents.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_size_t,
                                                C.c_int, C.c_int]
        L.ncb_loader_from_text.argtypes = [C.c_char_p, C.c_void_p, C.c_int, C.c_int, C.c_size_t, C.c_int, C.c_int]
        L.ncb_loader_zipf.argtypes = [C.c_int, C.c_int, C.c_double, C.c_uint64, C.c_int, C.c_int, C.c_size_t]
        L.nanochat_loader_create.argtypes = [C.POINTER(C.c_char_p), C.c_int, C.c_char_p, C.c_void_p, C.c_int, C.c_int,
                                             C.c_uint64, C.c_int, C.c_size_t]
        L.nanochat_loader_next.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        L.nanochat_loader_free.argtypes = [C.c_void_p]
        L.nanochat_loader_token_bytes.restype = C.POINTER(C.c_uint8)
        L.nanochat_loader_token_bytes.argtypes = [C.c_void_p, C.POINTER(C.c_int)]
        L.ncb_loader_save_cursor.argtypes = [C.c_void_p, C.c_char_p]
        L.ncb_loader_load_cursor.argtypes = [C.c_void_p, C.c_char_p]
        L.ncb_loader_epoch.restype = C.c_uint64
        L.ncb_loader_epoch.argtypes = [C.c_void_p]
        L.nanochat_checkpoint_read.argtypes = [C.c_char_p, C.POINTER(C.c_void_p), C.POINTER(C.POINTER(Record)),
                                               C.POINTER(C.c_int64), C.POINTER(C.POINTER(Record)),
                                               C.POINTER(C.c_int64)]
        L.nanochat_checkpoint_free.argtypes = [C.c_void_p]
        L.nanochat_checkpoint_metadata_read.argtypes = [C.c_char_p, C.POINTER(C.c_void_p), C.POINTER(MetadataC)]
        L.ncb_checkpoint_write_meta.argtypes = [C.c_char_p, C.POINTER(Record), C.c_int64, C.POINTER(Record), C.c_int64,
                                                C.POINTER(ConfigC), C.c_int32, C.c_int64, C.c_int64, C.c_int32,
                                                C.c_char_p, C.c_char_p]
        L.ncb_parquet_read.restype = C.c_int64
        L.ncb_parquet_read.argtypes = [C.c_char_p, C.c_char_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64,
                                       C.POINTER(C.c_int64)]
        L.ncb_sample_token.argtypes = [C.c_void_p, C.c_int, C.c_float, C.c_int, C.c_uint64, C.c_uint64, C.c_uint64]
        _lib = L
    return _lib


def last_error() -> str:
    return (lib().nanochat_last_error() or b"").decode("utf-8", "replace")


# ----------------------------------------------------------------------------------------------- tokenizer
class Tokenizer:
    """NCTOKEN1 byte-level BPE tokenizer (native)."""

    def __init__(self, handle):
        if not handle:
            raise RuntimeError(last_error() or "tokenizer handle is null")
        self._h = handle

    @classmethod
    def load(cls, path: str) -> "Tokenizer":
        return cls(lib().nanochat_tokenizer_load(path.encode()))

    @classmethod
    def train(cls, *, text: str = "", parquet: str = "", text_column: str = "text", vocab_size: int = 32768,
              doc_cap: int = 0, max_chars: int = 0) -> "Tokenizer":
        return cls(lib().ncb_tokenizer_train(text.encode() if text else None, parquet.encode() if parquet else None,
                                             text_column.encode(), vocab_size, doc_cap, max_chars))

    def save(self, path: str) -> None:
        if lib().ncb_tokenizer_save(self._h, path.encode()) != 0:
            raise RuntimeError("cannot write " + path)

    @property
    def vocab_size(self) -> int:
        return lib().ncb_tokenizer_vocab_size(self._h)

    def special_id(self, name: str) -> int:
        return lib().ncb_tokenizer_special_id(self._h, name.encode())

    @property
    def bos_id(self) -> int:
        return self.special_id("<|bos|>")

    def encode(self, text, prepend: int = -1, append: int = -1) -> List[int]:
        raw = text.encode("utf-8") if isinstance(text, str) else bytes(text)
        cap = len(raw) + 2
        buf = np.empty(cap, dtype=np.int32)
        n = lib().ncb_encode_n(self._h, raw, len(raw), prepend, append, buf.ctypes.data, cap)
        return buf[:n].tolist()

    def decode_bytes(self, ids: Sequence[int]) -> bytes:
        arr = np.asarray(list(ids), dtype=np.int32)
        cap = 16 * max(1, arr.size) + 64
        while True:
            out = C.create_string_buffer(cap)
            n = lib().nanochat_decode(self._h, arr.ctypes.data, int(arr.size), out, cap)
            if n < cap:
                return out.raw[:n]
            cap = n + 1

    def decode(self, ids: Sequence[int]) -> str:
        return self.decode_bytes(ids).decode("utf-8", "replace")

    def __del__(self):
        try:
            if self._h:
                lib().nanochat_tokenizer_free(self._h)
        except Exception:
            pass


def split_pattern(text) -> List[bytes]:
    raw = text.encode("utf-8") if isinstance(text, str) else bytes(text)
    ends = np.empty(len(raw) + 1, dtype=np.int64)
    n = lib().ncb_split_pattern(raw, len(raw), ends.ctypes.data, ends.size)
    out, a = [], 0
    for e in ends[:n]:
        out.append(raw[a:int(e)])
        a = int(e)
    return out


# ----------------------------------------------------------------------------------------------- loader
class DataLoader:
    """BOS-aligned best-fit packing loader (native, with a producer thread)."""

    def __init__(self, handle, batch: int, seq: int, keep=None):
        if not handle:
            raise RuntimeError(last_error() or "loader handle is null")
        self._h, self.batch, self.seq, self._keep = handle, batch, seq, keep

    @classmethod
    def from_documents(cls, docs: Sequence[Sequence[int]], batch: int, seq: int, buffer_docs: int = 1000,
                       rank: int = 0, world: int = 1, source_batch: int = 1) -> "DataLoader":
        flat = np.concatenate([np.asarray(d, dtype=np.int32) for d in docs]) if docs else np.zeros(0, np.int32)
        offs = np.zeros(len(docs) + 1, dtype=np.int64)
        np.cumsum([len(d) for d in docs], out=offs[1:])
        os.environ["NANOCHAT_SOURCE_BATCH"] = str(source_batch)
        try:
            h = lib().ncb_loader_from_documents(flat.ctypes.data, offs.ctypes.data, len(docs), batch, seq, buffer_docs,
                                                rank, world)
        finally:
            os.environ.pop("NANOCHAT_SOURCE_BATCH", None)
        return cls(h, batch, seq)

    @classmethod
    def from_text(cls, path: str, tokenizer: Tokenizer, batch: int, seq: int, buffer_docs: int = 1000, rank: int = 0,
                  world: int = 1) -> "DataLoader":
        return cls(lib().ncb_loader_from_text(path.encode(), tokenizer._h, batch, seq, buffer_docs, rank, world), batch,
                   seq, keep=tokenizer)

    @classmethod
    def from_parquet(cls, paths: Sequence[str], tokenizer: Tokenizer, batch: int, seq: int, text_column: str = "text",
                     buffer_docs: int = 1000, seed: int = 0, tokenizer_threads: int = 4, rank: int = 0,
                     world: int = 1) -> "DataLoader":
        """With `world > 1` document i goes to rank i % world (reference src/data.cc:823-880)."""
        if world > 1:
            bos = tokenizer.bos_id
            docs = [tokenizer.encode(t.decode("utf-8", "replace"), prepend=bos)
                    for p in paths for t in read_parquet_strings(p, text_column)]
            return cls.from_documents(docs, batch, seq, buffer_docs, rank, world)
        arr = (C.c_char_p * len(paths))(*[p.encode() for p in paths])
        return cls(lib().nanochat_loader_create(arr, len(paths), text_column.encode(), tokenizer._h, batch, seq, seed,
                                                tokenizer_threads, buffer_docs), batch, seq, keep=tokenizer)

    @classmethod
    def zipf(cls, vocab: int, batch: int, seq: int, s: float = 1.1, seed: int = 0, doc_len: int = 0) -> "DataLoader":
        return cls(lib().ncb_loader_zipf(vocab, doc_len or seq, s, seed, batch, seq, 64), batch, seq)

    def next(self) -> Tuple[np.ndarray, np.ndarray]:
        tok = np.empty((self.batch, self.seq), dtype=np.int32)
        tgt = np.empty((self.batch, self.seq), dtype=np.int32)
        lib().nanochat_loader_next(self._h, tok.ctypes.data, tgt.ctypes.data)
        return tok, tgt

    def next_into(self, tok: np.ndarray, tgt: np.ndarray) -> None:
        lib().nanochat_loader_next(self._h, tok.ctypes.data, tgt.ctypes.data)

    def save_cursor(self, path: str) -> None:
        if lib().ncb_loader_save_cursor(self._h, path.encode()) != 0:
            raise RuntimeError("cannot write " + path)

    def load_cursor(self, path: str) -> None:
        if lib().ncb_loader_load_cursor(self._h, path.encode()) != 0:
            raise RuntimeError("cannot read " + path)

    @property
    def epoch(self) -> int:
        return int(lib().ncb_loader_epoch(self._h))

    def __del__(self):
        try:
            if self._h:
                lib().nanochat_loader_free(self._h)
        except Exception:
            pass


# ----------------------------------------------------------------------------------------------- checkpoints
_NP_OF = {0: np.dtype("<f4"), 1: np.dtype("<u2"), 2: np.dtype("i1"), 4: np.dtype("u1"), 5: np.dtype("u1")}


def _records_from(ptr, count) -> "Dict[str, Tuple[int, np.ndarray, dict]]":
    out = {}
    for i in range(count):
        r = ptr[i]
        dims = [r.dims[k] for k in range(r.ndim)]
        raw = C.string_at(r.data, r.bytes) if r.bytes else b""
        arr = np.frombuffer(raw, dtype=_NP_OF[r.dtype]).reshape(dims).copy()
        attrs = {}
        for a in range(r.attribute_count):
            ar = r.attributes[a]
            adims = [ar.dims[k] for k in range(ar.ndim)]
            araw = C.string_at(ar.data, ar.bytes) if ar.bytes else b""
            attrs[ar.name.decode()] = np.frombuffer(araw, dtype=_NP_OF[ar.dtype]).reshape(adims).copy()
        out[r.name.decode()] = (int(r.dtype), arr, attrs)
    return out


def read_checkpoint(path: str):
    """Returns (records, optimizer_records, metadata dict). Record values are (dtype code, ndarray, attributes);
    bf16 payloads come back as uint16 bit patterns."""
    L = lib()
    owner = C.c_void_p()
    recs, opt = C.POINTER(Record)(), C.POINTER(Record)()
    n, m = C.c_int64(), C.c_int64()
    if L.nanochat_checkpoint_read(path.encode(), C.byref(owner), C.byref(recs), C.byref(n), C.byref(opt),
                                  C.byref(m)) != 0:
        raise RuntimeError(last_error())
    try:
        records = _records_from(recs, n.value)
        optimizer = _records_from(opt, m.value)
    finally:
        L.nanochat_checkpoint_free(owner)
    return records, optimizer, read_metadata(path)


def read_metadata(path: str) -> dict:
    import json
    L = lib()
    owner = C.c_void_p()
    meta = MetadataC()
    if L.nanochat_checkpoint_metadata_read(path.encode(), C.byref(owner), C.byref(meta)) != 0:
        raise RuntimeError(last_error())
    try:
        d = dict(schema=meta.schema, stage=meta.stage, step=meta.step, world_size=meta.world_size,
                 precision=meta.precision, config=json.loads(meta.config_json.decode()),
                 tokenizer_id=(meta.tokenizer_id or b"").decode(), git_revision=(meta.git_revision or b"").decode(),
                 created_utc=(meta.created_utc or b"").decode(),
                 notes=[meta.notes[i].decode() for i in range(meta.note_count)])
    finally:
        L.nanochat_checkpoint_free(owner)
    return d


def _make_records(items):
    keep = []
    arr = (Record * len(items))()
    for i, (name, code, data) in enumerate(items):
        data = np.ascontiguousarray(data)
        dims = (C.c_int64 * data.ndim)(*data.shape)
        nb = name.encode()
        keep += [data, dims, nb]
        arr[i].name = nb
        arr[i].dtype = code
        arr[i].ndim = data.ndim
        arr[i].dims = dims
        arr[i].data = data.ctypes.data
        arr[i].bytes = data.nbytes
        arr[i].attribute_count = 0
        arr[i].attributes = None
    return arr, keep


def write_checkpoint(path: str, records, optimizer=(), *, config: Optional[dict] = None, stage: int = 0,
                     step: int = 0, world_size: int = 1, precision: int = 0, tokenizer_id: str = "",
                     notes: str = "") -> None:
    """`records` / `optimizer`: iterables of (name, dtype code, ndarray). fp32 arrays use code 0, bf16 bit patterns
    (uint16) code 1."""
    recs, keep1 = _make_records(list(records))
    opts, keep2 = _make_records(list(optimizer))
    cfg = None
    if config is not None:
        cfg = ConfigC(config["num_layers"], config["num_heads"], config["num_kv_heads"], config["hidden_dim"],
                      config["seq_len"], config["vocab_size"], config["padded_vocab_size"],
                      float(config.get("rope_base", 100000.0)), config.get("window_pattern", "SSSL").encode(),
                      1 if config.get("value_embedding", True) else 0)
    if lib().ncb_checkpoint_write_meta(path.encode(), recs, len(recs), opts, len(opts),
                                       C.byref(cfg) if cfg is not None else None, stage, step, world_size, precision,
                                       tokenizer_id.encode(), notes.encode()) != 0:
        raise RuntimeError(last_error())


def read_parquet_strings(path: str, column: str = "text") -> List[bytes]:
    total = C.c_int64()
    n = lib().ncb_parquet_read(path.encode(), column.encode(), None, 0, None, 0, C.byref(total))
    if n < 0:
        raise RuntimeError(last_error())
    buf = np.empty(max(1, total.value), dtype=np.uint8)
    offs = np.empty(n + 1, dtype=np.int64)
    lib().ncb_parquet_read(path.encode(), column.encode(), buf.ctypes.data, buf.size, offs.ctypes.data, offs.size,
                           C.byref(total))
    raw = buf.tobytes()
    return [raw[int(offs[i]):int(offs[i + 1])] for i in range(n)]


def sample_token(logits: np.ndarray, temperature: float, top_k: int, seed: int, row: int = 0, step: int = 0) -> int:
    arr = np.ascontiguousarray(logits, dtype=np.float32)
    return lib().ncb_sample_token(arr.ctypes.data, arr.size, temperature, top_k, seed, row, step)


def fp8_encode(values, fmt: str = "e4m3") -> np.ndarray:
    """Saturating round-to-nearest-even fp8 codes (uint8) of `values`; `fmt` is "e4m3" or "e5m2"."""
    v = np.ascontiguousarray(np.asarray(values, dtype=np.float32).reshape(-1))
    out = np.empty(v.size, dtype=np.uint8)
    lib().ncb_fp8_encode(v.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p), C.c_longlong(v.size),
                         0 if fmt == "e4m3" else 1)
    return out.reshape(np.asarray(values).shape)


def fp8_decode(codes, fmt: str = "e4m3") -> np.ndarray:
    c = np.ascontiguousarray(np.asarray(codes, dtype=np.uint8).reshape(-1))
    out = np.empty(c.size, dtype=np.float32)
    lib().ncb_fp8_decode(c.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p), C.c_longlong(c.size),
                         0 if fmt == "e4m3" else 1)
    return out.reshape(np.asarray(codes).shape)
