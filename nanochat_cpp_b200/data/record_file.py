"""Reader/writer for the fixture record container.

Layout (reference `src/record_file.h`): magic[8], u32 version (=1), u32 count, then
records `{u16 name_len, name, u8 dtype, u8 rank, u64 dims[rank], payload}`; dtype codes
0 f32, 1 i32, 2 f64, 3 i64, 4 u8 (reference `tests/oracle_fixture.h:140-146`).
Magics seen: NANOORC1, NANOEVL1, NANOTOK1, NANONUM1, NCSFT001. All little-endian.
"""
from __future__ import annotations

import struct
from collections import OrderedDict
from typing import Dict, Tuple

import numpy as np

_DTYPES = {0: np.dtype("<f4"), 1: np.dtype("<i4"), 2: np.dtype("<f8"), 3: np.dtype("<i8"), 4: np.dtype("u1")}
_CODES = {v: k for k, v in _DTYPES.items()}


def read_records(path: str) -> Tuple[str, "OrderedDict[str, np.ndarray]"]:
    with open(path, "rb") as f:
        blob = f.read()
    magic = blob[:8].decode("ascii", "replace")
    version, count = struct.unpack_from("<II", blob, 8)
    if version != 1:
        raise ValueError(f"{path}: unsupported record-file version {version}")
    off = 16
    out: "OrderedDict[str, np.ndarray]" = OrderedDict()
    for _ in range(count):
        (nlen,) = struct.unpack_from("<H", blob, off)
        off += 2
        name = blob[off:off + nlen].decode("utf-8")
        off += nlen
        dtype, rank = struct.unpack_from("<BB", blob, off)
        off += 2
        dims = struct.unpack_from(f"<{rank}Q", blob, off) if rank else ()
        off += 8 * rank
        dt = _DTYPES[dtype]
        n = int(np.prod(dims)) if rank else 1
        arr = np.frombuffer(blob, dtype=dt, count=n, offset=off).reshape(dims if rank else ())
        off += n * dt.itemsize
        out[name] = arr
    return magic, out


def write_records(path: str, magic: str, records: Dict[str, np.ndarray]) -> None:
    assert len(magic) == 8
    with open(path, "wb") as f:
        f.write(magic.encode("ascii"))
        f.write(struct.pack("<II", 1, len(records)))
        for name, arr in records.items():
            arr = np.ascontiguousarray(arr)
            dt = arr.dtype.newbyteorder("<") if arr.dtype.byteorder == ">" else arr.dtype
            code = _CODES[np.dtype(dt.str.replace("=", "<").replace("|", "")) if dt.itemsize > 1 else np.dtype("u1")]
            nb = name.encode("utf-8")
            f.write(struct.pack("<H", len(nb)))
            f.write(nb)
            f.write(struct.pack("<BB", code, arr.ndim))
            for d in arr.shape:
                f.write(struct.pack("<Q", d))
            f.write(arr.astype(_DTYPES[code]).tobytes())
