"""Argument checks of the allocation-free decode entry point. Every refusal happens before the entry point
touches its scratch array or the CUDA runtime, so these cases need no GPU: the pointers are never dereferenced."""
import ctypes
import os

import pytest

SO = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "nanochat_cpp_b200", "_C.so")


def _fn():
    if not os.path.exists(SO):
        pytest.skip("extension not built")
    import torch  # noqa: F401  (the extension links against torch's libraries)
    lib = ctypes.CDLL(SO)
    fn = lib.nc_paged_decode_attention_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int] * 7 + [ctypes.c_float, ctypes.c_int, ctypes.c_void_p,
                                                               ctypes.c_char_p, ctypes.c_int]
    return fn


def _call(fn, ptrs, B=2, H=4, KV=2, D=128, max_pages=4, page=16, splits=0):
    msg = ctypes.create_string_buffer(256)
    rc = fn(*ptrs, B, H, KV, D, max_pages, page, -1, 1.0, splits, None, msg, len(msg))
    return rc, msg.value.decode()


def test_refusals_need_no_device():
    fn = _fn()
    good = [0x10000, 0x20000, 0x30000, 0x40000, 0x50000, 0x60000]      # q, k, v, table, lens, out (never read)
    rc, text = _call(fn, [None] + good[1:])
    assert rc == 1 and "null" in text
    for i in (0, 1, 2, 5):                                              # 16-byte alignment of q, k_pool, v_pool, out
        p = list(good)
        p[i] += 8
        rc, text = _call(fn, p)
        assert rc == 1 and "aligned" in text, (i, text)
    rc, text = _call(fn, good, H=6, KV=2)                               # group size 3
    assert rc == 1 and "group" in text
    rc, text = _call(fn, good, H=5, KV=2)                               # H not a multiple of KV
    assert rc == 1
    rc, text = _call(fn, good, D=96)
    assert rc == 1
    rc, text = _call(fn, good, max_pages=1 << 28, page=16)              # key index would overflow 32 bits
    assert rc == 1 and "32-bit" in text
    rc, text = _call(fn, good, B=4096, H=64, KV=8, splits=32)           # beyond the fixed scratch array
    assert rc == 2 and "scratch" in text
