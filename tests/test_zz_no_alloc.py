"""The allocation-free C entry point of paged decode attention against the tensor-level entry point.

Collected last on purpose (file name): the entry point keeps its scratch in a fixed device array of the loaded
library, so it has to give the same answer in a fresh process and after every other test has used the GPU.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_FLOATS = 2 * 1024 * 1024


def _lib():
    from nanochat_cpp_b200.ops import cuda as K
    lib = ctypes.CDLL(K._SO)      # the library the extension was imported from
    fn = lib.nc_paged_decode_attention_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int] * 7 + [ctypes.c_float, ctypes.c_int, ctypes.c_void_p,
                                                               ctypes.c_char_p, ctypes.c_int]
    lib.nc_paged_decode_attention_splits.restype = ctypes.c_int
    lib.nc_paged_decode_attention_splits.argtypes = [ctypes.c_int] * 5
    return K, lib


def _case(B, H, KV, D, max_seq, lens, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    page = 16
    pages = (max_seq + page - 1) // page
    kp = torch.randn(B * pages, page, KV, D, device="cuda", generator=g).to(torch.bfloat16)
    vp = torch.randn(B * pages, page, KV, D, device="cuda", generator=g).to(torch.bfloat16)
    table = torch.randperm(B * pages, device="cuda", generator=g).to(torch.int32).view(B, pages).contiguous()
    q = torch.randn(B, H, D, device="cuda", generator=g).to(torch.bfloat16)
    return q, kp, vp, table, torch.tensor(lens, device="cuda", dtype=torch.int32)


def _call(lib, q, kp, vp, table, lens, out, window, scale, splits=0):
    msg = ctypes.create_string_buffer(256)
    B, H, D = q.shape
    rc = lib.nc_paged_decode_attention_noalloc(
        q.data_ptr(), kp.data_ptr(), vp.data_ptr(), table.data_ptr(), lens.data_ptr(), out.data_ptr(), B, H,
        kp.shape[2], D, table.shape[1], kp.shape[1], window, scale, splits,
        torch.cuda.current_stream().cuda_stream, msg, len(msg))
    return rc, msg.value.decode()


@pytest.mark.parametrize("H,KV,D,window", [(4, 2, 128, -1), (8, 2, 64, 300)])
def test_no_alloc_entry_matches_tensor_entry_twice(H, KV, D, window):
    K, lib = _lib()
    B, max_seq = 3, 1024
    assert lib.nc_paged_decode_attention_splits(B, KV, max_seq // 16, 16, window) > 1   # the scratch is in use
    scale = D ** -0.5
    for call, lens in enumerate([[1000, 517, 33], [64, 1024, 700]]):      # two calls in a row share the scratch
        q, kp, vp, table, sl = _case(B, H, KV, D, max_seq, lens, seed=call)
        want = K.paged_decode_attention(q, kp, vp, table, sl, window, scale)
        got = torch.empty_like(q)
        rc, msg = _call(lib, q, kp, vp, table, sl, got, window, scale)
        assert rc == 0, msg
        torch.cuda.synchronize()
        assert (got.float() - want.float()).abs().max() <= 2e-2 * want.float().abs().max()
    K.check_status()


def test_no_alloc_entry_rejects_oversize_and_bad_arguments():
    K, lib = _lib()
    q, kp, vp, table, sl = _case(2, 4, 2, 128, 64, [10, 20], seed=0)
    out = torch.empty_like(q)
    # claimed sizes beyond the fixed array: refused before anything is launched
    msg = ctypes.create_string_buffer(256)
    rc = lib.nc_paged_decode_attention_noalloc(q.data_ptr(), kp.data_ptr(), vp.data_ptr(), table.data_ptr(),
                                               sl.data_ptr(), out.data_ptr(), 4096, 64, 8, 128, 4, 16, -1, 1.0, 32,
                                               None, msg, len(msg))
    assert rc == 2 and b"scratch" in msg.value
    assert 4096 * 64 * 32 * 130 > MAX_FLOATS
    rc, text = _call(lib, q, kp, vp, table, sl, out, -1, 1.0, splits=1)
    assert rc == 0, text
    rc = lib.nc_paged_decode_attention_noalloc(None, kp.data_ptr(), vp.data_ptr(), table.data_ptr(), sl.data_ptr(),
                                               out.data_ptr(), 2, 4, 2, 128, 4, 16, -1, 1.0, 0, None, msg, len(msg))
    assert rc == 1
    # a pointer that is not 16-byte aligned, a group size H / KV outside {1, 2, 4, 8}, and a key range beyond
    # 32 bits are all refused as bad arguments, before set-up and before any launch
    rc = lib.nc_paged_decode_attention_noalloc(q.data_ptr() + 2, kp.data_ptr(), vp.data_ptr(), table.data_ptr(),
                                               sl.data_ptr(), out.data_ptr(), 2, 4, 2, 128, 4, 16, -1, 1.0, 0, None,
                                               msg, len(msg))
    assert rc == 1 and b"aligned" in msg.value
    rc = lib.nc_paged_decode_attention_noalloc(q.data_ptr(), kp.data_ptr(), vp.data_ptr(), table.data_ptr(),
                                               sl.data_ptr(), out.data_ptr(), 2, 6, 2, 128, 4, 16, -1, 1.0, 0, None,
                                               msg, len(msg))
    assert rc == 1 and b"group" in msg.value
    rc = lib.nc_paged_decode_attention_noalloc(q.data_ptr(), kp.data_ptr(), vp.data_ptr(), table.data_ptr(),
                                               sl.data_ptr(), out.data_ptr(), 2, 4, 2, 128, 1 << 28, 16, -1, 1.0, 0,
                                               None, msg, len(msg))
    assert rc == 1 and b"32-bit" in msg.value
    torch.cuda.synchronize()


def test_no_alloc_entry_clamps_a_length_beyond_the_page_table():
    """`seq_lens` lives on the device, so the entry point cannot check it; the kernel clamps instead. A length
    above max_pages * page_size must give the same answer as the clamped length (and never index past the table)."""
    K, lib = _lib()
    B, H, KV, D, max_seq = 2, 4, 2, 128, 64
    q, kp, vp, table, _ = _case(B, H, KV, D, max_seq, [64, 64], seed=4)
    ok = torch.tensor([64, 40], device="cuda", dtype=torch.int32)
    over = torch.tensor([64 + 4096, 40], device="cuda", dtype=torch.int32)
    a, b = torch.empty_like(q), torch.empty_like(q)
    for lens, out in ((ok, a), (over, b)):
        rc, text = _call(lib, q, kp, vp, table, lens, out, -1, D ** -0.5)
        assert rc == 0, text
    torch.cuda.synchronize()
    assert torch.equal(a, b)
    K.check_status()
