"""The CUDA-core kernels of csrc/cuda, compiled by the host compiler (csrc/emu/cuda_emu.h: every CUDA thread a fiber,
shuffles and barriers as rendezvous) and run here, on a machine without a GPU, against the PyTorch definitions of the
same operators. What is executed is the kernels' own source: index arithmetic, vector tails, masks, reductions."""
import ctypes
import os

import numpy as np
import pytest
import torch

import nanochat_cpp_b200
from nanochat_cpp_b200.ops import ref

LIB = os.path.join(os.path.dirname(nanochat_cpp_b200.__file__), "libnc_emu.so")
pytestmark = pytest.mark.skipif(not os.path.exists(LIB), reason="host build of the kernels not present")


SCHEDULES = {"ascending": 0, "descending": 1, "shuffled": 2}


@pytest.fixture(scope="module", params=list(SCHEDULES))
def E(request):
    """Every test of this file runs under three fiber schedules (threads of a block resumed in ascending, descending
    and per-pass shuffled order). The kernels have to give the expected result under each: an ordering between
    threads that no barrier, shuffle or atomic enforces shows up as a failure of one of the three."""
    lib = ctypes.CDLL(LIB)
    lib.nc_emu_set_schedule(SCHEDULES[request.param], ctypes.c_ulonglong(20240229))
    return lib


def P(t):
    return ctypes.c_void_p(t.data_ptr())


def bf(*shape, scale=1.0, gen=None):
    return (torch.randn(*shape, generator=gen) * scale).to(torch.bfloat16).contiguous()


def close(got, want, rtol=2.0 ** -7, atol=2.0 ** -8):
    got, want = got.float(), want.float()
    err = (got - want).abs()
    bound = atol * want.abs().mean().clamp_min(1e-6) + rtol * want.abs()
    assert (err <= bound).all(), float((err - bound).max())


@pytest.mark.parametrize("rows,dim", [(19, 256), (8, 1280), (5, 40), (33, 100)])
def test_rmsnorm_forward_and_backward(E, rows, dim):
    g = torch.Generator().manual_seed(rows + dim)
    x, dy, res = bf(rows, dim, gen=g), bf(rows, dim, gen=g), bf(rows, dim, gen=g)
    y = torch.empty_like(x)
    rstd = torch.empty(rows)
    E.nc_emu_rmsnorm(0, P(x), None, None, None, None, P(y), P(rstd), rows, dim, ctypes.c_float(1e-6))
    yr, rr = ref.rmsnorm_fwd(x, 1e-6)
    close(y, yr)
    assert torch.allclose(rstd, rr, rtol=1e-5)
    dx = torch.empty_like(x)
    E.nc_emu_rmsnorm_bwd(P(x), P(dy), P(rstd), P(res), P(dx), rows, dim)
    close(dx, ref.rmsnorm_bwd(x, dy, rr, res))


@pytest.mark.parametrize("rows,dim,extra_cols,accumulate", [(19, 256, 12, 1), (8, 1280, 0, 0), (40, 64, 12, 0)])
def test_fused_norm_blend_backward(E, rows, dim, extra_cols, accumulate):
    g = torch.Generator().manual_seed(7)
    x, x0, dh, res = (bf(rows, dim, gen=g) for _ in range(4))
    lam_r, lam_0 = torch.tensor([0.9]), torch.tensor([0.2])
    xr = (lam_r * x.float() + lam_0 * x0.float()).to(torch.bfloat16)
    _, rstd = ref.rmsnorm_fwd(xr, 1e-6)
    extra = torch.randn(rows, extra_cols, generator=g) if extra_cols else None
    base = bf(rows, dim, gen=g) if accumulate else None
    gsc = torch.tensor([0.25, -0.5])
    want_g = gsc.clone()
    want_dx, want_dx0 = ref.norm_blend_bwd(xr, dh, rstd, res, x, x0, lam_r[0], lam_0[0], want_g[0:1], want_g[1:2],
                                           dx0_acc=base.clone() if accumulate else None, extra=extra)
    dx = torch.empty_like(x)
    dx0 = base.clone() if accumulate else torch.empty_like(x)
    E.nc_emu_norm_blend_bwd(P(xr), P(dh), P(rstd), P(res), P(extra) if extra is not None else None, extra_cols, P(x),
                            P(x0), P(lam_r), P(lam_0), P(dx), P(dx0), accumulate, P(gsc[0:1]), P(gsc[1:2]), rows, dim)
    close(dx, want_dx)
    close(dx0, want_dx0, atol=2.0 ** -7)
    assert torch.allclose(gsc, want_g, rtol=1e-3, atol=1e-2)


@pytest.mark.parametrize("heads,D", [(3, 64), (2, 128)])
def test_qk_preparation(E, heads, D):
    g = torch.Generator().manual_seed(D)
    B_, T = 2, 9
    x = bf(B_, T, heads, D, gen=g)
    cos, sin = ref.build_rope(T, D, 10000.0, "cpu")
    out = torch.empty_like(x)
    E.nc_emu_qk_prep_fwd(P(x), ctypes.c_longlong(heads * D), P(out), ctypes.c_longlong(heads * D), P(cos.contiguous()),
                         P(sin.contiguous()), None, B_ * T, T, heads, D, ctypes.c_float(1e-6), ctypes.c_float(1.2))
    want, _ = ref.qk_prep_fwd(x, x, cos, sin, 1e-6, 1.2)
    close(out, want)


def test_embedding_kernels_check_their_indices(E):
    g = torch.Generator().manual_seed(1)
    table = bf(50, 64, gen=g)
    ids = torch.tensor([3, 50, 7, -1, 49, 3], dtype=torch.int32)
    out = torch.full((6, 64), 7.0, dtype=torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32)
    E.nc_emu_embedding_fwd(P(ids), P(table), P(out), 6, 64, 50, P(status))
    assert torch.equal(out[[0, 2, 4, 5]], table[[3, 7, 49, 3]]) and not out[[1, 3]].any()
    assert int(status) == 7                                  # an id outside the table was skipped and reported
    dout = bf(6, 64, gen=g)
    want = torch.zeros(50, 64)
    for r, i in enumerate(ids.tolist()):
        if 0 <= i < 50:
            want[i] += dout[r].float()
    for sorted_order in (False, True):
        dt = torch.zeros(50, 64)
        status.zero_()
        if sorted_order:
            s, perm = torch.sort(ids, stable=True)
            s32, perm32 = s.int().contiguous(), perm.int().contiguous()      # named: they must outlive the call
            E.nc_emu_embedding_bwd_sorted(P(s32), P(perm32), P(dout), ctypes.c_longlong(64), P(dt), 6, 64, 50,
                                          P(status))
        else:
            E.nc_emu_embedding_bwd(P(ids), P(dout), ctypes.c_longlong(64), P(dt), 6, 64, 50, P(status))
        assert torch.allclose(dt, want, atol=1e-6) and int(status) == 7


def test_softcap_cross_entropy(E):
    g = torch.Generator().manual_seed(2)
    rows, vocab, padded = 7, 250, 256
    logits = bf(rows, padded, scale=4.0, gen=g)
    targets = torch.randint(0, vocab, (rows,), generator=g).int()
    targets[2] = -1
    targets[5] = vocab + 3                                   # outside the vocabulary: ignored, reported
    work = logits.clone()
    losses = torch.empty(rows)
    scale = torch.tensor([0.5])
    status = torch.zeros(1, dtype=torch.int32)
    E.nc_emu_classifier(P(work), ctypes.c_longlong(padded), P(targets), P(losses), None, P(scale), rows, vocab, padded,
                        ctypes.c_float(15.0), -1, 1, P(status))
    ok = torch.tensor([t not in (2, 5) for t in range(rows)])
    safe_t = torch.where(ok, targets, torch.zeros_like(targets))
    want_l, want_d = ref.classifier_fwd_bwd(logits[ok].clone(), safe_t[ok], vocab, dlogit_scale=0.5)
    assert torch.allclose(losses[ok], want_l.float(), rtol=2e-3, atol=2e-3)
    assert not losses[~ok].any() and not work[~ok].any()
    close(work[ok][:, :vocab], want_d[:, :vocab], rtol=2.0 ** -6, atol=2.0 ** -5)
    assert not work[:, vocab:].any()
    assert int(status) == 7


@pytest.mark.parametrize("n", [4096 + 3, 17])
def test_adamw_kernel(E, n):
    g = torch.Generator().manual_seed(n)
    master, grad = torch.randn(n, generator=g), torch.randn(n, generator=g)
    m, v = torch.rand(n, generator=g) * 0.1, torch.rand(n, generator=g) * 0.01
    rm, rmm, rv = master.clone(), m.clone(), v.clone()
    value = torch.zeros(n, dtype=torch.bfloat16)
    scale = torch.tensor([0.5])
    kw = dict(lr=0.01, beta1=0.8, beta2=0.95, eps=1e-10, weight_decay=0.01, step=3)
    f = ctypes.c_float
    E.nc_emu_adamw(P(master), P(value), P(grad), P(m), P(v), ctypes.c_longlong(n), f(kw["lr"]), f(kw["beta1"]),
                   f(kw["beta2"]), f(kw["eps"]), f(kw["weight_decay"]), kw["step"], P(scale), 3)
    ref.adamw_update(rm, None, grad, rmm, rv, grad_scale=0.5, **kw)
    assert torch.allclose(master, rm, rtol=1e-5, atol=1e-6) and torch.allclose(m, rmm, rtol=1e-6)
    assert torch.allclose(v, rv, rtol=1e-6) and torch.equal(value, master.to(torch.bfloat16))


@pytest.mark.parametrize("B,H,KV,D,window,splits", [(3, 4, 2, 64, -1, 1), (2, 4, 1, 128, 20, 3), (2, 2, 2, 128, -1, 2)])
def test_paged_decode_attention(E, B, H, KV, D, window, splits):
    """Split-KV single-query attention over 16-token pages with a shuffled page table, GQA and a left window."""
    g = torch.Generator().manual_seed(B * 100 + D + splits)
    page, max_pages = 16, 6
    pages = B * max_pages
    k_pool, v_pool = bf(pages, page, KV, D, gen=g), bf(pages, page, KV, D, gen=g)
    table = torch.randperm(pages, generator=g).int().view(B, max_pages).contiguous()
    lens = torch.tensor([37, 90, 5][:B], dtype=torch.int32)
    q = bf(B, H, D, gen=g)
    out = torch.zeros(B, H, D, dtype=torch.bfloat16)
    part_acc = torch.zeros(B, H, splits, D)
    part_ml = torch.zeros(B, H, splits, 2)
    scale = 1.0 / D ** 0.5
    rc = E.nc_emu_paged_decode(P(q), P(k_pool), P(v_pool), P(table), max_pages, P(lens), B, H, KV, D, page, window,
                               ctypes.c_float(scale), splits, P(part_acc), P(part_ml), P(out))
    assert rc == 0
    want = ref.paged_decode_attention(q, k_pool, v_pool, table, lens, window, scale)
    close(out, want, rtol=2.0 ** -6, atol=2.0 ** -6)


def test_kv_append_and_argmax(E):
    g = torch.Generator().manual_seed(4)
    pages, page, KV, D = 4, 16, 2, 64
    k_pool, v_pool = torch.zeros(pages, page, KV, D, dtype=torch.bfloat16), torch.zeros(pages, page, KV, D,
                                                                                        dtype=torch.bfloat16)
    table = torch.tensor([[0, 9], [2, 3]], dtype=torch.int32)
    positions = torch.tensor([[3, 20], [40, 17]], dtype=torch.int32)
    k_new, v_new = bf(2, 2, KV, D, gen=g), bf(2, 2, KV, D, gen=g)
    status = torch.zeros(1, dtype=torch.int32)
    E.nc_emu_kv_append(P(k_pool), P(v_pool), P(table), 2, P(positions), P(k_new), ctypes.c_longlong(KV * D), P(v_new),
                       ctypes.c_longlong(KV * D), 2, 2, page, KV * D, pages, P(status))
    want = torch.zeros_like(k_pool)
    want[0, 3], want[3, 1] = k_new[0, 0], k_new[1, 1]
    assert torch.equal(k_pool, want) and int(status) == 7
    logits = bf(5, 300, gen=g)
    logits[1, 250] = 50.0                                     # beyond the vocabulary: must not win
    logits[2, 7] = logits[2, 100] = 40.0                      # a tie: the lowest index
    out = torch.zeros(5, dtype=torch.int64)
    E.nc_emu_argmax_rows(P(logits), ctypes.c_longlong(300), P(out), 5, 250)
    assert torch.equal(out, logits[:, :250].float().argmax(dim=-1)) and int(out[2]) == 7


def _ptrs(tensors):
    arr = (ctypes.c_longlong * len(tensors))(*[t.data_ptr() for t in tensors])
    return arr


def test_bf16_push_reduce_scatter_across_four_emulated_ranks(E):
    """The transport's reduce-scatter on the CPU: every "rank" pushes what the others own (bf16, scaled) into their
    receive slots and publishes its flag; every owner then reduces in fixed rank order in fp32. Odd run lengths
    exercise the partial-vector tails, NaN-filled receive buffers show an element nobody pushed."""
    world, n, scale = 4, 1 << 14, 0.5
    g = torch.Generator().manual_seed(12)
    grads = [torch.randn(n, generator=g) for _ in range(world)]
    orig = [t.clone() for t in grads]
    runs = {r: [(r * 2048, 2048 - 3 * r), (10000 + r * 40, 37)] for r in range(world)}
    placed, cap = {}, 0
    for r in range(world):
        pos, rows = 0, []
        for off, cnt in runs[r]:
            rows.append((off, cnt, pos))
            pos += (cnt + 7) // 8 * 8
        placed[r], cap = rows, max(cap, pos)
    recv = [torch.full((world * cap,), float("nan"), dtype=torch.bfloat16) for _ in range(world)]
    flags = [torch.zeros(2 * world, dtype=torch.int32) for _ in range(world)]
    for src in range(world):
        rows, first = [], 0
        for owner in range(world):
            if owner == src:
                continue
            for off, cnt, pos in placed[owner]:
                rows.append([first, off, pos, owner, cnt])
                first += (cnt + 7) // 8
        segs = torch.tensor(rows, dtype=torch.int64)
        E.nc_emu_grad_push(P(grads[src]), _ptrs(recv), world, ctypes.c_longlong(cap), src, P(segs), len(rows),
                           ctypes.c_longlong(first), ctypes.c_float(scale), 3)
        E.nc_emu_comm_signal(_ptrs(flags), world, src, 1, 3)
    status = torch.zeros(1, dtype=torch.int32)
    for owner in range(world):
        assert flags[owner][world:2 * world].tolist() == [3] * world      # every rank's flag arrived at this owner
        rows, first = [], 0
        for off, cnt, pos in placed[owner]:
            rows.append([first, off, pos, cnt])
            first += (cnt + 7) // 8
        segs = torch.tensor(rows, dtype=torch.int64)
        acc = torch.zeros(1, dtype=torch.float64)
        E.nc_emu_grad_reduce_local(P(grads[owner]), P(recv[owner]), ctypes.c_longlong(cap), world, owner, P(segs),
                                   len(rows), ctypes.c_longlong(first), ctypes.c_float(scale), P(flags[owner]), 1, 3,
                                   P(acc), P(status), 2)
        ss = 0.0
        for off, cnt, _ in placed[owner]:
            want = torch.zeros(cnt)
            for r in range(world):
                part = orig[r][off:off + cnt] * scale
                want += part if r == owner else part.to(torch.bfloat16).float()
            assert torch.allclose(grads[owner][off:off + cnt], want, rtol=2e-6, atol=1e-7), (owner, off)
            ss += float(want.double().square().sum())
        assert abs(float(acc) - ss) <= 1e-6 * ss
        mask = torch.ones(n, dtype=torch.bool)
        for off, cnt, _ in placed[owner]:
            mask[off:off + cnt] = False
        assert torch.equal(grads[owner][mask], orig[owner][mask])           # nothing outside the owned runs moved
    assert int(status) == 0


def test_a_wait_for_a_flag_nobody_sets_gives_up_with_a_status(E):
    flags = torch.zeros(8, dtype=torch.int32)
    flags[4:8] = torch.tensor([2, 2, 1, 2])                    # rank 2 is one step behind in slot 1
    status = torch.zeros(1, dtype=torch.int32)
    E.nc_emu_comm_wait(P(flags), 4, 1, 2, P(status), ctypes.c_ulonglong(20_000_000))     # 20 ms
    assert int(status) == 5
    status.zero_()
    flags[6] = 2
    E.nc_emu_comm_wait(P(flags), 4, 1, 2, P(status), ctypes.c_ulonglong(20_000_000))
    assert int(status) == 0


def test_adamw_update_pushed_into_every_rank(E):
    world, n, off = 3, 2048 + 5, 64
    g = torch.Generator().manual_seed(9)
    values = [torch.zeros(4096, dtype=torch.bfloat16) for _ in range(world)]
    master, grad = torch.randn(n, generator=g), torch.randn(n, generator=g)
    m, v = torch.zeros(n), torch.zeros(n)
    rm, rmm, rv = master.clone(), m.clone(), v.clone()
    scale = torch.tensor([0.5])
    kw = dict(lr=0.01, beta1=0.8, beta2=0.95, eps=1e-10, weight_decay=0.01, step=3)
    f = ctypes.c_float
    E.nc_emu_adamw_push(P(master), _ptrs(values), world, ctypes.c_longlong(off), P(grad), P(m), P(v), ctypes.c_longlong(n),
                        f(kw["lr"]), f(kw["beta1"]), f(kw["beta2"]), f(kw["eps"]), f(kw["weight_decay"]), kw["step"],
                        P(scale), 2)
    ref.adamw_update(rm, None, grad, rmm, rv, grad_scale=0.5, **kw)
    assert torch.allclose(master, rm, rtol=1e-5, atol=1e-6)
    for val in values:
        assert torch.equal(val[off:off + n], master.to(torch.bfloat16))
        assert not val[:off].any() and not val[off + n:].any()


@pytest.mark.parametrize("world", [8, 3])
def test_whole_model_reduce_scatter_plan_on_emulated_ranks(E, world):
    """The transport's plan for a real parameter list (ownership of Muon matrices and AdamW slices, buckets per layer,
    receive layout) driven through the kernels for every rank and every bucket: each owner ends up with the scaled
    sum of all ranks' gradients on exactly the elements it owns, in every bucket, at eight ranks as at three."""
    import types
    from nanochat_cpp_b200.config import Config
    from nanochat_cpp_b200.models.params import param_specs
    from nanochat_cpp_b200.parallel import dp
    from nanochat_cpp_b200.parallel.fused import plan_reduce_scatter, push_rows
    cfg = Config(num_layers=3, num_heads=2, num_kv_heads=1, hidden_dim=128, seq_len=64, vocab_size=200,
                 padded_vocab_size=256, window_pattern="SL")
    specs = param_specs(cfg)
    owners = dp.assign_owners(types.SimpleNamespace(specs=specs, cfg=cfg), world)
    L = cfg.num_layers
    placed, cap = plan_reduce_scatter(specs, owners, world, L)
    total = max(s.offset + s.count for s in specs)
    g = torch.Generator().manual_seed(world)
    grads = [torch.randn(total, generator=g) for _ in range(world)]
    orig = torch.stack(grads)
    scale = 1.0 / world
    recv = [torch.full((world * max(cap, 8),), float("nan"), dtype=torch.bfloat16) for _ in range(world)]
    flags = [torch.zeros((L + 4) * world, dtype=torch.int32) for _ in range(world)]
    status = torch.zeros(1, dtype=torch.int32)
    for b in range(L + 2):
        for src in range(world):
            rows, first = push_rows(placed, src, world, b)          # the table the transport itself builds
            assert len(rows) <= 128
            if len(rows) > 1 and world > 2:                           # rotated: the first destination follows the sender
                assert rows[0][3] == next(r for r in ((src + k) % world for k in range(1, world)) if placed[r][b])
            if rows:
                segs = torch.tensor(rows, dtype=torch.int64)
                E.nc_emu_grad_push(P(grads[src]), _ptrs(recv), world, ctypes.c_longlong(cap), src, P(segs), len(rows),
                                   ctypes.c_longlong(first), ctypes.c_float(scale), 2)
            E.nc_emu_comm_signal(_ptrs(flags), world, src, b, 1)
        for owner in range(world):
            rows, first = [], 0
            for off, cnt, pos in placed[owner][b]:
                rows.append([first, off, pos, cnt])
                first += (cnt + 7) // 8
            if not rows:
                continue
            segs = torch.tensor(rows, dtype=torch.int64)
            acc = torch.zeros(1, dtype=torch.float64)
            E.nc_emu_grad_reduce_local(P(grads[owner]), P(recv[owner]), ctypes.c_longlong(cap), world, owner, P(segs),
                                       len(rows), ctypes.c_longlong(first), ctypes.c_float(scale), P(flags[owner]), b, 1,
                                       P(acc), P(status), 2)
    assert int(status) == 0
    covered = torch.zeros(total, dtype=torch.int32)
    for owner in range(world):
        for b in range(L + 2):
            for off, cnt, _ in placed[owner][b]:
                covered[off:off + cnt] += 1
                want = orig[owner, off:off + cnt] * scale
                for r in range(world):
                    if r != owner:
                        want = want + (orig[r, off:off + cnt] * scale).to(torch.bfloat16).float()
                # fixed rank order in the kernel; the sum here adds the owner's term first: equal to fp32 rounding
                assert torch.allclose(grads[owner][off:off + cnt], want, rtol=1e-5, atol=1e-6), (owner, b, off)
    live = torch.zeros(total, dtype=torch.bool)
    for s in specs:
        live[s.offset:s.offset + s.count] = True
    assert torch.equal(covered[live], torch.ones_like(covered[live]))      # every parameter has exactly one owner


def test_value_gate_forward_with_gathered_rows_and_backward(E):
    g = torch.Generator().manual_seed(21)
    M, C, KV, D, vocab = 11, 128, 2, 64, 30
    h = bf(M, C, gen=g)
    table = bf(vocab, KV * D, gen=g)
    gw = bf(KV, 12, scale=0.3, gen=g)
    ids = torch.randint(0, vocab, (M,), generator=g).int()
    ids[4] = vocab + 2                                         # outside the table: that row keeps its value
    v0 = bf(M, KV * D, gen=g)
    v = v0.clone()
    gate = torch.zeros(M, KV, dtype=torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32)
    E.nc_emu_value_gate_fwd(P(h), ctypes.c_longlong(C), P(table), P(gw), P(v), ctypes.c_longlong(KV * D), P(gate), M, KV, D,
                            P(ids), vocab, P(status))
    ok = torch.ones(M, dtype=torch.bool)
    ok[4] = False
    ve = table[ids.long().clamp_max(vocab - 1)]
    want_v, want_gate = ref.value_gate_fwd(h, ve, gw, v0, D)
    close(v[ok], want_v[ok])
    close(gate[ok], want_gate[ok])
    assert torch.equal(v[4], v0[4]) and int(status) == 7
    # backward on the rows' own value embeddings
    dv = bf(M, KV * D, gen=g)
    dve = torch.zeros(M, KV * D, dtype=torch.bfloat16)
    dh12 = torch.zeros(M, 12)
    dgw = torch.zeros(KV, 12)
    E.nc_emu_value_gate_bwd(P(h), ctypes.c_longlong(C), P(ve.contiguous()), P(gw), P(want_gate.contiguous()), P(dv),
                            ctypes.c_longlong(KV * D), P(dve), P(dh12), P(dgw), M, KV, D)
    r_dve, r_dh12, r_dgw = ref.value_gate_bwd(h, ve, gw, want_gate, dv, D)
    close(dve, r_dve)
    assert torch.allclose(dh12, r_dh12, rtol=2e-2, atol=2e-2) and torch.allclose(dgw, r_dgw, rtol=2e-2, atol=5e-2)


def test_smear_forward_and_qk_preparation_backward(E):
    g = torch.Generator().manual_seed(31)
    B_, T, C = 2, 7, 64
    emb = bf(B_ * T, C, gen=g)
    gw = bf(24, scale=0.3, gen=g)
    lam = torch.tensor([0.4])
    x0 = torch.zeros_like(emb)
    sig = torch.zeros(B_ * T)
    E.nc_emu_smear_fwd(P(emb), P(gw), P(lam), None, P(x0), P(sig), B_ * T, T, C)
    want_x0, want_sig = ref.smear_fwd(emb, gw, lam[0], T)
    close(x0, want_x0)
    assert torch.allclose(sig, want_sig.reshape(-1), rtol=1e-4, atol=1e-5)
    heads, D = 3, 64
    pre, grad = bf(B_, T, heads, D, gen=g), bf(B_, T, heads, D, gen=g)
    cos, sin = ref.build_rope(T, D, 10000.0, "cpu")
    out = torch.zeros_like(pre)
    E.nc_emu_qk_prep_bwd(P(pre), ctypes.c_longlong(heads * D), P(grad), ctypes.c_longlong(heads * D), P(out),
                         ctypes.c_longlong(heads * D), P(cos.contiguous()), P(sin.contiguous()), B_ * T, T, heads, D,
                         ctypes.c_float(1e-6), ctypes.c_float(1.2))
    want, _ = ref.qk_prep_bwd(pre, pre, grad, grad, cos, sin, 1e-6, 1.2)
    close(out, want, rtol=2.0 ** -6, atol=2.0 ** -6)


@pytest.mark.parametrize("stage", [0, 1, 2])
@pytest.mark.parametrize("vocab,padded", [(4096, 4096), (8200, 8256)])
def test_softcap_cross_entropy_vector_kernel(E, stage, vocab, padded):
    """The kernel of the training step (512 threads per row, 16-byte accesses, fixed-cap maximum), with the row
    re-read from memory, with the row parked in shared memory, and with exp(z - cap) cached in place (2)."""
    g = torch.Generator().manual_seed(vocab + stage)
    rows = 5
    logits = bf(rows, padded, scale=6.0, gen=g)
    targets = torch.randint(0, vocab, (rows,), generator=g, dtype=torch.int32)
    targets[1] = -1                       # ignored
    targets[3] = vocab + 3                # out of range: treated as ignored, reported
    scale, rs = torch.tensor([0.37]), torch.rand(rows, generator=g)
    ok = torch.tensor([True, False, True, False, True])
    safe = torch.where(ok, targets, torch.full_like(targets, -1))
    want_l, want_d = ref.classifier_fwd_bwd(logits.clone(), safe, vocab, dlogit_scale=scale[0], row_scale=rs)
    work, losses, status = logits.clone(), torch.full((rows,), 9.0), torch.zeros(1, dtype=torch.int32)
    E.nc_emu_classifier_smem(stage, P(work), ctypes.c_longlong(padded), P(targets), P(losses), P(rs), P(scale), rows,
                             vocab, padded, ctypes.c_float(15.0), -1, 1, P(status))
    assert int(status) == 7
    assert torch.allclose(losses, want_l.float(), rtol=2e-3, atol=1e-4)
    assert float(work[~ok].abs().max()) == 0.0 and float(work[:, vocab:].abs().sum()) == 0.0
    err = (work.float() - want_d.float()).abs()
    assert float(err.max()) <= 2e-2 * float(want_d.float().abs().max())
    # loss only: the logits stay as they were
    work2, losses2 = logits.clone(), torch.zeros(rows)
    E.nc_emu_classifier_smem(stage, P(work2), ctypes.c_longlong(padded), P(targets), P(losses2), None, P(scale), rows,
                             vocab, padded, ctypes.c_float(15.0), -1, 0, P(status))
    assert torch.equal(work2, logits) and torch.allclose(losses2, losses)


def test_smear_backward_and_column_add(E):
    g = torch.Generator().manual_seed(21)
    B, T, dim = 2, 9, 64
    tokens = B * T
    emb, dx0, gw = bf(tokens, dim, gen=g), bf(tokens, dim, gen=g), bf(24, scale=0.3, gen=g)
    lam = torch.tensor([0.4])
    x0 = torch.empty_like(emb)
    sig = torch.empty(tokens)
    E.nc_emu_smear_fwd(P(emb), P(gw), P(lam), None, P(x0), P(sig), tokens, T, dim)
    de, dgw, dlam = torch.empty_like(emb), torch.zeros(24), torch.zeros(1)
    E.nc_emu_smear_bwd(P(emb), P(gw), P(lam), P(sig), P(dx0), P(de), P(dgw), P(dlam), tokens, T, dim)
    want_de, want_dgw, want_dlam = ref.smear_bwd(emb, gw, lam, sig, dx0, T)
    close(de, want_de.reshape(tokens, dim))
    assert torch.allclose(dgw, want_dgw.float().reshape(-1), rtol=2e-2, atol=2e-2 * float(want_dgw.abs().max()))
    assert torch.allclose(dlam, want_dlam.float().reshape(-1), rtol=2e-2, atol=1e-3)
    rows, ld, ncols = 7, 40, 12
    dh, extra = bf(rows, ld, gen=g), torch.randn(rows, ncols, generator=g)
    want = dh.clone()
    want[:, :ncols] = (dh[:, :ncols].float() + extra).to(torch.bfloat16)
    E.nc_emu_add_cols(P(dh), ctypes.c_longlong(ld), P(extra), rows, ncols)
    assert torch.equal(dh, want)


def test_gradient_norm_and_clip_over_several_spans(E):
    g = torch.Generator().manual_seed(5)
    spans = [torch.randn(n, generator=g) for n in (100_003, 17, 4096, 1)]      # tails of every length class
    acc, out = torch.zeros(1, dtype=torch.float64), torch.zeros(2)
    E.nc_emu_grad_norm(_ptrs(spans), (ctypes.c_longlong * 4)(*[s.numel() for s in spans]), 4, P(acc),
                       ctypes.c_float(1.0), P(out), 3)
    norm = torch.cat(spans).double().norm()
    assert abs(float(out[0]) - float(norm)) < 1e-3 and abs(float(out[1]) - 1.0 / float(norm)) < 1e-7
    E.nc_emu_grad_norm(_ptrs(spans), (ctypes.c_longlong * 4)(*[s.numel() for s in spans]), 4, P(acc),
                       ctypes.c_float(0.0), P(out), 3)
    assert float(out[1]) == 1.0


@pytest.mark.parametrize("rows,cols", [(64, 128), (128, 64), (96, 96)])
def test_muon_elementwise_stages(E, rows, cols):
    """Momentum, equilibration, bf16 hand-over, Muon+ / NorMuon statistics and the cautious update for a group of three
    matrices, against the definition run with no Newton-Schulz iteration."""
    import math
    g = torch.Generator().manual_seed(rows * 3 + cols)
    Pn = 3
    grads = [torch.randn(rows, cols, generator=g) * 0.02 for _ in range(Pn)]
    master = [torch.randn(rows, cols, generator=g) * 0.05 for _ in range(Pn)]
    buf1 = [torch.randn(rows, cols, generator=g) * 0.01 for _ in range(Pn)]
    lines = rows if rows >= cols else cols
    buf2 = [torch.rand(lines, generator=g) * 1e-4 for _ in range(Pn)]
    values = [m.to(torch.bfloat16) for m in master]
    gs = torch.tensor([0.5])
    kw = dict(lr=0.02, momentum=0.9, beta2=0.95, weight_decay=0.1)
    rm, rb1, rb2 = torch.stack(master).clone(), torch.stack(buf1).clone(), torch.stack(buf2).clone()
    rv = torch.stack(values).clone()
    ref.muon_update(torch.stack(grads), rm, rv, rb1, rb2, ns_steps=0, grad_scale=0.5, **kw)
    x32, X = torch.empty(Pn, rows, cols), torch.empty(Pn, rows, cols, dtype=torch.bfloat16)
    row_ss, row_scale, all_scale = torch.empty(Pn, rows), torch.empty(Pn, rows), torch.empty(Pn)
    line_ss, scale, line_scale = torch.empty(Pn, lines), torch.empty(Pn), torch.empty(Pn, lines)
    before = [m.clone() for m in master]
    E.nc_emu_muon_group_no_ns(_ptrs(grads), _ptrs(buf1), _ptrs(buf2), _ptrs(master), _ptrs(values), P(x32), P(row_ss),
                              P(row_scale), P(all_scale), P(X), P(line_ss), P(scale), P(line_scale), Pn, rows, cols,
                              ctypes.c_float(kw["momentum"]), ctypes.c_float(kw["beta2"]), ctypes.c_float(kw["lr"]),
                              ctypes.c_float(kw["weight_decay"]), P(gs))
    assert torch.allclose(torch.stack(buf1), rb1, rtol=1e-5, atol=1e-8)
    assert torch.allclose(torch.stack(buf2), rb2, rtol=2e-2, atol=1e-7)          # X passed through bf16
    # after equilibration and normalisation every matrix has Frobenius norm 1 / 1.01
    assert torch.allclose(X.float().flatten(1).norm(dim=1), torch.full((Pn,), 1 / 1.01), rtol=5e-3)
    upd, want = torch.stack(master) - torch.stack(before), rm - torch.stack(before)
    assert float((upd - want).norm() / want.norm()) < 1e-2
    assert float(upd.flatten(1).norm(dim=1).mean()) > 0.5 * kw["lr"] * math.sqrt(min(rows, cols))
    for p in range(Pn):
        assert torch.equal(values[p], master[p].to(torch.bfloat16))


def test_decode_prologue_and_soft_capped_logits(E):
    g = torch.Generator().manual_seed(12)
    B, H, KV, D, page, pages = 3, 4, 2, 128, 16, 6
    qkv = bf(B, (H + 2 * KV) * D, gen=g)
    qk, v = qkv[:, :(H + KV) * D], qkv[:, (H + KV) * D:]
    cos, sin = ref.build_rope(64, D, 10000.0)
    cos, sin = cos.reshape(64, D // 2).float().contiguous(), sin.reshape(64, D // 2).float().contiguous()
    positions = torch.tensor([5, 33, 16], dtype=torch.int32)
    table = torch.tensor([[0, -1, -1], [1, 2, 3], [4, 5, -1]], dtype=torch.int32)
    k_pool = torch.zeros(pages, page, KV, D, dtype=torch.bfloat16)
    v_pool = torch.zeros_like(k_pool)
    q_out, status = torch.empty(B, H, D, dtype=torch.bfloat16), torch.zeros(1, dtype=torch.int32)
    E.nc_emu_decode_prep_append(P(qk), ctypes.c_longlong(qkv.stride(0)), P(v), ctypes.c_longlong(qkv.stride(0)), P(cos),
                                P(sin), P(positions), P(table), 3, page, P(q_out), P(k_pool), P(v_pool), B, H, KV,
                                ctypes.c_float(1e-6), ctypes.c_float(1.2), pages, P(status))
    assert int(status) == 0
    for b in range(B):
        pos = int(positions[b])
        c, s = cos[pos].view(1, 1, 1, D // 2), sin[pos].view(1, 1, 1, D // 2)
        qw, kw_ = ref.qk_prep_fwd(qk[b, :H * D].reshape(1, 1, H, D), qk[b, H * D:].reshape(1, 1, KV, D), c, s, 1e-6, 1.2)
        close(q_out[b], qw.reshape(H, D))
        pg = int(table[b, pos // page])
        close(k_pool[pg, pos % page], kw_.reshape(KV, D))
        assert torch.equal(v_pool[pg, pos % page], v[b].reshape(KV, D))
    assert int((k_pool.float().abs().sum((1, 2, 3)) > 0).sum()) == 3            # one page touched per sequence
    # a position whose page is not mapped: skipped and reported
    positions[0] = 20
    E.nc_emu_decode_prep_append(P(qk), ctypes.c_longlong(qkv.stride(0)), P(v), ctypes.c_longlong(qkv.stride(0)), P(cos),
                                P(sin), P(positions), P(table), 3, page, P(q_out), P(k_pool), P(v_pool), B, H, KV,
                                ctypes.c_float(1e-6), ctypes.c_float(1.2), pages, P(status))
    assert int(status) == 7
    logits = bf(3, 72, scale=20.0, gen=g)
    out = torch.empty(3, 70)
    E.nc_emu_softcap_logits(P(logits), ctypes.c_longlong(72), P(out), 3, 70, ctypes.c_float(15.0))
    assert torch.allclose(out, 15.0 * torch.tanh(logits[:, :70].float() / 15.0), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("rows,cols,lines_are_rows", [(64, 128, 0), (128, 64, 1)])
def test_muon_update_pushed_into_every_rank(E, rows, cols, lines_are_rows):
    """The data-parallel form of the Muon update writes the same master weights as the local form, bit for bit, and
    leaves their bf16 copy at each matrix's offset in every rank's parameter buffer (and nowhere else)."""
    g = torch.Generator().manual_seed(rows + cols)
    Pn, world = 3, 4
    lines = rows if lines_are_rows else cols
    X = bf(Pn, rows, cols, scale=0.1, gen=g)
    scale0, line_scale = torch.rand(Pn, generator=g) + 0.5, torch.rand(Pn, lines, generator=g) + 0.5
    local = [torch.randn(rows, cols, generator=g) * 0.05 for _ in range(Pn)]
    pushed = [m.clone() for m in local]
    local_vals = [torch.zeros(rows, cols, dtype=torch.bfloat16) for _ in range(Pn)]
    E.nc_emu_muon_apply_batched(_ptrs(local), _ptrs(local_vals), P(X), P(scale0), P(line_scale), lines_are_rows, Pn,
                                rows, cols, ctypes.c_float(0.02), ctypes.c_float(0.1), 5)
    n = rows * cols
    offsets = [16, 16 + n + 64, 16 + 2 * n + 128]                    # gaps between the matrices stay untouched
    total = offsets[-1] + n + 40
    bufs = [torch.full((total,), 7.0, dtype=torch.bfloat16) for _ in range(world)]
    E.nc_emu_muon_apply_push_batched(_ptrs(pushed), (ctypes.c_longlong * Pn)(*offsets), _ptrs(bufs), world, P(X),
                                     P(scale0), P(line_scale), lines_are_rows, Pn, rows, cols, ctypes.c_float(0.02),
                                     ctypes.c_float(0.1), 3)
    for p in range(Pn):
        assert torch.equal(pushed[p], local[p])
    keep = torch.ones(total, dtype=torch.bool)
    for p, off in enumerate(offsets):
        keep[off:off + n] = False
        for r in range(world):
            assert torch.equal(bufs[r][off:off + n], local_vals[p].reshape(-1)), (p, r)
    for r in range(world):
        assert bool((bufs[r][keep] == 7.0).all())


def test_the_three_schedules_differ(request):
    lib = ctypes.CDLL(LIB)
    seen = {}
    for name, mode in SCHEDULES.items():
        lib.nc_emu_set_schedule(mode, ctypes.c_ulonglong(7))
        a, b = torch.zeros(64, dtype=torch.int32), torch.zeros(64, dtype=torch.int32)
        lib.nc_emu_selftest_order(P(a), P(b))
        assert sorted(a.tolist()) == list(range(64)) and sorted(b.tolist()) == list(range(64))
        seen[name] = (a.tolist(), b.tolist())
    assert seen["ascending"][0] == list(range(64)) and seen["descending"][0] == list(range(63, -1, -1))
    assert seen["shuffled"][0] not in (seen["ascending"][0], seen["descending"][0])
    # the thread that completes a barrier goes on first: leaving order is not arrival order
    assert seen["ascending"][1][0] == 63 and seen["descending"][1][0] == 0
    lib.nc_emu_set_schedule(0, ctypes.c_ulonglong(1))


@pytest.mark.parametrize("rows,cols,Pn", [(10, 12, 4), (1, 24, 1), (12, 10, 3), (32, 32, 2), (5, 5, 2)])
def test_one_launch_muon_step_of_small_matrices(E, rows, cols, Pn):
    """The gate projections are too small for the batched tensor-core path: their whole Muon step is one kernel, held
    here to the definition (fp32 throughout, five Polar Express iterations)."""
    g = torch.Generator().manual_seed(rows * 100 + cols)
    grads = [torch.randn(rows, cols, generator=g) * 0.02 for _ in range(Pn)]
    master = [torch.randn(rows, cols, generator=g) * 0.05 for _ in range(Pn)]
    buf1 = [torch.randn(rows, cols, generator=g) * 0.01 for _ in range(Pn)]
    lines = rows if rows >= cols else cols
    buf2 = [torch.rand(lines, generator=g) * 1e-3 for _ in range(Pn)]
    values = [torch.zeros(rows, cols, dtype=torch.bfloat16) for _ in range(Pn)]
    kw = dict(lr=0.02, momentum=0.9, beta2=0.95, weight_decay=0.1)
    rm, rb1, rb2 = torch.stack(master).clone(), torch.stack(buf1).clone(), torch.stack(buf2).clone()
    ref.muon_update(torch.stack(grads), rm, None, rb1, rb2, ns_steps=5, grad_scale=0.5, **kw)
    coeffs = torch.tensor(ref.POLAR_COEFFS, dtype=torch.float32).contiguous()
    gs = torch.tensor([0.5])
    before = torch.stack(master).clone()
    E.nc_emu_muon_tiny(_ptrs(grads), _ptrs(buf1), _ptrs(buf2), _ptrs(master), _ptrs(values), Pn, rows, cols,
                       ctypes.c_float(kw["momentum"]), ctypes.c_float(kw["beta2"]), ctypes.c_float(kw["lr"]),
                       ctypes.c_float(kw["weight_decay"]), 5, P(gs), P(coeffs))
    assert torch.allclose(torch.stack(buf1), rb1, rtol=1e-6, atol=1e-9)
    assert torch.allclose(torch.stack(buf2), rb2, rtol=1e-3, atol=1e-9)
    upd, want = torch.stack(master) - before, rm - before
    assert float((upd - want).norm() / want.norm()) < 1e-3, float((upd - want).norm() / want.norm())
    for p in range(Pn):
        assert torch.equal(values[p], master[p].to(torch.bfloat16))
