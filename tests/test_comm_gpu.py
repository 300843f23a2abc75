"""Communication kernels with the ranks emulated on one GPU: each "rank" is a separate set of buffers, flags are
published before any kernel that waits for them is launched, so no launch ever waits for a later one."""
import pytest
import torch

from nanochat_cpp_b200.ops import ref

pytestmark = pytest.mark.gpu


def _K():
    from nanochat_cpp_b200.ops import cuda as K
    return K


def test_reduce_pull_and_flags():
    K = _K()
    C = K._C
    world, n = 4, 1 << 16
    grads = [torch.randn(n, device="cuda") for _ in range(world)]
    flags = [torch.zeros(3 * world, dtype=torch.int32, device="cuda") for _ in range(world)]
    gptrs = [g.data_ptr() for g in grads]
    fptrs = [f.data_ptr() for f in flags]
    want = torch.stack(grads).sum(0) * 0.25
    status = C.status_tensor(0)
    for r in range(world):                      # every rank publishes slot 1 = step 7
        C.comm_signal(fptrs, r, 1, 7)
    torch.cuda.synchronize()
    assert all(int(f[world:2 * world].min()) == 7 for f in flags)
    segs_of = lambda r: torch.tensor([[r * 4096, 4096], [32768 + r * 1024, 1024]], dtype=torch.int64, device="cuda")
    for r in range(world):
        acc = torch.zeros(1, dtype=torch.float64, device="cuda")
        C.comm_reduce_pull(gptrs, r, segs_of(r), 5120, 0.25, flags[r], 1, 7, acc, status, 8)
        for off, cnt in ((r * 4096, 4096), (32768 + r * 1024, 1024)):
            got = grads[r][off:off + cnt]
            assert torch.allclose(got, want[off:off + cnt], rtol=1e-6, atol=1e-6)
        ss = float(want[r * 4096:(r + 1) * 4096].double().square().sum() +
                   want[32768 + r * 1024:32768 + (r + 1) * 1024].double().square().sum())
        assert abs(float(acc) - ss) < 1e-6 * ss
    C.comm_wait(flags[0], world, 1, 7, status)
    K.check_status()


def test_bf16_push_reduce_scatter_with_ranks_emulated_on_one_gpu():
    """grad_push + grad_reduce_local: every "rank" pushes what the others own (bf16, scaled) into their receive
    slots, flags are published, then every owner reduces locally. Runs odd counts so the partial-vector tails are
    exercised, and a poisoned receive buffer so an element nobody pushed would show."""
    K = _K()
    C = K._C
    world, n, scale = 4, 1 << 15, 0.5
    g = torch.Generator(device="cuda").manual_seed(12)
    grads = [torch.randn(n, device="cuda", generator=g) for _ in range(world)]
    orig = [t.clone() for t in grads]
    # owner r holds two runs: a long aligned one and a short odd one
    runs = {r: [(r * 4096, 4096 - 3 * r), (20000 + r * 40, 37)] for r in range(world)}
    placed, cap = {}, 0
    for r in range(world):
        pos, rows = 0, []
        for off, cnt in runs[r]:
            rows.append((off, cnt, pos))
            pos += (cnt + 7) // 8 * 8
        placed[r], cap = rows, max(cap, pos)
    recv = [torch.full((world * cap,), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    rptrs = [t.data_ptr() for t in recv]
    flags = [torch.zeros(2 * world, dtype=torch.int32, device="cuda") for _ in range(world)]
    fptrs = [f.data_ptr() for f in flags]
    status = C.status_tensor(0)
    for src in range(world):
        rows, first = [], 0
        for owner in range(world):
            if owner == src:
                continue
            for off, cnt, pos in placed[owner]:
                rows.append([first, off, pos, owner, cnt])
                first += (cnt + 7) // 8
        C.comm_grad_push(grads[src], rptrs, cap, src, torch.tensor(rows, dtype=torch.int64, device="cuda"), first,
                         scale, 16)
        C.comm_signal(fptrs, src, 1, 3)
    torch.cuda.synchronize()
    for owner in range(world):
        rows, first = [], 0
        for off, cnt, pos in placed[owner]:
            rows.append([first, off, pos, cnt])
            first += (cnt + 7) // 8
        acc = torch.zeros(1, dtype=torch.float64, device="cuda")
        C.comm_grad_reduce_local(grads[owner], recv[owner], cap, world, owner,
                                 torch.tensor(rows, dtype=torch.int64, device="cuda"), first, scale, flags[owner], 1, 3,
                                 acc, status, 8)
        ss = 0.0
        for off, cnt, _ in placed[owner]:
            want = torch.zeros(cnt, device="cuda")
            for r in range(world):
                part = orig[r][off:off + cnt] * scale
                want += part if r == owner else part.to(torch.bfloat16).float()
            got = grads[owner][off:off + cnt]
            assert torch.allclose(got, want, rtol=2e-6, atol=1e-7), (owner, off)     # the kernel may fuse scale * own into an FMA
            ss += float(want.double().square().sum())
        assert abs(float(acc) - ss) <= 1e-6 * ss
        # nothing outside the owned runs was touched
        mask = torch.ones(n, dtype=torch.bool, device="cuda")
        for off, cnt, _ in placed[owner]:
            mask[off:off + cnt] = False
        assert torch.equal(grads[owner][mask], orig[owner][mask])
    K.check_status()


def test_adamw_and_muon_push():
    K = _K()
    C = K._C
    world, n, off = 3, 4096 + 2, 128
    values = [torch.zeros(8192, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    vptrs = [v.data_ptr() for v in values]
    master = torch.randn(n, device="cuda")
    grad = torch.randn(n, device="cuda")
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    rm, rmm, rv = master.clone(), m.clone(), v.clone()
    scale = torch.tensor([0.5], device="cuda")
    kw = dict(lr=0.01, beta1=0.8, beta2=0.95, eps=1e-10, weight_decay=0.01, step=3)
    C.comm_adamw_push(master, vptrs, off, grad, m, v, kw["lr"], kw["beta1"], kw["beta2"], kw["eps"],
                      kw["weight_decay"], kw["step"], scale)
    ref.adamw_update(rm, None, grad, rmm, rv, grad_scale=0.5, **kw)
    assert torch.allclose(master, rm, rtol=1e-5, atol=1e-6)
    for val in values:
        assert torch.equal(val[off:off + n], rm.to(torch.bfloat16)) or \
            (val[off:off + n].float() - rm).abs().max() < 1e-2
        assert float(val[:off].abs().max()) == 0.0
    rows, cols = 64, 96
    mast = torch.randn(rows, cols, device="cuda")
    xb = torch.randn(rows, cols, device="cuda").to(torch.bfloat16)
    s0 = torch.tensor([1.7], device="cuda")
    ls = torch.rand(rows, device="cuda") + 0.5
    x = xb.float() * 1.7 * ls[:, None]
    want = mast - 0.02 * x - torch.where(x * mast >= 0, 0.02 * 0.1 * mast, torch.zeros_like(mast))
    C.comm_muon_apply_push(mast, vptrs, 1024, xb, s0, ls, True, 0.02, 0.1)
    assert torch.allclose(mast, want, rtol=1e-5, atol=1e-6)
    for val in values:
        assert (val[1024:1024 + rows * cols].float().view(rows, cols) - want).abs().max() < 2e-2
    K.check_status()


def test_gemm_waits_for_flags_and_gathers_weight():
    K = _K()
    m, n, k = 512, 768, 256
    x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    w_owner = torch.randn(n, k, device="cuda").to(torch.bfloat16)   # the owner's copy ("peer" memory)
    w_local = torch.zeros_like(w_owner)                               # this rank's stale copy
    flags = torch.full((4,), 5, dtype=torch.int32, device="cuda")    # already published
    out = K.gemm(x, w_owner, wait_flags=flags, wait_value=5)
    want = x.float() @ w_owner.float().t()
    assert (out.float() - want).abs().max() <= 2e-2 * want.abs().max()
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    out2 = K.gemm(x, w_local, gather_src=w_owner.data_ptr(), gather_counter=counter, gather_base=0)
    assert torch.equal(w_local, w_owner)
    assert (out2.float() - want).abs().max() <= 2e-2 * want.abs().max()
    base = int(counter.item())
    w_owner.mul_(2.0)
    out3 = K.gemm(x, w_local, gather_src=w_owner.data_ptr(), gather_counter=counter, gather_base=base)
    assert (out3.float() - 2 * want).abs().max() <= 2e-2 * 2 * want.abs().max()
    K.check_status()


def test_wait_that_runs_out_reports_status_and_context_survives():
    """A flag that nothing sets: the wait gives up after its budget, records the peer-wait code in the status
    word, and the next kernels on the same context run normally."""
    import time
    K = _K()
    dev = torch.device("cuda", torch.cuda.current_device())
    K.check_status()
    flags = torch.zeros(8, dtype=torch.int32, device=dev)
    t0 = time.perf_counter()
    K._C.comm_wait(flags, 2, 1, 5, K._C.status_tensor(dev.index), 300)       # 0.3 s budget
    torch.cuda.synchronize()
    assert 0.25 < time.perf_counter() - t0 < 5.0
    with pytest.raises(RuntimeError, match="status code 5"):
        K.check_status()
    K.check_status()                                                           # the word was cleared
    a = torch.randn(256, 256, device=dev).to(torch.bfloat16)
    assert torch.isfinite(K.gemm(a, a).float()).all()
    flags.fill_(5)
    K._C.comm_wait(flags, 2, 1, 5, K._C.status_tensor(dev.index), 300)        # a satisfied wait returns at once
    K.check_status()
