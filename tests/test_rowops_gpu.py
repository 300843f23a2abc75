"""Row kernels against the PyTorch definitions in ops.ref (same bf16 inputs, fp32 math)."""
import pytest
import torch

from nanochat_cpp_b200.ops import ref

pytestmark = pytest.mark.gpu


def _K():
    from nanochat_cpp_b200.ops import cuda as K
    return K


def _r(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def _close(a, b, tol=2e-2, name=""):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    mag = b.abs().max().item() + 1e-6
    assert err <= tol * mag, (name, err, mag)


@pytest.mark.parametrize("rows,dim", [(37, 1280), (64, 768), (5, 32), (9, 100)])
def test_rmsnorm(rows, dim):
    K = _K()
    x, dy, res = _r(rows, dim), _r(rows, dim), _r(rows, dim)
    y, rstd = K.rmsnorm_fwd(x)
    yr, rr = ref.rmsnorm_fwd(x)
    _close(y, yr, 1e-2)
    _close(rstd, rr, 1e-4)
    _close(K.rmsnorm_apply(x, rstd), yr, 1e-2)
    _close(K.rmsnorm_bwd(x, dy, rstd, res), ref.rmsnorm_bwd(x, dy, rr, res), 1e-2)
    _close(K.rmsnorm_bwd(x, dy, rstd), ref.rmsnorm_bwd(x, dy, rr), 1e-2)


def test_blend_backout_add():
    K = _K()
    rows, dim = 300, 1280
    x, x0, g = _r(rows, dim), _r(rows, dim), _r(rows, dim)
    a = torch.tensor(1.1, device="cuda")
    b = torch.tensor(0.15, device="cuda")
    xr, h, rstd = K.blend_norm_fwd(x, x0, a, b)
    xr_r, h_r, rstd_r = ref.blend_norm_fwd(x, x0, a, b)
    _close(xr, xr_r, 1e-2)
    _close(h, h_r, 1e-2)
    dx, dx0, dlr, dl0 = K.blend_bwd(g, x, x0, a, b)
    rdx, rdx0, rdlr, rdl0 = ref.blend_bwd(g, x, x0, a, b)
    _close(dx, rdx, 1e-2)
    _close(dx0, rdx0, 1e-2)
    assert abs(dlr.item() - rdlr.item()) <= 2e-3 * abs(rdlr.item()) + 0.5
    assert abs(dl0.item() - rdl0.item()) <= 2e-3 * abs(rdl0.item()) + 0.5
    acc = _r(rows, dim)
    want = ref.add(acc, rdx0)
    K.blend_bwd(g, x, x0, a, b, dx0_acc=acc)
    _close(acc, want, 2e-2)
    lam = torch.tensor(0.2, device="cuda")
    _close(K.backout_fwd(x, x0, lam), ref.backout_fwd(x, x0, lam), 1e-2)
    _, dxb, dlam = K.backout_bwd(g, x0, lam)
    _, rdxb, rdlam = ref.backout_bwd(g, x0, lam)
    _close(dxb, rdxb, 1e-2)
    assert abs(dlam.item() - rdlam.item()) <= 2e-3 * abs(rdlam.item()) + 0.5
    _close(K.add(x, x0), ref.add(x, x0), 1e-2)
    dh = _r(rows, dim)
    extra = torch.randn(rows, 12, device="cuda")
    want = ref.add_cols(dh.clone(), extra)
    _close(K.add_cols(dh, extra), want, 1e-2)


@pytest.mark.parametrize("D,H,KV", [(128, 4, 2), (64, 2, 2), (4, 8, 2)])
def test_qk_prep(D, H, KV):
    K = _K()
    B, T = 2, 24
    wide = _r(B * T, (H + 2 * KV) * D)
    q_pre = wide[:, : H * D].as_strided((B, T, H, D), (T * wide.stride(0), wide.stride(0), D, 1), 0)
    k_pre = wide.as_strided((B, T, KV, D), (T * wide.stride(0), wide.stride(0), D, 1), H * D)
    cos, sin = ref.build_rope(T, D, 10000.0, "cuda")
    q, k = K.qk_prep_fwd(q_pre, k_pre, cos, sin)
    qr, kr = ref.qk_prep_fwd(q_pre, k_pre, cos, sin)
    _close(q, qr, 2e-2)
    _close(k, kr, 2e-2)
    dq, dk = _r(B, T, H, D), _r(B, T, KV, D)
    gq, gk = K.qk_prep_bwd(q_pre, k_pre, dq, dk, cos, sin)
    rq, rk = ref.qk_prep_bwd(q_pre, k_pre, dq, dk, cos, sin)
    _close(gq, rq, 2e-2)
    _close(gk, rk, 2e-2)


def test_value_gate_smear_embedding():
    K = _K()
    M, C, KV, D, V = 96, 256, 2, 64, 50
    h, ve, v = _r(M, C), _r(M, KV * D), _r(M, KV * D)
    gw = _r(KV, 12, scale=0.3)
    v_ref, gate_ref = ref.value_gate_fwd(h, ve, gw, v, D)
    v_out, gate = K.value_gate_fwd(h, ve, gw, v.clone(), D)
    _close(v_out, v_ref, 1e-2)
    _close(gate, gate_ref, 1e-2)
    dv = _r(M, KV * D)
    dve, dh12, dgw = K.value_gate_bwd(h, ve, gw, gate, dv, D)
    rdve, rdh12, rdgw = ref.value_gate_bwd(h, ve, gw, gate, dv, D)
    _close(dve, rdve, 1e-2)
    _close(dh12, rdh12, 1e-2)
    _close(dgw, rdgw, 1e-2)
    seq = 24
    emb = _r(M, C)
    sw = _r(1, 24, scale=0.3)
    lam = torch.tensor(0.4, device="cuda")
    x0, sig = K.smear_fwd(emb, sw, lam, seq)
    rx0, rsig = ref.smear_fwd(emb, sw, lam, seq)
    _close(x0, rx0, 1e-2)
    _close(sig, rsig, 1e-3)
    prev = _r(M // seq, C)
    x0p, sigp = K.smear_fwd(emb, sw, lam, seq, prev)
    rx0p, rsigp = ref.smear_fwd(emb, sw, lam, seq, prev)
    _close(x0p, rx0p, 1e-2)
    g = _r(M, C)
    de, dgw2, dlam = K.smear_bwd(emb, sw, lam, sig, g, seq)
    rde, rdgw2, rdlam = ref.smear_bwd(emb, sw, lam, rsig, g, seq)
    _close(de, rde, 1e-2)
    _close(dgw2, rdgw2, 1e-2)
    assert abs(dlam.item() - rdlam.item()) <= 1e-2 * abs(rdlam.item()) + 1e-2
    ids = torch.randint(0, V, (M,), device="cuda", dtype=torch.int32)
    table = _r(V, C)
    assert torch.equal(K.embedding_fwd(ids, table), ref.embedding_fwd(ids, table))
    dt = torch.zeros(V, C, device="cuda")
    rdt = torch.zeros(V, C, device="cuda")
    K.embedding_bwd(ids, g, dt)
    ref.embedding_bwd(ids, g, rdt)
    _close(dt, rdt, 1e-3)


@pytest.mark.parametrize("vocab,padded", [(4096, 4096), (1000, 1024), (50, 64)])
def test_classifier(vocab, padded):
    K = _K()
    R = 33
    logits = _r(R, padded, scale=6.0)
    targets = torch.randint(0, vocab, (R,), device="cuda", dtype=torch.int32)
    targets[3] = -1
    scale = torch.tensor(0.37, device="cuda")
    rs = torch.rand(R, device="cuda")
    rl, rd = ref.classifier_fwd_bwd(logits.clone(), targets, vocab, dlogit_scale=scale, row_scale=rs)
    l2, _ = K.classifier_fwd_bwd(logits.clone(), targets, vocab, dlogit_scale=None, want_grad=False)
    _close(l2, rl, 2e-3)
    buf = logits.clone()
    l1, d1 = K.classifier_fwd_bwd(buf, targets, vocab, dlogit_scale=scale, row_scale=rs)
    _close(l1, rl, 2e-3)
    _close(d1, rd, 2e-2)
    assert d1.data_ptr() == buf.data_ptr()
    assert float(d1[3].abs().max()) == 0.0
    if padded > vocab:
        assert float(d1[:, vocab:].abs().max()) == 0.0


def test_grad_norm():
    K = _K()
    g = torch.randn(1_000_003, device="cuda")
    norm, scale = K.grad_norm_and_clip([g], 1.0)
    assert abs(norm.item() - g.double().norm().item()) < 1e-2
    assert abs(scale.item() - 1.0 / g.double().norm().item()) < 1e-6
    norm2, scale2 = K.grad_norm_and_clip([g[:1000], g[1000:]], 0.0)
    assert abs(norm2.item() - norm.item()) < 1e-2 and scale2.item() == 1.0


@pytest.mark.parametrize("tokens,vocab,dim", [(4096, 97, 1280), (1000, 5000, 100), (513, 3, 64)])
def test_embedding_bwd_sorted_is_exact_and_reproducible(tokens, vocab, dim):
    """The sorted single-writer scatter: equal to the fp32 index_add, and the same bits on every run."""
    K = _K()
    torch.manual_seed(tokens + vocab)
    ids = torch.randint(0, vocab, (tokens,), device="cuda", dtype=torch.int32)
    ids[: tokens // 3] = 1  # one very frequent token
    g = _r(tokens, dim)
    order = K.embedding_order(ids)
    assert torch.equal(order[0].long(), ids.long()[order[1].long()])
    outs = []
    for _ in range(3):
        dt = torch.ones(vocab, dim, device="cuda", dtype=torch.float32)
        K.embedding_bwd(ids, g, dt, order=order)
        outs.append(dt)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    want = ref.embedding_bwd(ids, g, torch.ones(vocab, dim, device="cuda", dtype=torch.float64)).float()
    torch.testing.assert_close(outs[0], want, rtol=1e-5, atol=1e-4)
    # a strided view (a column slice of a wider buffer) takes the same path
    wide = _r(tokens, dim + 64)
    dt = torch.zeros(vocab, dim, device="cuda", dtype=torch.float32)
    K.embedding_bwd(ids, wide[:, :dim], dt, order=order)
    want = ref.embedding_bwd(ids, wide[:, :dim], torch.zeros(vocab, dim, device="cuda", dtype=torch.float64)).float()
    torch.testing.assert_close(dt, want, rtol=1e-5, atol=1e-4)


@pytest.mark.parametrize("rows,dim,with_extra,accumulate", [(37, 1280, True, True), (64, 768, False, False),
                                                            (130, 256, True, False), (9, 64, False, True)])
def test_norm_blend_backward_fused(rows, dim, with_extra, accumulate):
    """add_cols + rmsnorm_bwd + blend_bwd + scalar-gradient adds in one launch, against the same chain in fp32."""
    from gpu_check import close_elementwise
    K = _K()
    x, x0 = _r(rows, dim), _r(rows, dim)
    lam_r, lam_0 = torch.tensor(0.9, device="cuda"), torch.tensor(0.2, device="cuda")
    xr = (lam_r * x.float() + lam_0 * x0.float()).to(torch.bfloat16)
    _, rstd = ref.rmsnorm_fwd(xr)
    dh, res = _r(rows, dim), _r(rows, dim)
    extra = torch.randn(rows, 12, device="cuda") if with_extra else None
    base = _r(rows, dim) if accumulate else None
    g = torch.tensor([0.5, -0.25], device="cuda")
    gr = g.clone()
    want_dx, want_dx0 = ref.norm_blend_bwd(xr, dh, rstd, res, x, x0, lam_r, lam_0, gr[0:1], gr[1:2],
                                           dx0_acc=base.clone() if accumulate else None, extra=extra)
    acc = base.clone() if accumulate else None
    dh_before = dh.clone()
    dx, dx0 = K.norm_blend_bwd(xr, dh, rstd, res, x, x0, lam_r, lam_0, g[0:1], g[1:2], dx0_acc=acc, extra=extra)
    rms = want_dx.float().square().mean().sqrt().item()
    close_elementwise(dx, want_dx, rtol=2.0 ** -7, atol=2.0 ** -8 * rms, name="dx")
    close_elementwise(dx0, want_dx0, rtol=2.0 ** -7, atol=2.0 ** -7 * want_dx0.float().abs().mean().item(), name="dx0")
    assert torch.allclose(g, gr, rtol=2e-4, atol=1e-2), (g, gr)
    assert torch.equal(dh, dh_before)                     # dh is an input here (the unfused add_cols wrote into it)
    if accumulate:
        assert dx0.data_ptr() == acc.data_ptr()
    K.check_status()
