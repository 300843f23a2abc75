"""Finite-difference checks of the fused backward kernels on the GPU (attention, classifier, q/k preparation, value
gate): the kernel's own forward is differenced, so a backward that agrees with a wrong reference still fails here."""
import pytest
import torch

from gpu_check import fd_regression, on_grid

pytestmark = pytest.mark.gpu


def _K():
    from nanochat_cpp_b200.ops import cuda as K
    return K


@pytest.mark.parametrize("B,T,H,KV,D,window", [(1, 192, 2, 1, 128, -1), (1, 256, 2, 2, 128, 96), (1, 160, 2, 2, 64, 40)])
def test_attention_backward_against_differences_of_the_forward_kernel(B, T, H, KV, D, window):
    K = _K()
    g = torch.Generator(device="cuda").manual_seed(T + D)
    q, k, v = (on_grid((B, T, n, D), span=1.5, gen=g) for n in (H, KV, KV))
    w = torch.randn(B, T, H, D, device="cuda", generator=g)            # loss = sum(o * w)
    o, lse = K.attention_fwd(q, k, v, window)
    dq, dk, dv = K.attention_bwd(q, k, v, o, lse, w.to(torch.bfloat16), window)
    wb = w.to(torch.bfloat16).float()

    def loss():
        out, _ = K.attention_fwd(q, k, v, window)
        return float((out.float() * wb).sum())
    # a probe moves one whole head row (D elements): the change in a single score from one element is below the
    # rounding of the bf16 output row it is observed through
    # the loss is linear in v, so its probe can be large (exact but for the rounding of the output): four times the
    # signal of the q / k probes over the same noise
    # q / k probes follow the sign of the analytic gradient: the strongest direction, so 2^-4 per element is enough
    # signal and the scores move by well under one unit (a random-sign probe large enough to be seen through the
    # rounding of the bf16 output moves them by more, where the softmax is no longer linear)
    for name, x, gr, delta in (("dq", q, dq, 2.0 ** -4), ("dk", k, dk, 2.0 ** -4), ("dv", v, dv, 1.0)):
        fd_regression(loss, x, gr, delta=delta, probes=96, gen=g, name=f"attention {name}", slope_tol=0.1,
                      min_corr=0.93, block=D, aligned=(name != "dv"))
    K.check_status()


def test_classifier_backward_against_differences_of_its_own_loss():
    K = _K()
    g = torch.Generator(device="cuda").manual_seed(3)
    R, vocab, padded = 24, 250, 256
    logits = on_grid((R, padded), step=2.0 ** -3, span=6.0, gen=g)
    targets = torch.randint(0, vocab, (R,), device="cuda", generator=g).to(torch.int32)
    targets[5] = -1
    work = logits.clone()
    _, dl = K.classifier_fwd_bwd(work, targets, vocab, dlogit_scale=1.0)
    dl = dl.clone()

    def loss():
        losses, _ = K.classifier_fwd_bwd(logits.clone(), targets, vocab, dlogit_scale=1.0, want_grad=False)
        return float(losses.double().sum())
    fd_regression(loss, logits, dl, delta=2.0 ** -3, probes=96, gen=g, name="classifier", slope_tol=0.05)
    assert float(dl[5].abs().max()) == 0.0 and float(dl[:, vocab:].abs().max()) == 0.0
    K.check_status()


def test_qk_prep_backward_against_differences_of_the_forward_kernel():
    K = _K()
    from nanochat_cpp_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(8)
    B, T, H, KV, D = 1, 48, 2, 1, 128
    q_pre, k_pre = on_grid((B, T, H, D), gen=g), on_grid((B, T, KV, D), gen=g)
    cos, sin = ops.build_rope(T, D, 10000.0, torch.device("cuda"))
    wq = torch.randn(B, T, H, D, device="cuda", generator=g).to(torch.bfloat16)
    wk = torch.randn(B, T, KV, D, device="cuda", generator=g).to(torch.bfloat16)
    dq, dk = K.qk_prep_bwd(q_pre, k_pre, wq, wk, cos, sin)

    def loss():
        qo, ko = K.qk_prep_fwd(q_pre, k_pre, cos, sin)
        return float((qo.float() * wq.float()).sum() + (ko.float() * wk.float()).sum())
    fd_regression(loss, q_pre, dq, delta=2.0 ** -3, probes=64, gen=g, name="qk_prep dq", slope_tol=0.08, min_corr=0.95)
    fd_regression(loss, k_pre, dk, delta=2.0 ** -3, probes=64, gen=g, name="qk_prep dk", slope_tol=0.08, min_corr=0.95)
    K.check_status()


def test_value_gate_backward_against_differences_of_the_forward_kernel():
    K = _K()
    g = torch.Generator(device="cuda").manual_seed(21)
    M, KV, D, hidden = 40, 2, 128, 256
    h = on_grid((M, hidden), gen=g)
    ve = on_grid((M, KV * D), gen=g)
    gw = on_grid((KV, 12), step=2.0 ** -5, span=0.5, gen=g)
    v0 = on_grid((M, KV * D), gen=g)
    w = torch.randn(M, KV * D, device="cuda", generator=g).to(torch.bfloat16)
    _, gate = K.value_gate_fwd(h, ve, gw, v0.clone(), D)
    dve, dh12, dgw = K.value_gate_bwd(h, ve, gw, gate, w, D)

    def loss():
        v, _ = K.value_gate_fwd(h, ve, gw, v0.clone(), D)
        return float((v.float() * w.float()).sum())
    fd_regression(loss, ve, dve, delta=2.0 ** -3, probes=64, gen=g, name="value gate dve", slope_tol=0.06)
    # only the first 12 channels of h feed the gate
    dh = torch.zeros(M, hidden, device="cuda")
    dh[:, :12] = dh12.float()
    idx_loss_h = h[:, :12]
    full = torch.zeros_like(h, dtype=torch.float32)
    full[:, :12] = dh12.float()
    # probe inside the 12 gate channels: build a contiguous alias of those elements through a helper tensor
    probes = 48
    flat_idx = (torch.randint(0, M, (probes,), device="cuda", generator=g) * hidden +
                torch.randint(0, 12, (probes,), device="cuda", generator=g))
    fd, an = [], []
    hv = h.view(-1)
    for i in flat_idx.tolist():
        old = hv[i].item()
        hv[i] = old + 2.0 ** -3
        fp = loss()
        hv[i] = old - 2.0 ** -3
        fm = loss()
        hv[i] = old
        fd.append((fp - fm) / 2.0 ** -2)
        an.append(full.view(-1)[i].item())
    fd_t, an_t = torch.tensor(fd, dtype=torch.float64), torch.tensor(an, dtype=torch.float64)
    slope = float((fd_t * an_t).sum() / (an_t * an_t).sum())
    corr = float((fd_t * an_t).sum() / (fd_t.norm() * an_t.norm()))
    assert abs(slope - 1.0) < 0.1 and corr > 0.93, (slope, corr)
    fd_regression(loss, gw, dgw, delta=2.0 ** -5, probes=24, gen=g, name="value gate dgw", slope_tol=0.1, min_corr=0.93)
    K.check_status()
