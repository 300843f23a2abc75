"""Hand-written backward of `models.gpt.GPT` against autograd of `models.ref_gpt` (fp32, CPU)."""
import torch

from nanochat_cpp_b200.config import Config
from nanochat_cpp_b200.models import GPT
from nanochat_cpp_b200.models import ref_gpt


def _cfg(**kw):
    base = dict(num_layers=4, num_heads=4, num_kv_heads=2, hidden_dim=64, seq_len=32, vocab_size=96,
                padded_vocab_size=128, rope_base=10000.0, window_pattern="SL")
    base.update(kw)
    return Config(**base)


def _randomize(model, seed=1):
    g = torch.Generator().manual_seed(seed)
    for s in model.params.specs:
        t = model.params.m(s.name)
        if s.name.endswith("c_proj.weight"):
            t.copy_(torch.randn(t.shape, generator=g) * 0.05)
        if s.name in ("smear_lambda",):
            t.fill_(0.3)
    model.params.sync_compute()


def test_forward_backward_matches_autograd():
    torch.manual_seed(0)
    cfg = _cfg()
    m = GPT(cfg, "cpu", torch.float32, seed=3, head_chunk_rows=40)
    _randomize(m)
    B, T = 3, 32
    tokens = torch.randint(0, cfg.vocab_size, (B, T))
    targets = torch.randint(0, cfg.vocab_size, (B, T))
    targets[0, :5] = -1
    p = {k: v.detach().clone().requires_grad_(True) for k, v in m.state_dict().items()}
    loss_ref = ref_gpt.loss_fn(cfg, p, tokens, targets)
    loss_ref.backward()
    m.zero_grad()
    loss = m.forward_backward(tokens, targets)
    assert abs(loss.item() - loss_ref.item()) < 1e-5
    assert abs(m.forward_loss(tokens, targets).item() - loss_ref.item()) < 1e-5
    for name in m.params.names():
        g = m.params.g(name)
        gr = p[name].grad
        if gr is None:
            gr = torch.zeros_like(g)
        err = (g - gr.view(g.shape)).abs().max().item()
        scale = gr.abs().max().item() + 1e-8
        assert err <= 2e-5 * max(1.0, scale) + 1e-6, (name, err, scale)


def test_grad_accumulates_and_scales():
    cfg = _cfg(num_kv_heads=4, window_pattern="SSSL")
    m = GPT(cfg, "cpu", torch.float32, seed=5)
    _randomize(m, 2)
    tokens = torch.randint(0, cfg.vocab_size, (2, 32))
    targets = torch.randint(0, cfg.vocab_size, (2, 32))
    m.zero_grad()
    m.forward_backward(tokens, targets, grad_scale=0.5)
    g1 = m.params.grad.clone()
    m.forward_backward(tokens, targets, grad_scale=0.5)
    assert torch.allclose(m.params.grad, 2 * g1, rtol=1e-5, atol=1e-7)


def test_backward_memory_modes_agree(monkeypatch):
    """Keeping act / the normalised activations and rebuilding them in the backward give the same gradients."""
    import torch
    from nanochat_cpp_b200.config import Config
    from nanochat_cpp_b200.models import GPT
    cfg = Config(num_layers=2, num_heads=2, num_kv_heads=2, hidden_dim=64, seq_len=32, vocab_size=96,
                 padded_vocab_size=128, window_pattern="SL")
    tok = torch.randint(0, cfg.vocab_size, (2, cfg.seq_len + 1), generator=torch.Generator().manual_seed(0))
    grads = []
    for keep_act, keep_normed in ((True, True), (False, False)):
        m = GPT(cfg, "cpu", torch.float32, seed=4)
        for spec in m.params.specs:
            m.params.m(spec.name).add_(0.02 * torch.randn(spec.shape, generator=torch.Generator().manual_seed(7)))
        m.params.sync_compute()
        m.mlp_keep_act, m.keep_normed = keep_act, keep_normed
        m.zero_grad()
        loss = m.forward_backward(tok[:, :-1], tok[:, 1:])
        grads.append((float(loss), m.params.grad.clone()))
    assert grads[0][0] == grads[1][0]
    torch.testing.assert_close(grads[0][1], grads[1][1], rtol=1e-4, atol=1e-6)


def test_fp8_seam_operators_on_cpu():
    """The seam's fp8 entries run their definition on CPU tensors: codes and exponents of the MXFP8 quantizer, and
    a scaled product that tracks the bf16 product to fp8 accuracy."""
    import torch
    from nanochat_cpp_b200 import ops
    g = torch.Generator().manual_seed(0)
    x = torch.randn(48, 128, generator=g).to(torch.bfloat16)
    w = (torch.randn(40, 128, generator=g) * 0.1).to(torch.bfloat16)
    q, e = ops.quantize_fp8(x)
    assert q.dtype == torch.float8_e4m3fn and e.shape == (48, 4) and e.dtype == torch.uint8
    back = q.float().view(48, 4, 32) * torch.exp2(e.float() - 127).unsqueeze(-1)
    assert (back.view(48, 128) - x.float()).abs().max() <= 0.0715 * x.float().abs().max()
    y, act = ops.gemm_scaled_fp8(x, w, relu2=True)
    exact = x.float() @ w.float().t()
    assert (y.float() - exact).abs().max() <= 8e-2 * exact.abs().max()
    assert torch.equal(act, torch.relu(y.float()).square().to(torch.bfloat16))
