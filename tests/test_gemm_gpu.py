"""tcgen05 GEMM against an fp32 PyTorch product: every operand order, every epilogue, ragged shapes."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _K():
    from nanochat_cpp_b200.ops import cuda as K
    return K


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda", dtype=torch.float32) * scale).to(torch.bfloat16)


def _close(got, want, tol=2e-2):
    """Max-normalised bound, then a bound on every element: two bf16 roundings (2^-7 relative) plus, for elements
    that cancel towards zero, 2^-8 of the tensor's typical magnitude (fp32 results: accumulation order only)."""
    from gpu_check import close_elementwise
    is_bf16 = got.dtype == torch.bfloat16
    got, want = got.float(), want.float()
    err = (got - want).abs().max().item()
    ref = want.abs().max().item() + 1e-6
    assert err <= tol * ref, (err, ref)
    rms = want.square().mean().sqrt().item()
    if is_bf16:
        close_elementwise(got, want, rtol=2.0 ** -7, atol=2.0 ** -8 * rms)
    else:
        close_elementwise(got, want, rtol=2.0 ** -12, atol=2.0 ** -12 * rms)


SHAPES = [(128, 256, 64), (256, 512, 128), (384, 768, 1280), (200, 264, 72), (1000, 1288, 328), (64, 8, 16),
          (4096, 1280, 1280)]


@pytest.mark.parametrize("m,n,k", SHAPES)
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
def test_orders(m, n, k, a_mn, b_mn):
    K = _K()
    if (a_mn and m % 8) or (b_mn and n % 8):
        pytest.skip("MN-major operands need a leading dimension that is a multiple of 8")
    A = _rand(m, k)
    B = _rand(n, k)
    a = A.t().contiguous() if a_mn else A
    b = B.t().contiguous() if b_mn else B
    out = K.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    _close(out, A.float() @ B.float().t())
    K.check_status()


def test_epilogues():
    K = _K()
    m, n, k = 512, 768, 320
    A, B = _rand(m, k, scale=0.5), _rand(n, k, scale=0.5)
    R = _rand(m, n)
    want = A.float() @ B.float().t()
    _close(K.gemm(A, B, epi=K.EPI_BF16_RES, r=R, alpha=0.5, beta=2.0), 0.5 * want + 2.0 * R.float())
    pre = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    act = torch.empty_like(pre)
    K.gemm(A, B, epi=K.EPI_RELU2, out=pre, out2=act)
    _close(pre, want)
    assert torch.equal(act, torch.relu(pre.float()).square().to(torch.bfloat16))
    _close(K.gemm(A, B, epi=K.EPI_DRELU2, r=R), want * 2.0 * torch.relu(R.float()))
    g = torch.randn(m, n, device="cuda")
    g0 = g.clone()
    K.gemm(A, B, epi=K.EPI_F32, out=g, beta=1.0)
    _close(g, g0 + want, tol=1e-2)
    K.gemm(A, B, epi=K.EPI_F32, out=g, beta=0.0)
    _close(g, want, tol=1e-2)
    K.check_status()


def test_wgrad_split_k_and_views():
    K = _K()
    tokens, n, k = 8192, 256, 384          # few tiles -> the kernel splits K and reduces with red.add
    dy, x = _rand(tokens, n, scale=0.1), _rand(tokens, k, scale=0.1)
    g = torch.zeros(n, k, device="cuda")
    K.linear_wgrad(dy, x, g, accumulate=False)
    want = dy.float().t() @ x.float()
    _close(g, want, tol=1e-2)
    K.linear_wgrad(dy, x, g, accumulate=True)
    _close(g, 2 * want, tol=1e-2)
    # column-sliced operands (the fused QKV layout): leading dimension larger than the row
    wide = _rand(tokens, 3 * n, scale=0.1)
    part = wide[:, n:2 * n]
    g2 = torch.zeros(n, k, device="cuda")
    K.linear_wgrad(part, x, g2, accumulate=False)
    _close(g2, part.float().t() @ x.float(), tol=1e-2)
    w = _rand(n, k)
    _close(K.linear_dgrad(part, w), part.float() @ w.float())
    K.check_status()


def test_batched():
    K = _K()
    p, r, c = 6, 256, 384
    X = _rand(p, r, c, scale=0.2)
    a = K.gemm(X, X)                       # X X^T per matrix
    _close(a, X.float() @ X.float().transpose(1, 2))
    a2 = K.gemm(a, a, b_mn=True, epi=K.EPI_BF16_RES, r=a, alpha=0.5, beta=-1.5)
    _close(a2, 0.5 * (a.float() @ a.float()) - 1.5 * a.float())
    y = K.gemm(a2, X, b_mn=True, epi=K.EPI_BF16_RES, r=X, alpha=1.0, beta=3.0)
    _close(y, a2.float() @ X.float() + 3.0 * X.float())
    K.check_status()


@pytest.mark.parametrize("M,N,K", [(64, 1280, 1280), (64, 3840, 1280), (7, 1280, 5120), (64, 65536, 1280),
                                   (33, 520, 192), (1, 128, 64)])
def test_skinny_decode_gemm(M, N, K):
    """Small-M products (cluster split-K kernel): plain, residual and relu^2 epilogues."""
    from nanochat_cpp_b200.ops import cuda as Kmod
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N + K)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    r = torch.randn(M, N, device="cuda", generator=g).to(torch.bfloat16)
    want = x.float() @ w.float().t()
    tol = 2e-2 * want.abs().max()
    assert (Kmod.linear_fwd(x, w).float() - want).abs().max() <= tol
    assert (Kmod.linear_fwd(x, w, residual=r).float() - (want + r.float())).abs().max() <= tol + 2e-2 * r.abs().max()
    pre, act = Kmod.linear_relu2_fwd(x, w)
    assert (pre.float() - want).abs().max() <= tol
    assert torch.equal(act, torch.relu(pre.float()).square().to(torch.bfloat16))
    Kmod.check_status()


@pytest.mark.parametrize("M,N,K", [(512, 1024, 256), (300, 520, 192), (8, 256, 128)])
def test_relu2_from_the_saved_activation(M, N, K):
    """MLP with only act = relu(pre)^2 saved: forward without the pre-activation, backward through sqrt(act)."""
    from nanochat_cpp_b200.ops import cuda as Kmod, ref
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    pre, act_two = Kmod.linear_relu2_fwd(x, w)
    act = Kmod.linear_relu2_act_fwd(x, w)
    assert torch.equal(act, act_two)                       # same epilogue, the pre store is just skipped
    dy = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w2 = (torch.randn(K, N, device="cuda", generator=g) * 0.1).to(torch.bfloat16)   # c_proj: [out=K, in=N]
    got = Kmod.linear_dgrad_relu2_act(dy, w2, act).float()
    want = ref.linear_dgrad_relu2_act(dy.float(), w2.float(), act.float())
    assert (got - want).abs().max() <= 2e-2 * want.abs().max()
    # and it agrees with the derivative taken from the pre-activation (sqrt of a bf16 square loses < 1 bf16 ulp)
    from_pre = Kmod.linear_dgrad_relu2(dy, w2, pre).float()
    assert (got - from_pre).abs().max() <= 2e-2 * want.abs().max()
    Kmod.check_status()
