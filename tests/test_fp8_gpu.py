"""Block-scaled fp8: quantizers against their PyTorch definition, the GEMM against an fp32 product of the
dequantized operands."""
import pytest
import torch

from nanochat_cpp_b200.ops import fp8

pytestmark = pytest.mark.gpu


def test_quantizers_match_definition():
    g = torch.Generator(device="cuda").manual_seed(0)
    x = (torch.randn(300, 512, device="cuda", generator=g) * 3).to(torch.bfloat16)
    x[5] = 0                                     # an all-zero row keeps scale 1
    x[7, 130] = 1000.0                           # an outlier stays inside its own 128-block
    def same(q, s, qr, sr):
        # scales agree to an ulp of the division; codes agree except where that ulp moves a value across a
        # rounding boundary (rare, and then by one code)
        assert torch.allclose(s, sr, rtol=3e-7, atol=0)
        a, b = q.view(torch.float8_e4m3fn).float(), qr.float()
        differ = a != b
        assert differ.float().mean().item() < 2e-3
        assert ((a - b).abs()[differ] <= 0.126 * b.abs()[differ].clamp_min(2 ** -6)).all()

    q, s = fp8.quantize_rows(x)
    same(q, s, *fp8.ref_quantize_rows(x))
    assert float(s[0, 5]) == 1.0 and (q[5] == 0).all()                      # the all-zero row
    assert float(s[1, 7]) == pytest.approx(1000.0 / 448.0, rel=1e-6) and float(s[0, 7]) < 0.1
    w = (torch.randn(256, 384, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    q, s = fp8.quantize_blocks(w)
    same(q, s, *fp8.ref_quantize_blocks(w))


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (300, 640, 512), (1024, 1280, 1280), (257, 136, 384)])
def test_fp8_gemm_matches_dequantized_product(M, N, K):
    from nanochat_cpp_b200.ops import cuda as Kmod
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    Np = (N + 127) // 128 * 128
    w_full = (torch.randn(Np, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    xq, sx = fp8.quantize_rows(x)
    wq_full, sw = fp8.quantize_blocks(w_full)
    wq = wq_full[:N].contiguous()                 # N need not be a multiple of 128; the scale table covers the tail
    out = fp8.fp8_gemm(xq, sx, wq, sw)
    want = fp8.ref_fp8_linear(xq.view(torch.float8_e4m3fn), sx, wq_full.view(torch.float8_e4m3fn), sw)[:, :N]
    assert (out.float() - want).abs().max() <= 1e-2 * want.abs().max()
    # and the quantized product tracks the bf16 product to fp8 accuracy
    exact = x.float() @ w_full[:N].float().t()
    assert (out.float() - exact).abs().max() <= 8e-2 * exact.abs().max()
    pre, act = torch.empty_like(out), torch.empty_like(out)
    fp8.fp8_gemm(xq, sx, wq, sw, pre, act)
    assert torch.equal(pre, out) and torch.equal(act, torch.relu(out.float()).square().to(torch.bfloat16))
    Kmod.check_status()


@pytest.mark.parametrize("mode", ["block", "mx"])
def test_model_forward_in_fp8_tracks_bf16_and_trains(mode):
    from nanochat_cpp_b200.config import Config
    from nanochat_cpp_b200.models import GPT
    from nanochat_cpp_b200.optim import Optimizer
    cfg = Config(num_layers=2, num_heads=2, num_kv_heads=2, hidden_dim=256, seq_len=256, vocab_size=512,
                 padded_vocab_size=512, window_pattern="SL", short_window_override=128)
    a = GPT(cfg, "cuda", torch.bfloat16, seed=3)
    b = GPT(cfg, "cuda", torch.bfloat16, seed=3, fp8=mode)
    assert len(b._fp8_w) == 4 and b.fp8_mode == mode
    g = torch.Generator(device="cuda").manual_seed(0)
    for m in (a, b):                      # non-zero projections so that the fp8 products matter
        gg = torch.Generator().manual_seed(1)
        for s in m.params.specs:
            if s.name.endswith("c_proj.weight"):
                m.params.m(s.name).copy_((torch.randn(s.shape, generator=gg) * 0.02).cuda())
        m.params.sync_compute()
    b.refresh_fp8()
    tok = torch.randint(0, 512, (4, 256), device="cuda", generator=g)
    tgt = torch.roll(tok, -1, 1)
    la, lb = float(a.forward_loss(tok, tgt)), float(b.forward_loss(tok, tgt))
    assert abs(la - lb) < 2e-2 * abs(la)
    opt = Optimizer(b.params)
    first = None
    for step in range(1, 6):
        b.zero_grad()
        loss = float(b.forward_backward(tok, tgt))
        opt.step(step)
        b.refresh_fp8()
        first = loss if first is None else first
    assert loss < first


# ------------------------------------------------------------------------------------------------ MXFP8
def test_mx_quantizer_matches_definition_bit_for_bit():
    g = torch.Generator(device="cuda").manual_seed(0)
    x = (torch.randn(300, 512, device="cuda", generator=g) * 3).to(torch.bfloat16)
    x[5] = 0                                     # all-zero blocks keep the neutral exponent 127
    x[7, 130] = 1000.0                           # an outlier only coarsens its own 32-block
    x[9, :32] = 448.0                            # amax / 448 is exactly a power of two: no round-up
    for tile_rows in (128, 192, 224):
        q, sf = fp8.mx_quantize(x, tile_rows)
        qr, ebr = fp8.ref_mx_quantize(x)
        eb = fp8.mx_scales_from_atoms(sf, 300, 512, tile_rows)
        assert torch.equal(eb, ebr)
        assert torch.equal(q.view(torch.float8_e4m3fn).float(), qr.float())
    assert (ebr[5] == 127).all() and int(ebr[9, 0]) == 127
    assert int(ebr[7, 130 // 32]) == 127 + 2 and int(ebr[7, 0]) < 127     # 1000 / 448 -> 2^2
    back = fp8.ref_mx_dequantize(qr, ebr)
    assert (back - x.float()).abs().max() <= 0.0715 * x.float().abs().max()


@pytest.mark.parametrize("M,N,K", [(128, 192, 128), (128, 224, 128), (300, 640, 512), (1024, 1280, 1280),
                                   (257, 136, 384), (2048, 3840, 1280), (515, 5120, 256)])
@pytest.mark.parametrize("variant", [1, 2])          # one CTA per 128-row tile; CTA pairs on 256-row tiles
def test_mx_gemm_matches_dequantized_product(M, N, K, variant):
    from nanochat_cpp_b200.ops import cuda as Kmod
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    x[:, K // 2:] *= 37.0                         # scales differ along K: every scale byte of a column matters
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    w[N // 3:] *= 0.01                            # and along N
    xq, sx = fp8.mx_quantize(x, 128)
    wq, sw = fp8.mx_quantize(w, fp8.mx_tile_n(N))
    out = fp8.mx_gemm(xq, sx, wq, sw, variant=variant)
    xd = fp8.ref_mx_dequantize(*fp8.ref_mx_quantize(x))
    wd = fp8.ref_mx_dequantize(*fp8.ref_mx_quantize(w))
    want = xd @ wd.t()
    assert (out.float() - want).abs().max() <= 1e-2 * want.abs().max()
    exact = x.float() @ w.float().t()
    assert (out.float() - exact).abs().max() <= 8e-2 * exact.abs().max()
    pre, act = torch.empty_like(out), torch.empty_like(out)
    fp8.mx_gemm(xq, sx, wq, sw, pre, act, variant=variant)
    assert torch.equal(pre, out) and torch.equal(act, torch.relu(out.float()).square().to(torch.bfloat16))
    only_act = torch.empty_like(out)
    fp8.mx_gemm(xq, sx, wq, sw, only_act, only_act, variant=variant)
    assert torch.equal(only_act, act)
    Kmod.check_status()


@pytest.mark.parametrize("M,K", [(300, 512), (64, 384), (1025, 1280)])
def test_norm_kernels_emit_the_same_mxfp8_as_the_quantizer(M, K):
    """rmsnorm / blend+rmsnorm with the fused MXFP8 output: bf16 results identical to the plain kernels, codes and
    scales identical to quantizing that bf16 output in a separate pass (K % 256 == 128 covers the half-idle warp)."""
    from nanochat_cpp_b200.ops import cuda as Kmod
    g = torch.Generator(device="cuda").manual_seed(M + K)
    x = (torch.randn(M, K, device="cuda", generator=g) * 2).to(torch.bfloat16)
    x0 = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    y, rstd = Kmod.rmsnorm_fwd(x)
    y2, rstd2, yq, sf = Kmod.rmsnorm_fwd_mx(x)
    assert torch.equal(y, y2) and torch.equal(rstd, rstd2)
    q_ref, sf_ref = fp8.mx_quantize(y, 128)
    assert torch.equal(yq, q_ref)
    assert torch.equal(fp8.mx_scales_from_atoms(sf, M, K, 128), fp8.mx_scales_from_atoms(sf_ref, M, K, 128))
    lr = torch.tensor([0.9], device="cuda")
    l0 = torch.tensor([0.2], device="cuda")
    xr, h, r1 = Kmod.blend_norm_fwd(x, x0, lr, l0)
    xr2, h2, r2, hq, sfh = Kmod.blend_norm_fwd_mx(x, x0, lr, l0)
    assert torch.equal(xr, xr2) and torch.equal(h, h2) and torch.equal(r1, r2)
    q_ref, sf_ref = fp8.mx_quantize(h, 128)
    assert torch.equal(hq, q_ref)
    assert torch.equal(fp8.mx_scales_from_atoms(sfh, M, K, 128), fp8.mx_scales_from_atoms(sf_ref, M, K, 128))
    w = (torch.randn(256, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    wq, sw = fp8.mx_quantize(w, fp8.mx_tile_n(256))
    assert torch.equal(fp8.mx_gemm(hq, sfh, wq, sw), fp8.mx_gemm(q_ref, sf_ref, wq, sw))
    Kmod.check_status()
