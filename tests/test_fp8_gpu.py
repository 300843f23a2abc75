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
    q, s = fp8.quantize_rows(x)
    qr, sr = fp8.ref_quantize_rows(x)
    assert torch.equal(s, sr)
    assert torch.equal(q.view(torch.float8_e4m3fn).float(), qr.float())
    w = (torch.randn(256, 384, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    q, s = fp8.quantize_blocks(w)
    qr, sr = fp8.ref_quantize_blocks(w)
    assert torch.equal(s, sr) and torch.equal(q.view(torch.float8_e4m3fn).float(), qr.float())


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
