"""tcgen05 flash attention (forward and backward) against the fp32 masked-softmax definition."""
import math

import pytest
import torch

from nanochat_cpp_b200.ops import ref

pytestmark = pytest.mark.gpu


def _K():
    from nanochat_cpp_b200.ops import cuda as K
    return K


def _r(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def _close(a, b, tol, name=""):
    """Max-normalised bound, then every element: the probabilities and the score gradients pass through bf16 on
    their way into the second product (2^-9 each, relative to the terms they weight), the result is rounded to
    bf16 once more, so an element may be off by a few 2^-8 of its own size plus of the tensor's typical size."""
    from gpu_check import close_elementwise
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    mag = b.abs().max().item() + 1e-6
    assert err <= tol * mag, (name, err, mag)
    rms = b.square().mean().sqrt().item()
    grad = name.startswith("d")
    close_elementwise(a, b, rtol=2.0 ** -5 if grad else 2.0 ** -6, atol=(2.0 ** -5 if grad else 2.0 ** -6) * rms,
                      name=name, frac=1e-4)


CASES = [
    # B, T, H, KV, D, window
    (2, 256, 2, 2, 128, -1),
    (1, 512, 4, 2, 128, 128),
    (2, 384, 2, 1, 128, 100),
    (1, 200, 2, 2, 128, -1),      # ragged length
    (1, 333, 3, 1, 128, 64),      # ragged + window smaller than a tile + GQA 3
    (2, 256, 2, 2, 64, -1),
    (1, 320, 4, 2, 64, 96),
    (1, 1024, 2, 2, 128, 2048),   # window larger than the sequence
    (1, 777, 2, 2, 128, 40),      # window far below a tile: rows fully masked inside edge tiles
    (2, 2048, 2, 2, 128, 1024),
    (1, 160, 2, 2, 64, 40),       # head_dim 64: ragged length, window below a tile
    (1, 777, 2, 1, 64, 40),
]


@pytest.mark.parametrize("B,T,H,KV,D,window", CASES)
def test_forward_backward(B, T, H, KV, D, window):
    K = _K()
    torch.manual_seed(B * 1000 + T + H + D)
    q, k, v = _r(B, T, H, D), _r(B, T, KV, D), _r(B, T, KV, D)
    do = _r(B, T, H, D)
    o_ref, lse_ref = ref.attention_fwd(q, k, v, window)
    for variant in (1, 2):
        o, lse = K.attention_fwd(q, k, v, window, variant=variant)
        K.check_status()
        _close(o, o_ref, 2e-2, f"o v{variant}")
        _close(lse, lse_ref, 2e-3, f"lse v{variant}")
    dq, dk, dv = K.attention_bwd(q, k, v, o, lse, do, window)
    K.check_status()
    rdq, rdk, rdv = ref.attention_bwd(q, k, v, o_ref, lse_ref, do, window)
    _close(dq, rdq, 3e-2, "dq")
    _close(dk, rdk, 3e-2, "dk")
    _close(dv, rdv, 3e-2, "dv")


def test_strided_views_and_offsets():
    """q/k/v as column slices of one fused QKV buffer, gradients written into one dqkv buffer."""
    K = _K()
    torch.manual_seed(77)
    B, T, H, KV, D = 2, 256, 2, 2, 128
    C = H * D
    qkv = _r(B * T, 3 * C)
    view = lambda off, nh: qkv.as_strided((B, T, nh, D), (T * 3 * C, 3 * C, D, 1), off)
    q, k, v = view(0, H), view(C, KV), view(2 * C, KV)
    o, lse = K.attention_fwd(q, k, v, 128)
    o_ref, lse_ref = ref.attention_fwd(q, k, v, 128)
    _close(o, o_ref, 2e-2)
    do = _r(B, T, H, D)
    dqkv = torch.zeros(B * T, 3 * C, device="cuda", dtype=torch.bfloat16)
    dview = lambda off, nh: dqkv.as_strided((B, T, nh, D), (T * 3 * C, 3 * C, D, 1), off)
    K.attention_bwd(q, k, v, o, lse, do, 128, out=(dview(0, H), dview(C, KV), dview(2 * C, KV)))
    rdq, rdk, rdv = ref.attention_bwd(q, k, v, o_ref, lse_ref, do, 128)
    _close(dview(0, H), rdq, 3e-2, "dq")          # the names select the gradient tolerance
    _close(dview(C, KV), rdk, 3e-2, "dk")
    _close(dview(2 * C, KV), rdv, 3e-2, "dv")
    # decode-style call: 64 new queries against 256 cached keys
    qn = _r(B, 64, H, D)
    o2, _ = K.attention_fwd(qn, k, v, 100)
    o2_ref, _ = ref.attention_fwd(qn, k, v, 100)
    _close(o2, o2_ref, 2e-2)
    K.check_status()


@pytest.mark.parametrize("B,T,H,KV,D,window", [(1, 160, 2, 2, 64, 40), (1, 192, 2, 1, 128, 40), (2, 320, 2, 2, 64, -1)])
def test_forward_repeats_bit_for_bit_on_short_key_sweeps(B, T, H, KV, D, window):
    """Few key tiles per query tile: the epilogue reaches its wait for the output accumulator while products are
    still in flight. The two-tile kernel once read the accumulator two products early there (a parity wait cannot
    tell n - 2 completions from n); the result then changed from launch to launch."""
    K = _K()
    torch.manual_seed(T + D)
    q, k, v = _r(B, T, H, D), _r(B, T, KV, D), _r(B, T, KV, D)
    o_ref, _ = ref.attention_fwd(q, k, v, window)
    first, _ = K.attention_fwd(q, k, v, window, variant=2)
    _close(first, o_ref, 2e-2, "o")
    for _ in range(200):
        again, _ = K.attention_fwd(q, k, v, window, variant=2)
        assert torch.equal(again, first)
    K.check_status()
