"""Out-of-range indices and stray writes. The gather / scatter kernels check every index against its table before the
access: a bad one is skipped and reported through the device's status word (code 7), so the context stays usable.
The canary tests run kernels with ragged shapes into outputs that sit inside poisoned buffers and check that nothing
outside the output was written."""
import pytest
import torch

from gpu_check import guarded

pytestmark = pytest.mark.gpu


@pytest.fixture()
def K():
    from nanochat_cpp_b200.ops import cuda as K
    K.check_status()
    return K


def _expect_bad_index(K):
    with pytest.raises(RuntimeError, match="status code 7"):
        K.check_status()
    K.check_status()    # the word was reset


def test_embedding_forward_skips_ids_outside_the_table(K):
    table = torch.randn(100, 64, device="cuda").bfloat16()
    ids = torch.tensor([3, 100, 7, -1, 99, 1 << 30], dtype=torch.int32, device="cuda")
    out = K.embedding_fwd(ids, table)
    good = [0, 2, 4]
    assert torch.equal(out[good], table[ids[good].long()])
    assert not out[[1, 3, 5]].any()
    _expect_bad_index(K)


@pytest.mark.parametrize("sorted_order", [False, True])
def test_embedding_backward_skips_ids_outside_the_table(K, sorted_order):
    ids = torch.tensor([5, 250, 5, -7, 0], dtype=torch.int32, device="cuda")
    dout = torch.randn(5, 64, device="cuda").bfloat16()
    with guarded((100, 64), torch.float32) as g:
        K.embedding_bwd(ids, dout, g.out, order=K.embedding_order(ids) if sorted_order else None)
        torch.cuda.synchronize()
        want = torch.zeros(100, 64, device="cuda")
        want[5] = dout[0].float() + dout[2].float()
        want[0] = dout[4].float()
        assert torch.allclose(g.out, want, atol=1e-6)
    _expect_bad_index(K)


def test_value_gate_gather_skips_ids_outside_the_table(K):
    KV, D, vocab = 2, 64, 50
    h = torch.randn(4, 128, device="cuda").bfloat16()
    table = torch.randn(vocab, KV * D, device="cuda").bfloat16()
    gw = torch.randn(KV, 12, device="cuda").bfloat16()
    v = torch.randn(4, KV * D, device="cuda").bfloat16()
    v0 = v.clone()
    ids = torch.tensor([1, vocab, 2, -3], dtype=torch.int32, device="cuda")
    K.value_gate_fwd_gather(h, ids, table, gw, v, D)
    torch.cuda.synchronize()
    assert torch.equal(v[[1, 3]], v0[[1, 3]])          # rows with a bad id keep their value
    assert not torch.equal(v[[0, 2]], v0[[0, 2]])
    _expect_bad_index(K)


def test_classifier_counts_a_target_outside_the_vocabulary_as_ignored(K):
    vocab, padded = 1000, 1024
    logits = torch.randn(4, padded, device="cuda").bfloat16()
    targets = torch.tensor([5, vocab, -1, 1 << 20], dtype=torch.int32, device="cuda")
    losses, dl = K.classifier_fwd_bwd(logits, targets, vocab, dlogit_scale=1.0)
    torch.cuda.synchronize()
    assert losses[0] > 0 and not losses[1:].any()
    assert not dl[1:].any() and dl[0].any()
    _expect_bad_index(K)


def test_kv_append_skips_positions_and_pages_outside_the_pool(K):
    pages, page, KV, D = 4, 16, 2, 64
    with guarded((pages, page, KV, D), torch.bfloat16) as gk, guarded((pages, page, KV, D), torch.bfloat16) as gv:
        table = torch.tensor([[0, 9], [2, 3]], dtype=torch.int32, device="cuda")     # page 9 is not in the pool
        # rows: (seq 0, pos 3) ok; (seq 0, pos 20) -> page 9: skipped; (seq 1, pos 40) past the table: skipped
        positions = torch.tensor([[3, 20], [40, 17]], dtype=torch.int32, device="cuda")
        k_new = torch.randn(2, 2, KV, D, device="cuda").bfloat16()
        v_new = torch.randn(2, 2, KV, D, device="cuda").bfloat16()
        K.kv_append(gk.out, gv.out, table, positions, k_new, v_new)
        torch.cuda.synchronize()
        want = torch.zeros_like(gk.out)
        want[0, 3] = k_new[0, 0]
        want[3, 1] = k_new[1, 1]
        assert torch.equal(gk.out, want)
    _expect_bad_index(K)


@pytest.mark.parametrize("M,N,Kd", [(200, 264, 72), (1000, 1288, 328), (64, 8, 16)])
def test_gemm_writes_nothing_outside_a_ragged_output(K, M, N, Kd):
    a = torch.randn(M, Kd, device="cuda").bfloat16()
    b = torch.randn(N, Kd, device="cuda").bfloat16()
    with guarded((M, N), torch.bfloat16) as g:
        K.gemm(a, b, out=g.out)
        torch.cuda.synchronize()
        want = a.float() @ b.float().t()
        assert torch.allclose(g.out.float(), want, rtol=2e-2, atol=0.3)
    with guarded((N, Kd), torch.float32) as g:       # weight gradient: fp32 accumulate into the flat buffer's span
        dy = torch.randn(M, N, device="cuda").bfloat16()
        K.linear_wgrad(dy, a, g.out, accumulate=False)
        torch.cuda.synchronize()
        assert torch.allclose(g.out, dy.float().t() @ a.float(), rtol=2e-2, atol=0.5)
    K.check_status()


@pytest.mark.parametrize("T,window", [(200, -1), (333, 64)])
def test_attention_backward_writes_nothing_outside_its_outputs(K, T, window):
    B, H, KV, D = 1, 4, 2, 128
    q = torch.randn(B, T, H, D, device="cuda").bfloat16()
    k = torch.randn(B, T, KV, D, device="cuda").bfloat16()
    v = torch.randn(B, T, KV, D, device="cuda").bfloat16()
    o, lse = K.attention_fwd(q, k, v, window_left=window)
    do = torch.randn_like(o)
    with guarded((B, T, (H + 2 * KV) * D), torch.bfloat16) as g:
        out = g.out
        dq = out[..., :H * D].view(B, T, H, D)
        dk = out[..., H * D:(H + KV) * D].view(B, T, KV, D)
        dv = out[..., (H + KV) * D:].view(B, T, KV, D)
        K.attention_bwd(q, k, v, o, lse, do, window_left=window, out=(dq, dk, dv))
        torch.cuda.synchronize()
        assert torch.isfinite(out.float()).all() and out.any()
    K.check_status()
