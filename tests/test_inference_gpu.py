"""Paged-KV inference kernels and the engine on the GPU."""
import pytest
import torch

from nanochat_cpp_b200 import ops
from nanochat_cpp_b200.config import Config
from nanochat_cpp_b200.inference import GenerateParams, InferenceEngine, generate_multi
from nanochat_cpp_b200.models import GPT
from nanochat_cpp_b200.ops import ref

pytestmark = pytest.mark.gpu


def _K():
    from nanochat_cpp_b200.ops import cuda as K
    return K


@pytest.mark.parametrize("H,KV,D,window", [(4, 4, 128, -1), (8, 2, 128, 40), (4, 2, 64, 100)])
def test_paged_decode_kernels(H, KV, D, window):
    K = _K()
    B, max_seq, page = 5, 200, 16
    pages = (max_seq + page - 1) // page
    kp = torch.zeros(B * pages, page, KV, D, device="cuda", dtype=torch.bfloat16)
    vp = torch.zeros_like(kp)
    kp_r, vp_r = kp.clone(), vp.clone()
    table = torch.randperm(B * pages, device="cuda").to(torch.int32).view(B, pages)   # scattered pages
    lens = torch.tensor([1, 17, 64, 150, 199], device="cuda", dtype=torch.int32)
    T = int(lens.max())
    k_new = torch.randn(B, T, KV, D, device="cuda").to(torch.bfloat16)
    v_new = torch.randn(B, T, KV, D, device="cuda").to(torch.bfloat16)
    pos = torch.arange(T, device="cuda", dtype=torch.int32)[None, :].repeat(B, 1)
    pos = torch.where(pos < lens[:, None], pos, torch.full_like(pos, -1))
    K.kv_append(kp, vp, table, pos, k_new, v_new)
    ref.kv_append(kp_r, vp_r, table, pos, k_new, v_new)
    assert torch.equal(kp, kp_r) and torch.equal(vp, vp_r)
    q = torch.randn(B, H, D, device="cuda").to(torch.bfloat16)
    got = K.paged_decode_attention(q, kp, vp, table, lens, window)
    want = ref.paged_decode_attention(q, kp, vp, table, lens, window)
    assert (got.float() - want.float()).abs().max() <= 2e-2 * want.float().abs().max()


def test_engine_matches_torch_ops_and_graph_replay():
    cfg = Config(num_layers=4, num_heads=4, num_kv_heads=2, hidden_dim=512, seq_len=256, vocab_size=1000,
                 padded_vocab_size=1024, window_pattern="SSSL", short_window_override=128)
    m = GPT(cfg, "cuda", torch.bfloat16, seed=2)
    g = torch.Generator().manual_seed(0)
    for s in m.params.specs:
        if s.name.endswith("c_proj.weight"):
            m.params.m(s.name).copy_((torch.randn(s.shape, generator=g) * 0.02).cuda())
    m.params.m("lm_head.weight").copy_((torch.randn(1024, 512, generator=g) * 0.05).cuda())
    m.params.sync_compute()
    prompts = torch.randint(0, cfg.vocab_size, (4, 128), generator=g)
    params = GenerateParams(max_tokens=24)
    eng = InferenceEngine(m, use_cuda_graph=True)
    out_graph = generate_multi(eng, prompts, params)
    eager = InferenceEngine(m, use_cuda_graph=False)
    out_eager = generate_multi(eager, prompts, params)
    assert [s.tokens for s in out_graph] == [s.tokens for s in out_eager]
    # logits of the kernel path against the PyTorch-operator path on the same weights
    cache = eager.new_cache(4, 200)
    lg_k = eager.prefill(cache, prompts.cuda())
    ops.set_mode("torch")
    try:
        cache_t = eager.new_cache(4, 200)
        lg_t = eager.prefill(cache_t, prompts.cuda())
        nxt = lg_t.argmax(-1)
        lg_t2 = eager.decode(cache_t, nxt)
    finally:
        ops.set_mode("kernels")
    lg_k2 = eager.decode(cache, nxt)
    assert (lg_k - lg_t).abs().max() < 0.15 and (lg_k2 - lg_t2).abs().max() < 0.15
    _K().check_status()


def test_graph_replay_follows_the_cache_across_generate_calls():
    """Every `generate_multi` call builds a new cache; the engine's captured decode graph must be rebuilt for it
    (a freed cache's `id()` is reused by the next one). Two calls on one engine, different prompt lengths and the
    same row count, against an engine that never captures."""
    cfg = Config(num_layers=4, num_heads=4, num_kv_heads=2, hidden_dim=512, seq_len=256, vocab_size=1000,
                 padded_vocab_size=1024, window_pattern="SSSL", short_window_override=128)
    m = GPT(cfg, "cuda", torch.bfloat16, seed=3)
    g = torch.Generator().manual_seed(1)
    for s in m.params.specs:
        if s.name.endswith("c_proj.weight"):
            m.params.m(s.name).copy_((torch.randn(s.shape, generator=g) * 0.02).cuda())
    m.params.m("lm_head.weight").copy_((torch.randn(1024, 512, generator=g) * 0.05).cuda())
    m.params.sync_compute()
    eng = InferenceEngine(m, use_cuda_graph=True)
    eager = InferenceEngine(m, use_cuda_graph=False)
    params = GenerateParams(max_tokens=12)
    for length in (96, 40, 96, 64):
        prompts = torch.randint(0, cfg.vocab_size, (3, length), generator=g)
        got = generate_multi(eng, prompts, params)
        want = generate_multi(eager, prompts, params)
        assert [s.tokens for s in got] == [s.tokens for s in want], f"prompt length {length}"
    _K().check_status()


@pytest.mark.parametrize("H,KV", [(10, 10), (4, 2), (3, 1)])
def test_decode_prologue_matches_qk_prep_and_kv_append(H, KV):
    """The one-launch decode prologue writes exactly what `qk_prep_fwd` + `kv_append` write: q dense, k and v in the
    token's page; untouched cache rows stay as they were."""
    K = _K()
    D, B, page, max_pages = 128, 5, 16, 6
    g = torch.Generator(device="cuda").manual_seed(H * 7 + KV)
    width = (H + 2 * KV) * D
    qkv = torch.randn(B, width + 64, device="cuda", generator=g).to(torch.bfloat16)[:, :width]     # padded row stride
    v_own = torch.randn(B, KV * D, device="cuda", generator=g).to(torch.bfloat16)                 # a separate v buffer
    cos, sin = ops.build_rope(page * max_pages, D, 10000.0, torch.device("cuda"))
    pos = torch.tensor([0, 17, 31, 64, 95], device="cuda", dtype=torch.int32)
    table = torch.randperm(B * max_pages, device="cuda", generator=g).to(torch.int32).view(B, max_pages)
    for v_rows in (qkv[:, (H + KV) * D:], v_own):
        k_a = torch.randn(B * max_pages, page, KV, D, device="cuda", generator=g).to(torch.bfloat16)
        v_a = torch.randn_like(k_a)
        k_b, v_b = k_a.clone(), v_a.clone()
        q4 = qkv[:, : H * D].as_strided((B, 1, H, D), (qkv.stride(0), qkv.stride(0), D, 1))
        k4 = qkv[:, H * D:(H + KV) * D].as_strided((B, 1, KV, D), (qkv.stride(0), qkv.stride(0), D, 1),
                                                   qkv.storage_offset() + H * D)
        q_ref, k_ref = K.qk_prep_fwd(q4, k4, cos, sin, positions=pos)
        v4 = v_rows.as_strided((B, 1, KV, D), (v_rows.stride(0), v_rows.stride(0), D, 1), v_rows.storage_offset())
        K.kv_append(k_a, v_a, table, pos.view(B, 1), k_ref, v4)
        q_new = K.decode_prep_append(qkv, v_rows, cos, sin, pos, k_b, v_b, table, H)
        assert torch.equal(q_new, q_ref.reshape(B, H, D))
        assert torch.equal(k_a, k_b) and torch.equal(v_a, v_b)
    K.check_status()


def test_gather_fused_value_gate_and_softcap_match_their_compositions():
    K = _K()
    g = torch.Generator(device="cuda").manual_seed(5)
    B, KV, D, hidden, vocab = 7, 2, 128, 512, 1000
    h = torch.randn(B, hidden, device="cuda", generator=g).to(torch.bfloat16)
    table = torch.randn(vocab, KV * D, device="cuda", generator=g).to(torch.bfloat16)
    gw = (torch.randn(KV, 12, device="cuda", generator=g) * 0.3).to(torch.bfloat16)
    ids = torch.randint(0, vocab, (B,), device="cuda", generator=g).to(torch.int32)
    wide = torch.randn(B, 3 * KV * D, device="cuda", generator=g).to(torch.bfloat16)
    v_a, v_b = wide.clone()[:, KV * D: 2 * KV * D], wide.clone()[:, KV * D: 2 * KV * D]      # strided rows
    _, gate_a = K.value_gate_fwd(h, K.embedding_fwd(ids, table), gw, v_a, D)
    _, gate_b = K.value_gate_fwd_gather(h, ids, table, gw, v_b, D)
    assert torch.equal(v_a, v_b) and torch.equal(gate_a, gate_b)
    lg = (torch.randn(B, 1024, device="cuda", generator=g) * 20).to(torch.bfloat16)
    want = 15.0 * torch.tanh(lg[:, :vocab].float() / 15.0)
    got = K.softcap_logits(lg, vocab, 15.0)
    assert got.dtype == torch.float32 and got.shape == (B, vocab)
    assert (got - want).abs().max() <= 2e-5
    K.check_status()


def test_argmax_rows_takes_the_first_of_equal_maxima():
    K = _K()
    g = torch.Generator(device="cuda").manual_seed(9)
    for rows, width, vocab in ((5, 1024, 1000), (3, 72, 65), (64, 4096, 4096)):
        lg = torch.randn(rows, width, device="cuda", generator=g).to(torch.bfloat16)
        lg[0, 7] = lg[0, vocab - 1] = 50.0                       # a tie: the lower index wins
        lg[1, vocab:] = 99.0                                     # padding columns are ignored
        got = K.argmax_rows(lg, vocab)
        want = lg[:, :vocab].float().argmax(dim=-1)
        assert got.dtype == torch.int64 and torch.equal(got, want) and int(got[0]) == 7
    K.check_status()
