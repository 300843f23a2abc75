"""The KV page allocator: pages are mapped on demand, windowed layers give back pages that left the window, prompts of
different lengths are prefilled group by group, and none of it changes a logit."""
import pytest
import torch

from nanochat_cpp_b200.config import LOGIT_SOFTCAP, Config
from nanochat_cpp_b200.inference import GenerateParams, InferenceEngine, generate_multi
from nanochat_cpp_b200.inference.engine import PageAllocator, PagedKVCache
from nanochat_cpp_b200.models import GPT


def _model(window=8, seq=256):
    torch.manual_seed(0)
    cfg = Config(num_layers=4, num_heads=4, num_kv_heads=2, hidden_dim=64, seq_len=seq, vocab_size=96,
                 padded_vocab_size=128, rope_base=10000.0, window_pattern="SL", short_window_override=window)
    m = GPT(cfg, "cpu", torch.float32, seed=3)
    for s in m.params.specs:
        if s.name.endswith("c_proj.weight"):
            m.params.m(s.name).normal_(0, 0.05)
    m.params.m("smear_lambda").fill_(0.4)
    m.params.sync_compute()
    return cfg, m


def test_allocator_hands_out_and_takes_back():
    a = PageAllocator(3)
    got = [a.alloc() for _ in range(3)]
    assert sorted(got) == [0, 1, 2] and a.available == 0
    with pytest.raises(MemoryError):
        a.alloc()
    a.release(got[1])
    assert a.alloc() == got[1]


def test_windowed_layers_release_pages_and_logits_do_not_change():
    cfg, m = _model(window=24)
    B, T0, T1 = 2, 40, 100
    tokens = torch.randint(0, cfg.vocab_size, (B, T0 + T1))
    full = LOGIT_SOFTCAP * torch.tanh(m.logits(tokens) / LOGIT_SOFTCAP)
    eng = InferenceEngine(m)
    cache = eng.new_cache(B, T0 + T1 + 1)
    assert cache.is_windowed == [True, False, True, False]
    per_seq = 2 * ((24 + 16) // 16 + 1)
    assert cache.k[0].shape[0] == B * per_seq and cache.k[1].shape[0] == B * cache.pages_per_seq
    lg = eng.prefill(cache, tokens[:, :T0])
    assert (lg - full[:, T0 - 1]).abs().max() < 1e-4
    peak = 0
    for t in range(T0, T0 + T1):
        lg = eng.decode(cache, tokens[:, t])
        assert (lg - full[:, t]).abs().max() < 1e-4, t
        used = cache.pages_in_use()
        peak = max(peak, used["windowed"])
        assert used["full"] == B * ((t + 1 + 15) // 16)
    assert peak <= B * ((24 + 16) // 16 + 1)      # decoding needs half of what a prompt chunk may need
    # the early logical pages of the windowed map were released, the all-history map still holds them
    assert int(cache.win.host[0, 0]) == -1 and int(cache.full.host[0, 0]) >= 0
    cache.reset()
    assert cache.pages_in_use() == {"full": 0, "windowed": 0}


def test_chunked_prefill_longer_than_the_window():
    cfg, m = _model(window=8)
    B, T = 2, 90
    tokens = torch.randint(0, cfg.vocab_size, (B, T))
    full = LOGIT_SOFTCAP * torch.tanh(m.logits(tokens) / LOGIT_SOFTCAP)
    eng = InferenceEngine(m)
    cache = eng.new_cache(B, T + 8)
    eng.prefill(cache, tokens[:, :50])
    lg = eng.prefill(cache, tokens[:, 50:80])
    assert (lg - full[:, 79]).abs().max() < 1e-4
    for t in range(80, T):
        lg = eng.decode(cache, tokens[:, t])
        assert (lg - full[:, t]).abs().max() < 1e-4, t


def test_prompts_of_different_lengths():
    cfg, m = _model(window=8)
    eng = InferenceEngine(m)
    prompts = [torch.randint(0, cfg.vocab_size, (n,)).tolist() for n in (5, 33, 17, 33)]
    cache = eng.new_cache(4, 64)
    lg = eng.prefill_ragged(cache, prompts)
    assert cache.lens_host == [5, 33, 17, 33]
    nxt = lg.argmax(dim=-1)
    lg2 = eng.decode(cache, nxt)
    for r, p in enumerate(prompts):           # each sequence alone gives the same logits
        one = eng.new_cache(1, 64)
        a = eng.prefill(one, torch.tensor([p]))
        assert (a[0] - lg[r]).abs().max() < 1e-4
        b = eng.decode(one, nxt[r:r + 1])
        assert (b[0] - lg2[r]).abs().max() < 1e-4
    # generation over a list of prompts equals generation prompt by prompt
    params = GenerateParams(max_tokens=6, temperature=0.0)
    together = generate_multi(eng, prompts, params)
    for r, p in enumerate(prompts):
        alone = generate_multi(eng, torch.tensor([p]), params)[0]
        assert together[r].tokens == alone.tokens and together[r].mask == alone.mask


def test_an_over_subscribed_pool_runs_out_and_recovers():
    cfg, m = _model(window=8)
    cache = PagedKVCache(cfg, batch=2, max_seq=128, device="cpu", dtype=torch.float32, pool_pages=5)
    eng = InferenceEngine(m)
    eng.prefill(cache, torch.randint(0, cfg.vocab_size, (2, 32)))       # 2 pages per sequence
    assert cache.pages_in_use()["full"] == 4
    tok = torch.zeros(2, dtype=torch.long)
    with pytest.raises(MemoryError):
        for _ in range(40):
            eng.decode(cache, tok)
    cache.reset()
    assert cache.pages_in_use()["full"] == 0
    eng.prefill(cache, torch.randint(0, cfg.vocab_size, (2, 16)))
    assert cache.pages_in_use()["full"] == 2
