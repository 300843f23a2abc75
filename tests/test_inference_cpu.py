"""Inference engine on CPU (fp32): greedy generation equals the upstream fixture token for token, and the paged
prefill + decode path reproduces the logits of a plain full-sequence forward."""
import os

import numpy as np
import torch

from nanochat_cpp_b200.config import LOGIT_SOFTCAP, Config
from nanochat_cpp_b200.data.record_file import read_records
from nanochat_cpp_b200.inference import GenerateParams, InferenceEngine, generate, generate_multi
from nanochat_cpp_b200.models import GPT


def _fixture_model(recs):
    g = lambda k: int(recs["config/" + k][0])
    cfg = Config(num_layers=g("layers"), num_heads=g("heads"), num_kv_heads=g("kv_heads"), hidden_dim=g("embd"),
                 seq_len=g("seq"), vocab_size=g("vocab"), padded_vocab_size=g("padded_vocab"), rope_base=100000.0,
                 window_pattern=bytes(recs["config/window_pattern"]).decode())
    m = GPT(cfg, "cpu", torch.float32, init=False)
    m.load_state_dict({n: torch.from_numpy(np.array(recs["param/" + n])) for n in m.params.names()})
    return cfg, m


def test_greedy_generation_matches_fixture(data_dir):
    _, recs = read_records(os.path.join(data_dir, "generate_parity.bin"))
    cfg, m = _fixture_model(recs)
    prompt = recs["prompt/tokens"].tolist()
    params = GenerateParams(num_samples=1, max_tokens=int(recs["config/max_tokens"][0]), temperature=0.0,
                            bos_id=int(recs["config/bos_id"][0]))
    out = generate(InferenceEngine(m), prompt, params)[0]
    assert out.tokens == recs["generate/tokens"].tolist()
    assert out.mask == recs["generate/mask"].tolist()


def test_paged_decode_equals_full_forward():
    torch.manual_seed(0)
    cfg = Config(num_layers=4, num_heads=4, num_kv_heads=2, hidden_dim=64, seq_len=64, vocab_size=96,
                 padded_vocab_size=128, rope_base=10000.0, window_pattern="SL", short_window_override=8)
    m = GPT(cfg, "cpu", torch.float32, seed=3)
    for s in m.params.specs:  # non-trivial projections and smear
        if s.name.endswith("c_proj.weight"):
            m.params.m(s.name).normal_(0, 0.05)
    m.params.m("smear_lambda").fill_(0.4)
    m.params.sync_compute()
    B, T0, T1 = 3, 20, 12
    tokens = torch.randint(0, cfg.vocab_size, (B, T0 + T1))
    full = m.logits(tokens)  # raw logits [B, T, vocab]
    full = LOGIT_SOFTCAP * torch.tanh(full / LOGIT_SOFTCAP)
    eng = InferenceEngine(m)
    cache = eng.new_cache(B, T0 + T1 + 4)
    lg = eng.prefill(cache, tokens[:, :T0])
    assert (lg - full[:, T0 - 1]).abs().max() < 1e-4
    for t in range(T0, T0 + T1):
        lg = eng.decode(cache, tokens[:, t])
        assert (lg - full[:, t]).abs().max() < 1e-4, t
    # chunked prefill on top of an existing cache
    cache2 = eng.new_cache(B, T0 + T1 + 4)
    eng.prefill(cache2, tokens[:, :8])
    lg2 = eng.prefill(cache2, tokens[:, 8:T0])
    assert (lg2 - full[:, T0 - 1]).abs().max() < 1e-4


def test_sampling_streams_and_stops():
    cfg = Config(num_layers=2, num_heads=4, num_kv_heads=2, hidden_dim=64, seq_len=32, vocab_size=96,
                 padded_vocab_size=128, rope_base=10000.0, window_pattern="SL")
    m = GPT(cfg, "cpu", torch.float32, seed=1)
    m.params.m("lm_head.weight").normal_(0, 0.5)
    m.params.sync_compute()
    eng = InferenceEngine(m)
    prompts = torch.randint(0, cfg.vocab_size, (2, 5))
    p = GenerateParams(num_samples=3, max_tokens=6, temperature=1.0, top_k=10, seed=11)
    a = generate_multi(eng, prompts, p)
    b = generate_multi(eng, prompts, p)
    assert [s.tokens for s in a] == [s.tokens for s in b]           # one seed reproduces one run
    assert len({tuple(s.tokens) for s in a[:3]}) > 1                 # rows of one prompt draw different streams
    greedy = generate_multi(eng, prompts, GenerateParams(max_tokens=6))
    stop = greedy[0].tokens[5 + 2]
    cut = generate_multi(eng, prompts[:1], GenerateParams(max_tokens=6, stop_id=stop))
    assert cut[0].tokens == greedy[0].tokens[:5 + greedy[0].tokens[5:].index(stop)]
    forced = generate_multi(eng, prompts[:1], GenerateParams(max_tokens=4),
                            forced=lambda r, toks: 7 if len(toks) == 6 else None)
    assert forced[0].tokens[6] == 7 and forced[0].mask[6] == 0 and forced[0].mask[5] == 1
