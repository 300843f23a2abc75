"""Sampling streams: with a temperature, the Python inference engine and the native C++ engine draw the same
tokens for the same seed and weights (one xoshiro256** stream per (seed, row), one draw per sampled position,
inverse-CDF walk; reference src/generate.cc:54, 614-669)."""
import numpy as np
import torch

from nanochat_cpp_b200 import ops
from nanochat_cpp_b200.config import Config
from nanochat_cpp_b200.cpu_engine import CpuModel
from nanochat_cpp_b200.inference import GenerateParams, InferenceEngine, generate_multi
from nanochat_cpp_b200.models import GPT


def test_same_seed_same_rollouts_on_both_engines():
    cfg = Config(num_layers=3, num_heads=2, num_kv_heads=1, hidden_dim=64, seq_len=64, vocab_size=96,
                 padded_vocab_size=128, window_pattern="SL", rope_base=10000.0)
    py = GPT(cfg, "cpu", torch.float32, seed=3)
    g = torch.Generator().manual_seed(1)
    for s in py.params.specs:
        py.params.m(s.name).add_(0.05 * torch.randn(s.shape, generator=g))
    py.params.sync_compute()
    native = CpuModel(cfg, seed=0)
    for s in py.params.specs:
        native.write(s.name, py.params.m(s.name).numpy())
    prompt = torch.randint(0, cfg.vocab_size, (1, 9), generator=g)
    for temperature, top_k in ((1.0, 0), (0.7, 8)):
        params = GenerateParams(num_samples=4, max_tokens=10, temperature=temperature, top_k=top_k, seed=1234)
        got = generate_multi(InferenceEngine(py, use_cuda_graph=False), prompt, params)
        want = native.generate(prompt[0].tolist(), num_samples=4, max_tokens=10, temperature=temperature, top_k=top_k,
                               seed=1234)
        assert [r.tokens for r in got] == [w[0] for w in want]
        assert len({tuple(r.tokens) for r in got}) > 1        # rows really draw from different streams
