"""Fixture producers for the areas the upstream fixtures do not cover.

    python -m nanochat_cpp_b200.fixtures.generate [--out tests/data] [--check] [name ...]

The reference produces its `tests/data/*.bin` from the upstream PyTorch model (tools/dump_fixtures.py,
tools/fixture_format.py); this package reads those files as they are. What they cannot pin is what the reference does
not have: batched decoding over a paged, windowed KV cache with prompts of different lengths, and the block-scaled
fp8 formats of the tcgen05 path. The producers below write record files (the same NCRECORD container) for those:

  paged_decode   a seeded 4-layer model, four prompts of different lengths, and for every prompt the soft-capped
                 logits of the plain full-sequence forward (fp32) at the prompt's last position and at each of 24
                 greedy continuation steps: the oracle for prefill_ragged + decode over released pages, on the CPU
                 engine to 1e-4 and on the GPU kernels to bf16 accuracy.
  mxfp8          activations and weights on awkward scales (zeros, a row of subnormals, one huge block), their MXFP8
                 encoding (E4M3 codes + UE8M0 block exponents) by the definition in `ops/fp8.py`, and the fp32 product
                 of the decoded operands: the oracle for the device quantizers (bit for bit) and the block-scaled GEMM.
  train_trace    five optimizer steps of the tiny CPU configuration on the PyTorch-operator engine: loss per step and
                 a checksum per parameter tensor, for the native CPU engine and the C++ GPU engine to reproduce.

Everything is seeded and computed in fp32 on the CPU, so `--check` can regenerate a fixture in memory and compare it
with the committed file (a gate against silent drift of the definitions).
"""
from __future__ import annotations

import argparse
import os
import sys
from collections import OrderedDict

import numpy as np
import torch

from ..config import LOGIT_SOFTCAP, Config
from ..data.record_file import read_records, write_records

MAGIC = "NCB2FIX1"


def _cfg_records(cfg: Config) -> "OrderedDict[str, np.ndarray]":
    r = OrderedDict()
    for k, v in (("layers", cfg.num_layers), ("heads", cfg.num_heads), ("kv_heads", cfg.num_kv_heads),
                 ("embd", cfg.hidden_dim), ("seq", cfg.seq_len), ("vocab", cfg.vocab_size),
                 ("padded_vocab", cfg.padded_vocab_size), ("short_window", cfg.short_window)):
        r["config/" + k] = np.array([v], dtype=np.int32)
    r["config/window_pattern"] = np.frombuffer(cfg.window_pattern.encode(), dtype=np.uint8).copy()
    r["config/rope_base"] = np.array([cfg.rope_base], dtype=np.float32)
    return r


def config_from_records(recs) -> Config:
    g = lambda k: int(recs["config/" + k][0])
    return Config(num_layers=g("layers"), num_heads=g("heads"), num_kv_heads=g("kv_heads"), hidden_dim=g("embd"),
                  seq_len=g("seq"), vocab_size=g("vocab"), padded_vocab_size=g("padded_vocab"),
                  rope_base=float(recs["config/rope_base"][0]),
                  window_pattern=bytes(recs["config/window_pattern"]).decode(),
                  short_window_override=g("short_window"))


def _seeded_model(cfg: Config, seed: int):
    from ..models import GPT
    m = GPT(cfg, "cpu", torch.float32, seed=seed)
    g = torch.Generator().manual_seed(seed + 1)
    for s in m.params.specs:      # the default initialisation zeroes the output projections: make every path count
        if s.name.endswith("c_proj.weight"):
            m.params.m(s.name).copy_(torch.randn(s.shape, generator=g) * 0.05)
    m.params.m("smear_lambda").fill_(0.4)
    m.params.sync_compute()
    return m


# ------------------------------------------------------------------------------------------------- paged decode
PAGED_PROMPT_LENGTHS = (5, 41, 17, 41)
PAGED_STEPS = 24


def produce_paged_decode() -> "OrderedDict[str, np.ndarray]":
    cfg = Config(num_layers=4, num_heads=2, num_kv_heads=1, hidden_dim=128, seq_len=128, vocab_size=320,
                 padded_vocab_size=320, rope_base=10000.0, window_pattern="SSSL", short_window_override=24)
    m = _seeded_model(cfg, seed=11)
    recs = _cfg_records(cfg)
    for n in m.params.names():
        recs["param/" + n] = m.params.m(n).detach().numpy().astype(np.float32).copy()
    g = torch.Generator().manual_seed(5)
    recs["steps"] = np.array([PAGED_STEPS], dtype=np.int32)
    for r, length in enumerate(PAGED_PROMPT_LENGTHS):
        seq = torch.randint(0, cfg.vocab_size, (length,), generator=g).tolist()
        rows = []
        for _ in range(PAGED_STEPS + 1):       # greedy continuation by the plain forward over the whole sequence
            lg = m.logits(torch.tensor([seq]))[0, -1].float()
            lg = LOGIT_SOFTCAP * torch.tanh(lg / LOGIT_SOFTCAP)
            rows.append(lg.numpy().copy())
            seq.append(int(lg.argmax()))
        recs[f"row{r}/prompt"] = np.array(seq[:length], dtype=np.int32)
        recs[f"row{r}/tokens"] = np.array(seq[:length + PAGED_STEPS], dtype=np.int32)   # prompt + greedy tokens
        recs[f"row{r}/logits"] = np.stack(rows).astype(np.float32)   # [steps + 1, vocab]: after the prompt, then per step
    return recs


# ------------------------------------------------------------------------------------------------- MXFP8
def produce_mxfp8() -> "OrderedDict[str, np.ndarray]":
    from ..ops.fp8 import ref_mx_dequantize, ref_mx_quantize
    g = torch.Generator().manual_seed(23)
    M, N, K = 256, 192, 256
    x = torch.randn(M, K, generator=g)
    w = torch.randn(N, K, generator=g) * 0.05
    x[3] = 0.0                                     # an all-zero row: exponent 0 blocks
    x[5] *= 2.0 ** -20                             # tiny magnitudes
    x[7, 32:64] *= 2.0 ** 12                       # one huge block beside ordinary ones
    x[9, 5] = 448.0 * 3.0                          # above the E4M3 maximum before scaling
    w[11] *= 2.0 ** 9
    x, w = x.bfloat16().float(), w.bfloat16().float()   # the kernels read bf16 inputs
    recs = OrderedDict()
    recs["shape"] = np.array([M, N, K], dtype=np.int32)
    for name, t in (("x", x), ("w", w)):
        q, e = ref_mx_quantize(t)
        recs[name] = t.numpy().copy()
        recs[name + "/codes"] = q.view(torch.uint8).numpy().copy()
        recs[name + "/exponents"] = e.numpy().copy()
    y = ref_mx_dequantize(*ref_mx_quantize(x)).double() @ ref_mx_dequantize(*ref_mx_quantize(w)).double().t()
    recs["product"] = y.float().numpy().copy()
    return recs


# ------------------------------------------------------------------------------------------------- training trace
TRACE_STEPS = 5


def trace_config() -> Config:
    # no window override: the C ABI's config has none (the reference derives the short window from the sequence length,
    # include/nanochat/config.h:44-47), and this trace is for engines behind that ABI too. 384 -> window 128.
    return Config(num_layers=2, num_heads=2, num_kv_heads=2, hidden_dim=128, seq_len=384, vocab_size=512,
                  padded_vocab_size=512, rope_base=10000.0, window_pattern="SL")


def trace_batches():
    g = torch.Generator().manual_seed(31)
    cfg = trace_config()
    # Zipf-like ids: a learnable unigram distribution, so the loss falls instead of wandering
    p = 1.0 / torch.arange(1, cfg.vocab_size + 1).float() ** 1.1
    for _ in range(TRACE_STEPS):
        tok = torch.multinomial(p, 2 * (cfg.seq_len + 1), replacement=True, generator=g).view(2, cfg.seq_len + 1)
        yield tok[:, :-1].contiguous(), tok[:, 1:].contiguous()


TRACE_OPT = dict(unembedding_lr=0.004, embedding_lr=0.05, matrix_lr=0.01, scalar_lr=0.05, weight_decay=0.0, clip=1.0,
                 adam_eps=1e-10, muon_ns_steps=5, muon_beta2=0.9)
TRACE_SCHED = dict(num_iterations=TRACE_STEPS, warmup_steps=0, warmdown_ratio=0.5, final_lr_frac=0.0,
                   weight_decay_base=0.0, muon_momentum_warmup_steps=400.0, muon_momentum_start=0.85,
                   muon_momentum_peak=0.97, muon_momentum_final=0.90)


def produce_train_trace() -> "OrderedDict[str, np.ndarray]":
    from ..optim import Optimizer, OptimizerConfig, SchedulerConfig
    cfg = trace_config()
    m = _seeded_model(cfg, seed=17)
    recs = _cfg_records(cfg)
    for n in m.params.names():
        recs["init/" + n] = m.params.m(n).detach().numpy().astype(np.float32).copy()
    opt = Optimizer(m.params, OptimizerConfig(**TRACE_OPT), SchedulerConfig(**TRACE_SCHED))
    losses = []
    for k, (tok, tgt) in enumerate(trace_batches(), start=1):
        m.zero_grad()
        losses.append(float(m.forward_backward(tok.long(), tgt.long())))
        opt.step(k)
    recs["losses"] = np.array(losses, dtype=np.float32)
    for n in m.params.names():
        recs["final/" + n] = m.params.m(n).detach().numpy().astype(np.float32).copy()
    return recs


PRODUCERS = OrderedDict([
    ("paged_decode", ("paged_decode_fixture.bin", produce_paged_decode)),
    ("mxfp8", ("mxfp8_fixture.bin", produce_mxfp8)),
    ("train_trace", ("train_trace_fixture.bin", produce_train_trace)),
])


def compare(recs, path, atol=1e-6) -> list:
    """Names that differ between freshly produced records and the file at `path`."""
    magic, old = read_records(path)
    bad = [] if magic == MAGIC else ["<magic>"]
    for k in set(recs) | set(old):
        if k not in recs or k not in old:
            bad.append(k)
            continue
        a, b = np.asarray(recs[k]), np.asarray(old[k])
        if a.shape != b.shape or a.dtype != b.dtype:
            bad.append(k)
        elif a.dtype.kind == "f":
            if not np.allclose(a, b, rtol=1e-5, atol=atol):
                bad.append(k)
        elif not np.array_equal(a, b):
            bad.append(k)
    return sorted(bad)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("names", nargs="*", help="fixtures to produce (default: all): " + ", ".join(PRODUCERS))
    ap.add_argument("--out", default=os.path.join(os.path.dirname(__file__), "..", "..", "tests", "data"))
    ap.add_argument("--check", action="store_true", help="compare with the files in --out instead of writing them")
    a = ap.parse_args(argv)
    torch.set_num_threads(max(1, min(8, os.cpu_count() or 1)))
    rc = 0
    for name in (a.names or list(PRODUCERS)):
        if name not in PRODUCERS:
            print(f"unknown fixture '{name}'", file=sys.stderr)
            return 2
        fname, fn = PRODUCERS[name]
        path = os.path.join(a.out, fname)
        recs = fn()
        if a.check:
            bad = compare(recs, path)
            print(f"{name}: {'same as ' + fname if not bad else 'differs from ' + fname + ' in ' + ', '.join(bad[:6])}")
            rc |= 1 if bad else 0
        else:
            write_records(path, MAGIC, recs)
            print(f"{name}: wrote {path} ({os.path.getsize(path)} bytes, {len(recs)} records)")
    return rc


if __name__ == "__main__":
    sys.exit(main())
