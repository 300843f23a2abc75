"""The fixtures this package produces itself (fixtures/generate.py): the committed files are what the producers give
today, and the CPU engines reproduce them."""
import os

import numpy as np
import torch

from nanochat_cpp_b200.data.record_file import read_records
from nanochat_cpp_b200.fixtures import generate as G


def test_committed_files_are_what_the_producers_give(data_dir):
    for name in ("mxfp8", "train_trace"):          # (paged_decode is checked through the engine below)
        fname, fn = G.PRODUCERS[name]
        assert G.compare(fn(), os.path.join(data_dir, fname)) == [], name


def _paged_model(recs):
    from nanochat_cpp_b200.models import GPT
    cfg = G.config_from_records(recs)
    m = GPT(cfg, "cpu", torch.float32, init=False)
    m.load_state_dict({n: torch.from_numpy(np.array(recs["param/" + n])) for n in m.params.names()})
    return cfg, m


def test_paged_engine_reproduces_the_full_forward_logits(data_dir):
    from nanochat_cpp_b200.inference import InferenceEngine
    magic, recs = read_records(os.path.join(data_dir, "paged_decode_fixture.bin"))
    assert magic == G.MAGIC
    cfg, m = _paged_model(recs)
    steps = int(recs["steps"][0])
    rows = len(G.PAGED_PROMPT_LENGTHS)
    prompts = [recs[f"row{r}/prompt"].tolist() for r in range(rows)]
    want = [torch.from_numpy(np.array(recs[f"row{r}/logits"])) for r in range(rows)]
    tokens = [recs[f"row{r}/tokens"].tolist() for r in range(rows)]
    eng = InferenceEngine(m)
    cache = eng.new_cache(rows, max(len(t) for t in tokens) + 1)
    assert any(cache.is_windowed)
    lg = eng.prefill_ragged(cache, prompts)
    for s in range(steps + 1):
        for r in range(rows):
            assert (lg[r] - want[r][s]).abs().max() < 2e-4, (r, s)
        if s == steps:
            break
        nxt = torch.tensor([tokens[r][len(prompts[r]) + s] for r in range(rows)])
        assert torch.equal(nxt, lg.argmax(dim=-1))           # the greedy continuation itself
        lg = eng.decode(cache, nxt)
    assert int(cache.win.host[1, 0]) == -1                   # the longest rows released their first windowed page


def test_mxfp8_definition_properties(data_dir):
    from nanochat_cpp_b200.ops.fp8 import ref_mx_dequantize
    _, recs = read_records(os.path.join(data_dir, "mxfp8_fixture.bin"))
    x = torch.from_numpy(np.array(recs["x"]))
    q = torch.from_numpy(np.array(recs["x/codes"])).view(torch.float8_e4m3fn)
    e = torch.from_numpy(np.array(recs["x/exponents"]))
    back = ref_mx_dequantize(q, e)
    blocks = x.view(x.shape[0], -1, 32)
    amax = blocks.abs().amax(-1)
    scale = torch.exp2(e.float() - 127.0)
    assert (scale * 448.0 >= amax).all()                          # nothing saturates
    assert ((scale * 224.0 < amax) | (amax == 0) | (e == 1)).all()  # and the scale is the smallest such power of two
    assert (e[3] == 127).all() and not back[3].any()              # the all-zero row
    err = (back - x).view_as(blocks).abs().amax(-1)
    assert (err <= scale * 16.0 + 1e-30).all()                    # half a step of the top binade: 32 / 2 in code units


def test_native_cpu_engine_follows_the_training_trace(data_dir):
    from nanochat_cpp_b200.cpu_engine import CpuModel, CpuOptimizer
    _, recs = read_records(os.path.join(data_dir, "train_trace_fixture.bin"))
    cfg = G.config_from_records(recs)
    m = CpuModel(cfg, seed=0)
    for n in m.names():
        m.write(n, np.array(recs["init/" + n]).reshape(-1))
    opt = CpuOptimizer(m, **G.TRACE_OPT, **G.TRACE_SCHED)
    want = np.array(recs["losses"])
    assert want[-1] < want[0] - 0.1                              # the trace learns something
    for k, (tok, tgt) in enumerate(G.trace_batches(), start=1):
        m.zero_grad()
        loss = m.forward_loss(tok.numpy().astype(np.int32), tgt.numpy().astype(np.int32))
        m.backward()
        opt.step(k)
        assert abs(loss - want[k - 1]) < 2e-3, (k, loss, want[k - 1])
    for n in m.names():
        a, b = m.read(n).reshape(-1), np.array(recs["final/" + n]).reshape(-1)
        ref = np.array(recs["init/" + n]).reshape(-1)
        moved = np.linalg.norm(b - ref)
        assert np.linalg.norm(a - b) <= 0.05 * moved + 1e-5, n   # the same update, to 5 % of its own size
