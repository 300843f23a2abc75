"""The package's own fixtures (fixtures/generate.py, fp32 on the CPU) against the device paths: batched decoding over
released pages, the MXFP8 quantizer and block-scaled GEMM, and the C++ GPU engine's training trace."""
import os

import numpy as np
import pytest
import torch

from nanochat_cpp_b200.data.record_file import read_records
from nanochat_cpp_b200.fixtures import generate as G

pytestmark = pytest.mark.gpu


def test_paged_decode_on_the_device_follows_the_fp32_logits(data_dir):
    from nanochat_cpp_b200.inference import InferenceEngine
    from nanochat_cpp_b200.models import GPT
    from nanochat_cpp_b200.ops import cuda as K
    _, recs = read_records(os.path.join(data_dir, "paged_decode_fixture.bin"))
    cfg = G.config_from_records(recs)
    m = GPT(cfg, "cuda", torch.bfloat16, init=False)
    m.load_state_dict({n: torch.from_numpy(np.array(recs["param/" + n])) for n in m.params.names()})
    rows, steps = len(G.PAGED_PROMPT_LENGTHS), int(recs["steps"][0])
    prompts = [recs[f"row{r}/prompt"].tolist() for r in range(rows)]
    tokens = [recs[f"row{r}/tokens"].tolist() for r in range(rows)]
    want = [torch.from_numpy(np.array(recs[f"row{r}/logits"])).cuda() for r in range(rows)]
    for graphed in (False, True):
        eng = InferenceEngine(m, use_cuda_graph=graphed)
        cache = eng.new_cache(rows, max(len(t) for t in tokens) + 1)
        lg = eng.prefill_ragged(cache, prompts)
        agree = total = 0
        for s in range(steps + 1):
            for r in range(rows):
                err = (lg[r].float() - want[r][s]).abs()
                assert float(err.max()) < 0.08 + 0.05 * float(want[r][s].abs().max()), (graphed, r, s, float(err.max()))
                agree += int(lg[r].argmax() == want[r][s].argmax())
                total += 1
            if s == steps:
                break
            nxt = torch.tensor([tokens[r][len(prompts[r]) + s] for r in range(rows)], device="cuda")   # teacher forced
            lg = eng.decode_graphed(cache, nxt) if graphed else eng.decode(cache, nxt)
        assert agree >= 0.85 * total, (graphed, agree, total)
        assert int(cache.win.host[1, 0]) == -1
    K.check_status()


def test_device_mxfp8_quantizer_and_gemm_against_the_fixture(data_dir):
    from nanochat_cpp_b200.ops import fp8
    _, recs = read_records(os.path.join(data_dir, "mxfp8_fixture.bin"))
    M, N, Kd = (int(v) for v in recs["shape"])
    x = torch.from_numpy(np.array(recs["x"])).cuda().bfloat16()
    w = torch.from_numpy(np.array(recs["w"])).cuda().bfloat16()
    xq, sfx = fp8.mx_quantize(x, 128)
    wq, sfw = fp8.mx_quantize(w, fp8.mx_tile_n(N))
    for q, sf, rows_, tile, name in ((xq, sfx, M, 128, "x"), (wq, sfw, N, fp8.mx_tile_n(N), "w")):
        codes = torch.from_numpy(np.array(recs[name + "/codes"])).cuda()
        exps = torch.from_numpy(np.array(recs[name + "/exponents"])).cuda()
        assert torch.equal(q.view(torch.uint8), codes), name
        assert torch.equal(fp8.mx_scales_from_atoms(sf, rows_, Kd, tile), exps), name
    y = fp8.mx_gemm(xq, sfx, wq, sfw).float()
    want = torch.from_numpy(np.array(recs["product"])).cuda()
    # fp32 accumulation of exact products, one bf16 rounding on the way out
    assert ((y - want).abs() <= 2.0 ** -7 * want.abs() + 1e-3 * want.abs().max()).all()


def test_gpu_engine_behind_the_c_abi_follows_the_training_trace(data_dir):
    from nanochat_cpp_b200 import cpu_engine as E
    _, recs = read_records(os.path.join(data_dir, "train_trace_fixture.bin"))
    cfg = G.config_from_records(recs)
    E.select_device("cuda:0")
    try:
        m = E.CpuModel(cfg, seed=0)
        for n in m.names():
            m.write(n, np.array(recs["init/" + n]).reshape(-1))
        opt = E.CpuOptimizer(m, **G.TRACE_OPT, **G.TRACE_SCHED)
        want = np.array(recs["losses"])
        for k, (tok, tgt) in enumerate(G.trace_batches(), start=1):
            loss = m.train_step(tok.numpy().astype(np.int32), tgt.numpy().astype(np.int32), opt)
            assert abs(loss - want[k - 1]) < 0.04, (k, loss, want[k - 1])     # bf16 compute against the fp32 trace
        assert m.device_status() == 0
    finally:
        E.select_device("cpu")
