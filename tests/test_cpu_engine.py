"""The native C++ CPU engine through its C ABI, against the upstream-PyTorch fixtures and the Python engine."""
import os

import numpy as np
import torch

from nanochat_cpp_b200.cpu_engine import CpuModel, CpuOptimizer

from fixture_util import config_of, load, model_of, optim_of


def _native_from(recs, prefix="param/"):
    cfg = config_of(recs)
    m = CpuModel(cfg)
    for n in m.names():
        m.write(n, np.array(recs[prefix + n]))
    return cfg, m


def test_forward_backward_and_optimizer_match_debug_state(data_dir):
    recs = load(data_dir, "debug_state.bin")
    cfg, m = _native_from(recs)
    tok, tgt = np.array(recs["input/tokens"]), np.array(recs["input/targets"])
    loss = m.forward_loss(tok, tgt)
    assert abs(loss - float(recs["forward/loss"][0])) < 1e-5
    m.zero_grad()
    m.backward()
    for n in m.names():
        err = np.abs(m.read(n, grad=True) - np.array(recs["grad/" + n]).reshape(-1)).max()
        assert err < 1e-5, (n, err)
    # three optimizer steps
    cfg, m = _native_from(recs, "step/0/param/")
    o = lambda k: float(recs["config/opt/" + k][0])
    opt = CpuOptimizer(m, unembedding_lr=o("unembedding_lr"), embedding_lr=o("embedding_lr"), matrix_lr=o("matrix_lr"),
                       scalar_lr=o("scalar_lr"), weight_decay=o("weight_decay"), clip=o("clip"), adam_eps=o("adam_eps"),
                       num_iterations=0, warmup_steps=0, warmdown_ratio=0.0, final_lr_frac=0.0, weight_decay_base=0.0,
                       muon_momentum_warmup_steps=0.0, muon_momentum_start=0.95, muon_momentum_peak=0.95,
                       muon_momentum_final=0.95)
    for k in range(1, int(recs["config/steps"][0]) + 1):
        m.zero_grad()
        m.forward_loss(tok, tgt)
        m.backward()
        opt.step(k)
        assert abs(m.forward_loss(tok, tgt) - float(recs[f"step/{k}/loss"][0])) < 1e-5, k
        for n in m.names():
            err = np.abs(m.read(n) - np.array(recs[f"step/{k}/param/{n}"]).reshape(-1)).max()
            # 2e-4: backout_lambda's gradient is near zero on this fixture, and AdamW's first steps move a parameter by
            # the sign of its gradient; float (not double) partial sums in the vectorised products and attention
            # change that scalar by 1.1e-4 after three steps, every other tensor by < 5e-5
            assert err < (2e-4 if n == "backout_lambda" else 1e-4), (k, n, err)


def test_generate_score_rl_and_checkpoint(data_dir, tmp_path):
    recs = load(data_dir, "generate_parity.bin")
    _, m = _native_from(recs)
    prompt = np.array(recs["prompt/tokens"]).tolist()
    want = np.array(recs["generate/tokens"]).tolist()
    tokens, mask = m.generate(prompt, max_tokens=len(want) - len(prompt), temperature=0.0)[0]
    assert tokens == want and mask == np.array(recs["generate/mask"]).tolist()
    # scoring: same numbers as the PyTorch engine's score_batch
    cr = load(data_dir, "core_eval.bin")
    g = lambda k: int(cr["config/" + k][0])
    from nanochat_cpp_b200.config import Config
    cfg = Config(num_layers=g("layers"), num_heads=g("heads"), num_kv_heads=g("kv_heads"), hidden_dim=g("embd"),
                 seq_len=g("seq"), vocab_size=g("vocab"), padded_vocab_size=g("padded_vocab"),
                 window_pattern=bytes(cr["config/window_pattern"]).decode())
    sm = CpuModel(cfg)
    for n in sm.names():
        sm.write(n, np.array(cr["param/" + n]))
    toks, lens = np.array(cr["input/tokens"]), np.array(cr["input/lengths"])
    fpos, foff, fids = cr["input/focus_positions"], cr["input/focus_offsets"], cr["input/focus_ids"]
    focus = [(int(fpos[b]), [int(x) for x in fids[foff[b]:foff[b + 1]]]) if fpos[b] >= 0 else None
             for b in range(toks.shape[0])]
    out = sm.score(toks, lens, focus)
    roff, rlog = cr["result/focus_offsets"], cr["result/focus_logits"]
    for b, (nll, arg, fl) in enumerate(out):
        n = int(lens[b]) - 1
        assert np.allclose(nll[:n], cr["result/nll"][b, :n], atol=2e-5)
        assert arg[:n] == cr["result/argmax"][b, :n].tolist()
        assert np.allclose(fl, rlog[roff[b]:roff[b + 1]], atol=2e-5)
    # the RL step gives the same weights as the Python engine
    rl = load(data_dir, "rl_parity.bin")
    from nanochat_cpp_b200.optim import Optimizer
    from nanochat_cpp_b200.post import rl_step
    cfg, ref = model_of(rl)
    oc, sc = optim_of(rl)
    ropt = Optimizer(ref.params, oc, sc)
    _, nat = _native_from(rl)
    nopt = CpuOptimizer(nat, unembedding_lr=oc.unembedding_lr, embedding_lr=oc.embedding_lr, matrix_lr=oc.matrix_lr,
                        scalar_lr=oc.scalar_lr, weight_decay=oc.weight_decay, clip=oc.clip, adam_eps=oc.adam_eps,
                        num_iterations=sc.num_iterations, warmup_steps=sc.warmup_steps,
                        warmdown_ratio=sc.warmdown_ratio, final_lr_frac=sc.final_lr_frac,
                        weight_decay_base=sc.weight_decay_base,
                        muon_momentum_warmup_steps=sc.muon_momentum_warmup_steps,
                        muon_momentum_start=sc.muon_momentum_start, muon_momentum_peak=sc.muon_momentum_peak,
                        muon_momentum_final=sc.muon_momentum_final)
    passes, per = int(rl["config/num_passes"][0]), int(rl["config/examples_per_rank"][0])
    for k in range(int(rl["config/steps"][0])):
        tok, tgt = np.array(rl[f"rollout/{k}/tokens"]), np.array(rl[f"rollout/{k}/targets"])
        adv = np.array(rl[f"rollout/{k}/advantages"])
        a = rl_step(ref, ropt, tok, tgt, adv, passes, per, k + 1).loss
        b = nopt.rl_step(tok, tgt, adv, passes, per, k + 1)
        assert abs(a - b) < 1e-5, (k, a, b)
    for n in nat.names():
        assert np.abs(nat.read(n) - ref.params.m(n).reshape(-1).numpy()).max() < 2e-4, n
    # checkpoint written by the native engine loads in the Python engine
    path = str(tmp_path / "native.ckpt")
    nat.save(path)
    from nanochat_cpp_b200.train.checkpointer import load_checkpoint
    back, _ = load_checkpoint(path, device="cpu", dtype=torch.float32)
    assert np.allclose(back.params.m("lm_head.weight").reshape(-1).numpy(), nat.read("lm_head.weight"))
