"""The reference-style Python API on CPU with the reference's parquet and tokenizer test files."""
import os

import numpy as np

from nanochat_cpp_b200 import api


def test_config_depth_rule():
    c = api.Config(20)
    assert (c.num_layers, c.hidden_dim, c.num_heads, c.head_dim) == (20, 1280, 10, 128)
    c = api.Config(3, vocab_size=487)
    assert c.hidden_dim == 256 and c.num_heads == 2 and c.padded_vocab_size == 512
    flags = api.model_flags(c)
    assert flags[flags.index("--hidden") + 1] == "256"


def test_train_eval_generate_roundtrip(data_dir, tmp_path):
    tok = api.Tokenizer.load(os.path.join(data_dir, "loader_tokenizer.nctoken"))
    cfg = api.Config(num_layers=2, num_heads=8, num_kv_heads=2, hidden_dim=32, seq_len=8, vocab_size=tok.vocab_size,
                     window_pattern="SL")
    model = api.Model(cfg, device="cpu", seed=1234)
    data = api.TokenData(os.path.join(data_dir, "text.parquet"), tok, seq_len=8, batch=2)
    trainer = api.Trainer(model, data, num_iterations=4, warmup_steps=2, optimizer_config=dict(adam_eps=1e-4, clip=0.0),
                          scheduler_config=dict(warmdown_ratio=0.5, final_lr_frac=0.1))
    losses = [loss for _, loss in trainer]
    assert len(losses) == 4 and losses[-1] < losses[0] and all(np.isfinite(losses))
    ev = api.Evaluator(model)
    bpb = ev.bpb(api.TokenData(os.path.join(data_dir, "text.parquet"), tok, seq_len=8, batch=2), 3)
    assert 0.0 < bpb < 12.0
    assert abs(api.evaluate(model, os.path.join(data_dir, "text.parquet"), tok, steps=3, batch=2) - bpb) < 1e-6
    rep = ev.score([[1, 2, 3, 4, 5, 6, 7, 8]], lengths=[6], focus=[(2, [5, 9])])
    assert len(rep.nll[0]) == 8 and rep.argmax[0][5] == -1 and len(rep.focus_logits[0]) == 2
    rows = model.generate(tok.encode("hello", prepend=tok.get_bos_token_id()), max_tokens=5, temperature=0.0)
    assert len(rows) == 1 and sum(rows[0].mask) <= 5
    path = tmp_path / "m.ckpt"
    trainer.save(path)
    other = api.Model.from_checkpoint(path, device="cpu")
    a, b = model.params()[0], other.params()[0]
    assert a.name == b.name and np.allclose(a.value.numpy(), b.value.numpy())
    # forward / backward pieces of the low-level API
    tk, tg = data.next()
    loss = model.forward_loss(tk, tg)
    model.zero_grad()
    model.backward()
    g1 = model.params()[0].grad.clone()
    model.zero_grad()
    model.backward_accumulate(0.5)
    assert np.isfinite(loss) and np.allclose(model.params()[0].grad.numpy(), 0.5 * g1.numpy(), atol=1e-7)
    with model.no_grad():
        try:
            model.backward()
            raise AssertionError("backward inside no_grad must fail")
        except RuntimeError:
            pass
