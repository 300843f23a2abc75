"""Chat template, SFT packer, calculator tool and tasks against the reference's fixtures."""
import json
import os

import numpy as np
import torch

from nanochat_cpp_b200 import api
from nanochat_cpp_b200.chat import (ARC, GSM8K, MMLU, ChatEngine, PackedRowStream, TaskMixture, evaluate_task,
                                    pack_rows, render_conversation, render_for_completion, use_calculator)


def _json_fixture(path):
    blob = open(path, "rb").read()
    assert blob[:8] == b"NANCHAT1"
    return json.loads(blob[12:])


def test_completion_prompts_match_fixture(data_dir):
    fx = _json_fixture(os.path.join(data_dir, "chat_fixture.bin"))
    tok = api.Tokenizer.load(os.path.join(data_dir, "loader_tokenizer.nctoken"))
    for case in fx["cases"]:
        assert render_for_completion(case["conversation"], tok) == case["prompt_ids"], case["name"]
        ids, mask = render_conversation(case["conversation"], tok)
        assert ids[:len(case["prompt_ids"])] == case["prompt_ids"] and len(ids) == len(mask) and mask[0] == 0


class _PieceTokenizer:
    """The fixture's tokenizer: whole strings map to fixed id lists."""

    def __init__(self, table, specials):
        self.table, self.sp = table, specials

    def encode(self, text):
        return list(self.table[text])

    def encode_special(self, name):
        return self.sp.get(name, -1)

    def get_bos_token_id(self):
        return self.sp["<|bos|>"]


def test_render_mixture_and_packing_match_fixture(data_dir):
    fx = _json_fixture(os.path.join(data_dir, "sft_pack_fixture.bin"))
    names = ["<|bos|>", "<|user_start|>", "<|user_end|>", "<|assistant_start|>", "<|assistant_end|>",
             "<|python_start|>", "<|python_end|>", "<|output_start|>", "<|output_end|>"]
    sp = fx["tokenizer"].get("specials") or {n: i for i, n in enumerate(names)}
    tok = _PieceTokenizer(fx["tokenizer"]["pieces"], sp)
    convs = fx["conversations"]
    for conv, want in zip(convs, fx["render"]):
        ids, mask = render_conversation(conv, tok, max_tokens=fx["settings"]["render_max_tokens"])
        assert ids == want["ids"] and mask == want["mask"], conv.get("name")
    st = fx["settings"]
    n = st["conversations"]
    tokens, targets = pack_rows(convs[:n], tok, st["seq_len"], buffer_size=st["buffer_size"],
                                render_max_tokens=st["render_max_tokens"], rank=st["rank"],
                                world_size=st["world_size"])
    assert tokens[:st["rows"]].tolist() == fx["pack"]["inputs"]
    assert targets[:st["rows"]].tolist() == fx["pack"]["targets"]
    for key in ("mixture", "validation_mixture"):
        mix = TaskMixture([list(range(t["length"])) for t in fx[key]["tasks"]], seed=fx[key]["seed"])
        assert [list(p) for p in mix.index_map] == fx[key]["order"] and len(mix) == fx[key]["conversations"]


def test_calculator():
    assert use_calculator("8 * 5") == "40" and use_calculator("1,000 + 24") == "1024"
    assert use_calculator("7 / 2") == "3.5" and use_calculator("2 ** 8") is None
    assert use_calculator("'strawberry'.count('r')") == "3"
    assert use_calculator("__import__('os')") is None and use_calculator("open('x')") is None


def test_tool_use_and_tasks(data_dir):
    tok = api.Tokenizer.load(os.path.join(data_dir, "loader_tokenizer.nctoken"))
    cfg = api.Config(num_layers=2, num_heads=2, hidden_dim=64, seq_len=128, vocab_size=tok.vocab_size,
                     head_dim=32, window_pattern="L")
    model = api.Model(cfg, device="cpu", seed=5)
    eng = ChatEngine(model, tok)
    sp = eng.sp
    # make the model's "samples" a scripted tool call by forcing through the same hook the engine uses
    script = [sp["<|python_start|>"], *tok.encode("6*7"), sp["<|python_end|>"]]
    prompt = render_for_completion({"messages": [{"role": "user", "content": "6*7?"},
                                                 {"role": "assistant", "content": ""}]}, tok)
    from nanochat_cpp_b200.inference import GenerateParams, generate_multi
    inner = {}

    def hook(r, tokens):
        k = len(tokens) - len(prompt)
        if k < len(script):
            return script[k]
        return inner["forced"](r, tokens)

    # reuse the engine's own state machine for everything after the scripted call
    rows = None
    orig = generate_multi

    def run():
        import nanochat_cpp_b200.inference as inf
        real = inf.generate_multi

        def patched(engine, prompts, params, forced=None):
            inner["forced"] = forced
            return real(engine, prompts, params, forced=hook)
        inf.generate_multi = patched
        try:
            return eng.generate(prompt, max_tokens=len(script) + 6, temperature=0.0)
        finally:
            inf.generate_multi = real
    tokens, mask = run()[0]
    tail = tokens[len(prompt) + len(script):]
    want = [sp["<|output_start|>"], *tok.encode("42"), sp["<|output_end|>"]]
    assert tail[:len(want)] == want and mask[len(prompt) + len(script):][:len(want)] == [0] * len(want)
    # tasks
    mm = MMLU([{"question": "1+1?", "choices": ["1", "2", "3", "4"], "answer": 1, "subject": "math"}] * 3)
    assert mm[0]["messages"][0]["content"].startswith("Multiple Choice question: 1+1?\n- 1=A\n- 2=B")
    rep = evaluate_task(mm, model, tok, batch=2)
    assert rep["total"] == 3 and 0.0 <= rep["accuracy"] <= 1.0
    arc = ARC([{"question": "sky?", "choices": {"text": ["blue", "red"], "label": ["A", "B"]}, "answerKey": "A"}])
    assert arc.evaluate(arc[0], "A") and not arc.evaluate(arc[0], "B")
    g = GSM8K([{"question": "5 boxes of 8?", "answer": "8 * 5 = <<8*5=40>>40\n#### 40"}])
    parts = g[0]["messages"][1]["content"]
    assert [p["type"] for p in parts] == ["text", "python", "python_output", "text"] and parts[1]["text"] == "8*5"
    assert g.evaluate(g[0], "so #### 40") and not g.evaluate(g[0], "#### 41") and g.reward(g[0], "#### 40") == 1.0


def test_rl_loop_in_process_and_over_pipes(data_dir, tmp_path):
    from nanochat_cpp_b200.optim import Optimizer
    from nanochat_cpp_b200.post import RlWorker
    from nanochat_cpp_b200.post.rl_loop import InProcessWorker, PipeWorker, run
    tok = api.Tokenizer.load(os.path.join(data_dir, "loader_tokenizer.nctoken"))
    cfg = api.Config(num_layers=2, num_heads=2, hidden_dim=64, seq_len=64, vocab_size=tok.vocab_size, head_dim=32,
                     window_pattern="L")
    model = api.Model(cfg, device="cpu", seed=5)
    task = GSM8K([{"question": "2+2?", "answer": "#### 4"}, {"question": "3+3?", "answer": "#### 6"}])

    class LengthReward:     # a reward with variance on a random model: longer replies score higher
        def reward(self, conv, text):
            return float(len(text))
    convs = [task[0], task[1]]
    before = model.gpt.params.master.clone()
    ck = str(tmp_path / "rl.ckpt")
    rep = run(InProcessWorker(RlWorker(model.gpt, Optimizer(model.gpt.params))), LengthReward(), convs, tok,
              num_samples=3, steps=2, max_tokens=6, seed=1, checkpoint=ck)
    assert len(rep.losses) == 2 and all(np.isfinite(rep.losses)) and os.path.exists(ck)
    assert not torch.equal(before, model.gpt.params.master)
    env = dict(os.environ, PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    w = PipeWorker.spawn(api.model_flags(cfg), checkpoint=ck, device="cpu", env=env)
    try:
        rep2 = run(w, LengthReward(), convs, tok, num_samples=2, steps=1, max_tokens=4, seed=2)
    finally:
        w.close()
    assert len(rep2.losses) == 1 and np.isfinite(rep2.losses[0])


def test_pipeline_tiny_profile(data_dir, tmp_path):
    from nanochat_cpp_b200.pipeline import run_pipeline
    convs = [{"messages": [{"role": "user", "content": "Say hello."}, {"role": "assistant", "content": "Hello!"}]},
             {"messages": [{"role": "user", "content": "2+2?"}, {"role": "assistant", "content": "#### 4"}]}] * 3
    task = GSM8K([{"question": "2+2?", "answer": "#### 4"}])
    rep = run_pipeline("tiny", str(tmp_path), os.path.join(data_dir, "loader_tokenizer.nctoken"),
                       train_parquet=[os.path.join(data_dir, "text.parquet")], sft_conversations=convs,
                       rl_task=task, rl_conversations=[task[0]], device="cpu")
    assert rep.base["final_step"] == 8 and rep.sft["steps"] == 4 and rep.rl["steps"] == 1
    assert np.isfinite(rep.eval["val_bpb"]) and rep.eval["checkpoint"].endswith("rl.ckpt")
    assert os.path.exists(tmp_path / "pipeline.json")


def test_chat_evaluator_isolation_and_core_means(data_dir, tmp_path):
    from nanochat_cpp_b200.chat import (ALL_TASKS, BASELINES, ChatEvaluator, TaskReport, centered_mean, directory_loader)
    tok = api.Tokenizer.load(os.path.join(data_dir, "loader_tokenizer.nctoken"))
    cfg = api.Config(num_layers=2, num_heads=2, hidden_dim=64, seq_len=128, vocab_size=tok.vocab_size,
                     head_dim=32, window_pattern="L")
    model = api.Model(cfg, device="cpu", seed=5)
    arc_rows = [{"question": "sky?", "choices": {"text": ["blue", "red"], "label": ["A", "B"]}, "answerKey": "A"}] * 4
    mmlu_rows = [{"question": "1+1?", "choices": ["1", "2", "3", "4"], "answer": 1, "subject": "math"}] * 3
    for name, rows in (("ARC-Easy", arc_rows), ("ARC-Challenge", arc_rows[:2]), ("MMLU", mmlu_rows)):
        with open(tmp_path / f"{name}.jsonl", "w") as f:
            f.write("\n".join(json.dumps(r) for r in rows))
    ev = ChatEvaluator(model, tok, task_loader=directory_loader(str(tmp_path)), score_batch=2)
    one = ev.task("MMLU", max_problems=2)
    assert one.total == 2 and one.baseline == 0.25 and 0.0 <= one.accuracy <= 1.0 and not one.skipped
    rep = ev.run()                                  # GSM8K and HumanEval have no data: isolated, not fatal
    assert [r.name for r in rep.tasks] == list(ALL_TASKS)
    skipped = {r.name for r in rep.tasks if r.skipped}
    assert skipped == {"GSM8K", "HumanEval"} and all("FileNotFoundError" in r.error for r in rep.tasks if r.skipped)
    assert rep.chat_core is None                    # a skipped task voids the overall mean
    cat = [r for r in rep.tasks if not r.skipped]
    want = sum((r.accuracy - 0.25) / 0.75 for r in cat) / 3
    assert abs(rep.categorical_core - want) < 1e-12
    import pytest
    with pytest.raises(ValueError):
        ev.task("nonsense")
    with pytest.raises(FileNotFoundError):
        ev.task("GSM8K")
    full = [TaskReport(n, 1, 2, 0.5, BASELINES[n]) for n in ALL_TASKS]
    assert abs(centered_mean(full, ALL_TASKS) - (3 * (0.25 / 0.75) + 2 * 0.5) / 5) < 1e-12
