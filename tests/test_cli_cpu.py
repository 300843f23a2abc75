"""The command line on CPU: every sub-command runs end to end on tiny inputs."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from nanochat_cpp_b200 import cli
from nanochat_cpp_b200.data.record_file import read_records

TINY = ["--layers", "2", "--heads", "2", "--hidden", "64", "--seq", "32", "--vocab", "256"]


def test_train_resume_eval_generate(tmp_path, capsys):
    ck = str(tmp_path / "m.ckpt")
    assert cli.main(["train", *TINY, "--synthetic", "--batch", "2", "--num-iterations", "4", "--log-every", "2",
                     "--checkpoint", ck, "--device", "cpu", "--metrics-dir", str(tmp_path)]) == 0
    out = capsys.readouterr().out
    assert "step      4 | loss" in out and os.path.exists(ck) and os.path.exists(ck + ".cursor")
    lines = [json.loads(x) for x in open(tmp_path / "metrics.jsonl")]
    assert [r["step"] for r in lines] == [2, 4] and json.load(open(tmp_path / "summary.json"))["final_step"] == 4
    assert cli.main(["train", *TINY, "--synthetic", "--batch", "2", "--num-iterations", "6", "--log-every", "1",
                     "--resume", ck, "--device", "cpu"]) == 0
    out = capsys.readouterr().out
    assert "resumed" in out and "step      5 |" in out and "step      4 |" not in out
    assert cli.main(["eval", "--model", ck, "--synthetic", "--batch", "2", "--steps", "2", "--device", "cpu"]) == 0
    assert "train bpb" in capsys.readouterr().out
    res = str(tmp_path / "gen.jsonl")
    assert cli.main(["generate", "--model", ck, "--tokens", "1 2 3 4", "--max-tokens", "5", "--num-samples", "2",
                     "--temperature", "0.8", "--seed", "3", "--out", res, "--device", "cpu"]) == 0
    rows = [json.loads(x) for x in open(res)]
    assert len(rows) == 2 and all(r["tokens"][:4] == [1, 2, 3, 4] and len(r["tokens"]) <= 9 for r in rows)


def test_score_rl_sft_roofline_bench(tmp_path, data_dir, capsys):
    out = str(tmp_path / "score.bin")
    assert cli.main(["score", "--fixture", os.path.join(data_dir, "core_eval.bin"), "--out", out,
                     "--device", "cpu"]) == 0
    _, got = read_records(out)
    _, want = read_records(os.path.join(data_dir, "core_eval.bin"))
    assert np.array_equal(got["result/argmax"][0, :7], want["result/argmax"][0, :7])
    assert np.allclose(got["result/focus_logits"], want["result/focus_logits"], atol=2e-5)
    rl = str(tmp_path / "rl.bin")
    assert cli.main(["rl_step", "--fixture", os.path.join(data_dir, "rl_parity.bin"), "--out", rl]) == 0
    _, r1 = read_records(rl)
    rw = str(tmp_path / "rlw.bin")
    assert cli.main(["rl_worker", "--fixture", os.path.join(data_dir, "rl_parity.bin"), "--out", rw,
                     "--save", str(tmp_path / "rl.ckpt"), "--device", "cpu"]) == 0
    _, r2 = read_records(rw)
    assert int(r1["step/2/divisor"][0]) == 24 and np.allclose(r1["param/lm_head.weight"], r2["param/lm_head.weight"])
    assert cli.main(["sft", "--rows", os.path.join(data_dir, "sft_rows_fixture.nchsft"), "--warm-start",
                     os.path.join(data_dir, "sft_base_fixture.ckpt"), "--val-rows",
                     os.path.join(data_dir, "sft_rows_fixture.nchsft"), "--num-iterations", "2", "--grad-accum", "2",
                     "--checkpoint", str(tmp_path / "sft.ckpt"), "--device", "cpu"]) == 0
    err = capsys.readouterr().err
    assert "sft: step 2 epoch 1" in err and "sft: eval step 2 bpb" in err
    assert cli.main(["roofline", "--preset-model", "d20", "--devices", "8", "--json"]) == 0
    rep = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rep["schema"] == "nanochat.roofline.v3" and rep["tokens_per_step"] == 32 * 2048 * 8
    assert cli.main(["eval_bench", *TINY, "--batch", "2", "--iters", "2", "--warmup", "1", "--json",
                     "--device", "cpu"]) == 0
    assert json.loads(capsys.readouterr().out.strip().splitlines()[-1])["schema"] == "nanochat.bench.v3"


def test_rl_worker_pipe_and_tokenizer_training(tmp_path):
    env = dict(os.environ, PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = subprocess.run([sys.executable, "-m", "nanochat_cpp_b200.cli", "rl_worker", *TINY, "--device", "cpu"],
                       input="ping\nrollout prompt_len=3 num_prompts=2 prompts=1,2,3,4,5,6 num_samples=2 max_tokens=4 "
                             "temperature=1.0 seed=7\nquit\n", capture_output=True, text=True, env=env, timeout=300)
    lines = p.stdout.strip().splitlines()
    assert lines[0] == "pong ok=1" and lines[-1] == "quit ok=1", p.stderr[-2000:]
    f = dict(w.split("=") for w in lines[1].split(" ")[1:])
    assert f["ok"] == "1" and f["rows"] == "4"
    lengths = [int(x) for x in f["lengths"].split(",")]
    assert sum(lengths) == len(f["tokens"].split(",")) == len(f["masks"].split(","))
    text = tmp_path / "corpus.txt"
    text.write_text("the quick brown fox jumps over the lazy dog. " * 200)
    out = str(tmp_path / "tok.nctoken")
    assert cli.main(["tok_train", "--text", str(text), "--vocab-size", "300", "--out", out]) == 0
    from nanochat_cpp_b200.data.native import Tokenizer
    t = Tokenizer.load(out)
    assert t.decode(t.encode("the lazy fox")) == "the lazy fox"


def test_workflow_commands_devices_doctor_bench_list(capsys):
    """The workflow verbs exist on the command line; `devices` lists the host first, `doctor` reports the build
    state without failing, `bench list` names every benchmark module and an unknown name is an error."""
    import importlib
    import json
    from nanochat_cpp_b200 import cli, tools_cli
    assert cli.main(["devices"]) == 0
    first = json.loads(capsys.readouterr().out.splitlines()[0])
    assert first["kind"] == "cpu" and first["index"] == -1
    assert cli.main(["doctor"]) == 0
    rep = json.loads(capsys.readouterr().out)
    assert rep["extension_built"] and rep["host_library_built"] and rep["gloo"] and isinstance(rep["problems"], list)
    assert cli.main(["bench", "list"]) == 0
    listed = json.loads(capsys.readouterr().out)
    assert set(tools_cli.BENCHES) | {"step"} == set(listed)
    for mod in tools_cli.BENCHES.values():
        assert importlib.util.find_spec(f"nanochat_cpp_b200.bench.{mod}") is not None
    assert cli.main(["bench", "no-such-benchmark"]) == 2
    capsys.readouterr()
    assert cli.main(["verify"]) in (0, 1)          # 1 with a clear message when no GPU is visible
    assert "ok" in json.loads(capsys.readouterr().out.splitlines()[-1])


def test_seam_and_prune_commands(tmp_path, capsys):
    import json
    import os
    import time
    from nanochat_cpp_b200 import cli, ops, tools_cli
    assert cli.main(["seam"]) == 0
    rows = [json.loads(l) for l in capsys.readouterr().out.splitlines()]
    assert [r["operator"] for r in rows] == list(ops._NAMES) and all(r["definition"] for r in rows)
    assert all(r["kernel"] for r in rows)          # the built extension has a kernel for every operator of the seam
    for i in range(5):
        p = tmp_path / f"step{i}.ckpt"
        p.write_bytes(b"x")
        (tmp_path / f"step{i}.ckpt.cursor").write_bytes(b"y")
        os.utime(p, (time.time() + i, time.time() + i))
    removed = tools_cli.prune_checkpoints(str(tmp_path), keep=2)
    left = sorted(os.listdir(tmp_path))
    assert left == ["step3.ckpt", "step3.ckpt.cursor", "step4.ckpt", "step4.ckpt.cursor"] and len(removed) == 6
    assert cli.main(["prune", "--checkpoints", str(tmp_path), "--keep", "1"]) == 0
    assert sorted(os.listdir(tmp_path)) == ["step4.ckpt", "step4.ckpt.cursor"]
