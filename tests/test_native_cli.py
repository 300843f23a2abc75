"""The native `nanochat_cli` binary (C++ over the C ABI, CPU engine)."""
import json
import os
import subprocess

import numpy as np
import pytest

from nanochat_cpp_b200 import build
from nanochat_cpp_b200.config import Config
from nanochat_cpp_b200.cpu_engine import CpuModel
from nanochat_cpp_b200.post.sft import SftShard, save_sft_shard


@pytest.fixture(scope="module")
def cli():
    build.build_core()
    path = build.build_cli()
    assert path and os.path.exists(path)
    return path


def run(cli, *args, env=None):
    return subprocess.run([cli, *args], capture_output=True, text=True, timeout=300, env=env)


def test_version_params_and_sandbox_contract(cli):
    r = run(cli, "--version")
    assert r.returncode == 0 and "backend cpu" in r.stdout
    r = run(cli, "params", "--preset-model", "tiny")
    p = json.loads(r.stdout)
    cfg = Config(num_layers=2, num_heads=2, num_kv_heads=2, hidden_dim=64, seq_len=64, vocab_size=512,
                 padded_vocab_size=512)
    m = CpuModel(cfg, seed=0)
    assert p["total"] == sum(m.read(n).size for n in m.names())
    env = dict(os.environ, NANOCHAT_SANDBOX_ENFORCE="1")
    env.pop("NANOCHAT_SANDBOX", None)
    assert run(cli, "--version", env=env).returncode == 3
    env["NANOCHAT_SANDBOX"] = "train"
    assert "sandbox train" in run(cli, "--version", env=env).stdout
    assert run(cli, "nonsense").returncode == 2


def test_train_resume_generate(cli, tmp_path):
    rng = np.random.default_rng(0)
    tok = rng.integers(0, 512, size=(16, 65), dtype=np.int32)
    shard = str(tmp_path / "rows.nchsft")
    save_sft_shard(shard, SftShard(tok[:, :-1].copy(), tok[:, 1:].copy()))
    out = str(tmp_path / "run")
    common = ["--preset-model", "tiny", "--rows", shard, "--batch", "4", "--mesh", "2", "--out-dir", out]
    r = run(cli, "train", *common, "--num-iterations", "2")
    assert r.returncode == 0, r.stderr
    assert "2 steps" in r.stdout
    r = run(cli, "train", *common, "--num-iterations", "3", "--resume")
    assert r.returncode == 0 and "1 steps" in r.stdout
    summary = json.load(open(os.path.join(out, "summary.json")))
    assert summary["final_step"] == 3 and summary["world_size"] == 2
    ckpt = os.path.join(out, "checkpoint.ckpt")
    r = run(cli, "generate", "--preset-model", "tiny", "--model", ckpt, "--tokens", "1,2,3", "--max-tokens", "4")
    assert r.returncode == 0
    ids = [int(x) for x in r.stdout.strip().split(",")]
    assert ids[:3] == [1, 2, 3] and len(ids) == 7
    # greedy decoding agrees with the engine driven through Python
    cfg = Config(num_layers=2, num_heads=2, num_kv_heads=2, hidden_dim=64, seq_len=64, vocab_size=512,
                 padded_vocab_size=512)
    m = CpuModel(cfg, seed=0)
    m.load(ckpt)
    rows = m.generate([1, 2, 3], max_tokens=4)
    assert list(rows[0][0]) == ids
    r = run(cli, "train", "--preset-model", "tiny", "--rows", str(tmp_path / "missing"), "--out-dir", out)
    assert r.returncode == 1 and "nanochat_cli" in r.stderr


def test_native_roofline_matches_python_model(cli):
    """The native performance model and the Python one are the same arithmetic: row by row agreement."""
    from nanochat_cpp_b200.config import preset
    from nanochat_cpp_b200.perf import roofline as rf
    from nanochat_cpp_b200.train import mfu
    peaks = mfu.measured_peaks()
    for device, world in (("b200", 8), ("h100", 1)):
        r = run(cli, "roofline", "--preset-model", "d20", "--device", device, "--devices", str(world), "--batch", "32",
                "--bf16-tflops", repr(peaks["bf16_tflops_sustained"]), "--hbm-gbs", repr(peaks["hbm_gbs"]), "--json")
        assert r.returncode == 0, r.stderr
        native = json.loads(r.stdout)
        assert native["schema"] == "nanochat.roofline.v3"
        want = json.loads(rf.report_json(rf.estimate(preset("d20"), rf.RooflinePlan(device=device, world_size=world))))
        assert [x["name"] + x["phase"] for x in native["rows"]] == [x["name"] + x["phase"] for x in want["rows"]]
        for a, b in zip(native["rows"], want["rows"]):
            for k in ("flops", "bytes", "bound_seconds", "mfu"):
                assert abs(a[k] - b[k]) <= 1e-9 * max(1.0, abs(b[k])), (a["name"], k)
            assert a["limit"] == b["limit"]
        for k in ("step_seconds", "tokens_per_second", "model_mfu", "sync_seconds", "optimizer_flops"):
            assert abs(native[k] - want[k]) <= 1e-9 * max(1.0, abs(want[k])), k
    assert "step bound" in run(cli, "roofline", "--preset-model", "d12").stdout


def test_dist_launcher_matches_the_in_process_mesh(cli, tmp_path):
    """Two processes over the TCP ring end with the same weights as two mesh replicas inside one process."""
    rng = np.random.default_rng(1)
    tok = rng.integers(0, 512, size=(16, 65), dtype=np.int32)
    shard = str(tmp_path / "rows.nchsft")
    save_sft_shard(shard, SftShard(tok[:, :-1].copy(), tok[:, 1:].copy()))
    common = ["--preset-model", "tiny", "--rows", shard, "--num-iterations", "3", "--log-every", "1"]
    out_d, out_m = str(tmp_path / "dist"), str(tmp_path / "mesh")
    port = str(20000 + os.getpid() % 20000)
    r = run(cli, "dist", "--world-size", "2", "--port", port, "--", "train", *common, "--batch", "2", "--out-dir", out_d)
    assert r.returncode == 0, (r.stdout, r.stderr)
    assert r.stdout.count("step      3 |") == 1          # only rank 0 logs
    r = run(cli, "train", *common, "--batch", "4", "--mesh", "2", "--out-dir", out_m)
    assert r.returncode == 0, r.stderr
    cfg = Config(num_layers=2, num_heads=2, num_kv_heads=2, hidden_dim=64, seq_len=64, vocab_size=512,
                 padded_vocab_size=512)
    a, b = CpuModel(cfg, seed=0), CpuModel(cfg, seed=1)
    a.load(os.path.join(out_d, "checkpoint.ckpt"))
    b.load(os.path.join(out_m, "checkpoint.ckpt"))
    for name in a.names():
        assert np.array_equal(a.read(name), b.read(name)), name
    assert json.load(open(os.path.join(out_d, "summary.json")))["world_size"] == 2
    # a rank that never joins: the launcher reports the failure instead of hanging
    r = run(cli, "train", *common, "--batch", "2", "--rank", "1", "--world-size", "2", "--port", port, "--timeout-ms",
            "500", "--out-dir", out_d)
    assert r.returncode == 1 and "rendezvous" in r.stderr


def test_native_score_matches_the_fixture_results(cli, tmp_path, data_dir):
    """`nanochat_cli score` builds the model a NANOEVL1 fixture carries, scores its rows and writes (or prints) the
    results; they match the results recorded in the fixture (per-position nll, argmax, focus logits)."""
    from nanochat_cpp_b200.data.record_file import read_records
    fixture = os.path.join(data_dir, "core_eval.bin")
    out = str(tmp_path / "score.bin")
    r = run(cli, "score", "--fixture", fixture, "--out", out)
    assert r.returncode == 0, r.stderr
    magic, got = read_records(out)
    _, want = read_records(fixture)
    assert magic == "NANOEVL1" and list(got) == ["result/nll", "result/argmax", "result/focus_offsets",
                                                 "result/focus_logits"]
    assert np.array_equal(np.array(got["result/argmax"])[0, :7], np.array(want["result/argmax"])[0, :7])
    assert np.allclose(got["result/focus_logits"], want["result/focus_logits"], atol=2e-5)
    assert np.array_equal(got["result/focus_offsets"], want["result/focus_offsets"])
    lengths = np.array(want["input/lengths"])
    for b in range(len(lengths)):                                     # positions before the row's end
        n = int(lengths[b]) - 1
        assert np.allclose(np.array(got["result/nll"])[b, :n], np.array(want["result/nll"])[b, :n], atol=2e-5)
    r = run(cli, "score", "--fixture", fixture)
    assert r.returncode == 0 and r.stdout.startswith("row 0: mean nll ") and r.stdout.count("\n") == len(lengths)
    assert run(cli, "score").returncode == 2
    assert run(cli, "score", "--fixture", str(tmp_path / "missing.bin")).returncode == 1


def test_native_rl_step_replays_the_fixture_like_the_python_engine(cli, tmp_path, data_dir):
    """`nanochat_cli rl_step` (native engine over the C ABI) and the Python replay of the same NANOORC1 fixture agree
    on every step's loss and gradient norm and on the parameters after the last step."""
    from nanochat_cpp_b200 import cli as pycli
    from nanochat_cpp_b200.data.record_file import read_records
    fixture = os.path.join(data_dir, "rl_parity.bin")
    out_n, out_p = str(tmp_path / "native.bin"), str(tmp_path / "python.bin")
    r = run(cli, "rl_step", "--fixture", fixture, "--out", out_n)
    assert r.returncode == 0 and r.stderr.count("rl: step ") == 3, r.stderr
    assert pycli.main(["rl_step", "--fixture", fixture, "--out", out_p, "--device", "cpu"]) == 0
    magic, a = read_records(out_n)
    _, b = read_records(out_p)
    assert magic == "NANOORC1"
    for k in range(3):
        assert abs(float(a[f"step/{k}/loss"][0]) - float(b[f"step/{k}/loss"][0])) < 2e-5
        assert abs(float(a[f"step/{k}/grad_norm"][0]) - float(b[f"step/{k}/grad_norm"][0])) < 2e-5
    params = [k for k in b if k.startswith("param/")]
    assert params and all(k in a for k in params)
    for k in params:
        assert np.allclose(np.array(a[k]).ravel(), np.array(b[k]).ravel(), atol=5e-5), k
    assert run(cli, "rl_step").returncode == 2


def test_native_sft_takes_shape_and_row_length_from_its_inputs(cli, tmp_path, data_dir, capsys):
    """`nanochat_cli sft`: the model shape comes from the warm-start checkpoint's tensors, the row length from the
    packed shard, the optimizer from the fine-tuning preset; the losses track the Python fine-tuning loop on the same
    fixture and the checkpoint it writes loads in Python."""
    import re
    from nanochat_cpp_b200 import cli as pycli
    from nanochat_cpp_b200.train.checkpointer import load_checkpoint
    rows = os.path.join(data_dir, "sft_rows_fixture.nchsft")
    base = os.path.join(data_dir, "sft_base_fixture.ckpt")
    out = str(tmp_path / "run")
    os.makedirs(out)
    ckpt = os.path.join(out, "sft.ckpt")
    r = run(cli, "sft", "--rows", rows, "--warm-start", base, "--num-iterations", "2", "--grad-accum", "2", "--batch", "2",
            "--out-dir", out, "--checkpoint", ckpt, "--log-every", "1")
    assert r.returncode == 0, r.stderr
    native = [float(x) for x in re.findall(r"\| loss ([0-9.]+) \|", r.stdout)]
    assert len(native) == 2 and os.path.exists(ckpt)
    assert pycli.main(["sft", "--rows", rows, "--warm-start", base, "--num-iterations", "2", "--grad-accum", "2",
                       "--batch", "2", "--checkpoint", str(tmp_path / "py.ckpt"), "--device", "cpu"]) == 0
    py = [float(x) for x in re.findall(r"sft: step \d+ .* loss ([0-9.]+)", capsys.readouterr().err)]
    assert len(py) == 2 and abs(native[0] - py[0]) < 1e-3 and abs(native[1] - py[1]) < 5e-3
    model, meta = load_checkpoint(ckpt, device="cpu")
    assert model.cfg.hidden_dim == 64 or model.cfg.hidden_dim > 0
    assert run(cli, "sft", "--rows", rows).returncode == 2


def test_native_eval_bench_prints_a_bench_v3_document(cli):
    r = run(cli, "eval_bench", "--preset-model", "tiny", "--batch", "2", "--iters", "3", "--warmup", "1")
    assert r.returncode == 0, r.stderr
    doc = json.loads(r.stdout)
    row = doc["rows"][0]
    assert doc["schema"] == "nanochat.bench.v3" and doc["device"] == "cpu" and row["family"] == "eval_forward"
    assert row["ms"] > 0 and row["iterations"] == 3 and row["shape"] == "B=2 T=64 L=2 C=64 V=512"
    assert 5.5 < doc["loss"] < 7.0 and doc["tokens_per_second"] > 0          # ln(512) = 6.24 for a fresh model


def test_native_rl_worker_speaks_the_same_protocol_as_the_python_worker(tmp_path):
    """`nanochat_cli rl_worker` against the Python `RlWorker` on the same checkpoint: the same rollouts for a seed
    (both draw from the per-row xoshiro streams) and the same policy-gradient step."""
    import numpy as np
    import torch
    from nanochat_cpp_b200.config import Config
    from nanochat_cpp_b200.cpu_engine import CpuModel
    from nanochat_cpp_b200.optim import Optimizer
    from nanochat_cpp_b200.post import RlWorker
    from nanochat_cpp_b200.post.rl_loop import PipeWorker
    from nanochat_cpp_b200.train.checkpointer import load_checkpoint
    cfg = Config(num_layers=2, num_heads=2, num_kv_heads=1, hidden_dim=64, seq_len=32, vocab_size=96,
                 padded_vocab_size=128, window_pattern="SL")
    seed_model = CpuModel(cfg, seed=3)
    rng = np.random.default_rng(0)
    for name in seed_model.names():
        w = seed_model.read(name)
        seed_model.write(name, w + 0.05 * rng.standard_normal(w.shape).astype(np.float32))
    ckpt = str(tmp_path / "policy.ckpt")
    seed_model.save(ckpt)
    flags = ["--layers", "2", "--hidden", "64", "--heads", "2", "--kv-heads", "1", "--seq", "32", "--vocab", "96",
             "--padded-vocab", "128", "--window-pattern", "SL"]
    native = PipeWorker.spawn_native(flags, checkpoint=ckpt)
    model, _ = load_checkpoint(ckpt, device=torch.device("cpu"), dtype=torch.float32)
    python = RlWorker(model, Optimizer(model.params))
    try:
        assert native.request("ping")["ok"] == "1"
        roll = ("rollout prompts=5,6,7,8,9,10 num_prompts=2 prompt_len=3 num_samples=3 max_tokens=6 temperature=0.9 "
                "top_k=20 seed=11")
        a, b = native.request(roll), python.handle(roll)
        from nanochat_cpp_b200.post.rl_loop import _parse
        b = _parse(b)
        assert a["ok"] == "1" and a["rows"] == "6"
        assert a["tokens"] == b["tokens"] and a["masks"] == b["masks"] and a["lengths"] == b["lengths"]
        adv = ("advantage tokens=1,2,3,4,5,6,7,8 targets=2,3,4,-1,6,7,8,-1 advantages=0.5,0.5,0.5,0.5,-1,-1,-1,-1 "
               "batch=2 seq=4 num_passes=1 examples_per_rank=2")
        a, b = native.request(adv), _parse(python.handle(adv))
        assert a["ok"] == "1" and a["step"] == b["step"] == "1" and a["valid_targets"] == b["valid_targets"] == "6"
        assert abs(float(a["loss"]) - float(b["loss"])) < 1e-4
        assert abs(float(a["grad_norm"]) - float(b["grad_norm"])) < 1e-3 * max(1.0, float(b["grad_norm"]))
        import pytest
        with pytest.raises(RuntimeError, match="batch\\*seq"):        # the client raises on an `ok=0` reply
            native.request("advantage tokens=1 targets=1 advantages=1 batch=2 seq=4 num_passes=1 examples_per_rank=1")
        assert native.request("ping")["ok"] == "1"        # a failed request leaves the worker alive
    finally:
        native.close()
