"""The adapters to the Hub, hub datasets, tiktoken and guarded execution: all with fakes, no network."""
import json
import os
import shutil
from pathlib import Path

import numpy as np
import pytest

from nanochat_cpp_b200.bridge import MissingExtra, extras, hub, hub_data, sft_mixture, tiktoken_tok


class FakeApi:
    """Records calls and keeps uploaded folders in a directory that FakeDownload serves."""

    def __init__(self, store: Path):
        self.store, self.calls = store, []

    def whoami(self):
        return {"name": "someone"}

    def create_repo(self, **kw):
        self.calls.append(("create_repo", kw["repo_id"]))
        (self.store / kw["repo_id"]).mkdir(parents=True, exist_ok=True)

    def upload_folder(self, *, repo_id, folder_path, path_in_repo, **kw):
        self.calls.append(("upload_folder", repo_id, path_in_repo))
        shutil.copytree(folder_path, self.store / repo_id / path_in_repo, dirs_exist_ok=True)

    def upload_file(self, *, repo_id, path_or_fileobj, path_in_repo, **kw):
        self.calls.append(("upload_file", repo_id, path_in_repo))
        dst = self.store / repo_id / path_in_repo
        dst.parent.mkdir(parents=True, exist_ok=True)
        shutil.copyfile(path_or_fileobj, dst)

    def create_tag(self, *, repo_id, tag, **kw):
        self.calls.append(("create_tag", repo_id, tag))


def fake_download(store: Path):
    def download(*, repo_id, local_dir, allow_patterns, **kw):
        src = store / repo_id
        if not src.is_dir():
            raise FileNotFoundError(repo_id)
        for pat in allow_patterns:
            if (src / pat).is_file():
                dst = Path(local_dir) / pat
                dst.parent.mkdir(parents=True, exist_ok=True)
                shutil.copyfile(src / pat, dst)
        return local_dir
    return download


def test_stage_round_trip_through_a_fake_hub(tmp_path, data_dir):
    store = tmp_path / "hub"
    client = hub.HubClient(api=FakeApi(store), download=fake_download(store), environ={})
    assert client.repo_id("d20-run") == "someone/nanochat-d20-run"
    assert hub.HubClient(api=FakeApi(store), environ={"HF_USERNAME": "me"}).repo_id("x") == "me/nanochat-x"
    rec = hub.RunRecord(stage="sft", run_name="d20-run", git_revision="abc123", step=700,
                        parent_repo_id="someone/nanochat-d20-run", parent_revision="base-v1")
    folder = hub.write_stage(tmp_path / "out" / "sft", rec, model_json={"num_layers": 2}, train_json="{}",
                             tokenizer=os.path.join(data_dir, "loader_tokenizer.nctoken"),
                             checkpoint=os.path.join(data_dir, "sft_base_fixture.ckpt"), description="a test stage")
    assert sorted(p.name for p in folder.iterdir()) == ["README.md", "checkpoint.ckpt", "model.json", "run.json",
                                                        "tokenizer.nctoken", "train.json"]
    assert "parent: `someone/nanochat-d20-run` at `base-v1`" in (folder / "README.md").read_text()
    repo = client.repo_id("d20-run")
    client.publish_stage(repo, "sft", folder, tag="sft-v1")
    assert [c[0] for c in client.api.calls] == ["create_repo", "upload_folder", "create_tag"]
    got = client.fetch_stage(repo, "sft", tmp_path / "in", files=hub.ALL_FILES)
    info = hub.read_stage(got)
    assert info["model"] == {"num_layers": 2} and info["record"].step == 700 and info["record"].container == "NCHKPT01"
    assert info["checkpoint"].read_bytes() == Path(data_dir, "sft_base_fixture.ckpt").read_bytes()
    # the fetched stage loads through the package's own loaders
    model, tok, record = hub.load_stage(got)
    assert record.stage == "sft" and tok.vocab_size > 256 and model.cfg.num_layers >= 1
    # artefacts without their magic are refused before anything is uploaded
    bad = tmp_path / "bad.nctoken"
    bad.write_bytes(b"not a tokenizer")
    with pytest.raises(ValueError):
        hub.write_stage(tmp_path / "out2", rec, model_json="{}", train_json="{}", tokenizer=bad)
    with pytest.raises(ValueError):
        client.publish_tokenizer("someone/tok", 487, bad)


def test_tokenizer_and_shard_transfers(tmp_path, data_dir):
    store = tmp_path / "hub"
    client = hub.HubClient(api=FakeApi(store), download=fake_download(store), environ={})
    tok = os.path.join(data_dir, "loader_tokenizer.nctoken")
    assert client.publish_tokenizer("someone/tok", 487, tok) == "vocab-487.nctoken"
    assert client.fetch_tokenizer("someone/tok", 487, tmp_path / "t").read_bytes() == Path(tok).read_bytes()
    assert client.fetch_tokenizer("someone/tok", 999, tmp_path / "t") is None          # absent size: train one
    assert client.fetch_tokenizer("nobody/none", 487, tmp_path / "t") is None          # absent repository
    # shards: only the missing ones are requested
    asked = []
    c2 = hub.HubClient(api=FakeApi(store), download=lambda **kw: asked.append(kw["allow_patterns"]), environ={})
    dest = tmp_path / "shards"
    dest.mkdir()
    (dest / hub.PRETRAIN_SHARDS[0]).write_bytes(b"x")
    c2.fetch_shards(dest)
    assert asked == [[hub.PRETRAIN_SHARDS[1]]]
    (dest / hub.PRETRAIN_SHARDS[1]).write_bytes(b"x")
    c2.fetch_shards(dest)
    assert len(asked) == 1


def _parquet_bytes(rows):
    import io
    import pyarrow as pa
    import pyarrow.parquet as pq
    buf = io.BytesIO()
    pq.write_table(pa.Table.from_pylist(rows), buf)
    return buf.getvalue()


def _fake_fetch(counter):
    def fetch(repo_id, subset, split):
        counter.append((repo_id, subset, split))
        if repo_id == sft_mixture.SMOLTALK_REPO:
            rows = [{"messages": [{"role": "user", "content": f"q{i}"}, {"role": "assistant", "content": f"a{i}"}]}
                    for i in range(10)]
            rows[3]["messages"].insert(0, {"role": "system", "content": "be brief"})
        elif repo_id == sft_mixture.MMLU_REPO:
            rows = [{"question": f"mm{i}", "choices": ["w", "x", "y", "z"], "answer": i % 4, "subject": "s"}
                    for i in range(6)]
        else:
            rows = [{"question": f"g{i}", "answer": f"so <<{i}+1={i + 1}>> ok\n#### {i + 1}"} for i in range(5)]
        half = len(rows) // 2
        yield "00000.parquet", _parquet_bytes(rows[:half])        # two shards: order is the concatenation
        yield "00001.parquet", _parquet_bytes(rows[half:])
    return fetch


def test_hub_dataset_cache_shuffle_and_mixture(tmp_path):
    calls = []
    cache = hub_data.DatasetCache(tmp_path / "task_data", fetch=_fake_fetch(calls))
    ds = cache.load(sft_mixture.GSM8K_REPO, "main", "train")
    assert len(ds) == 5 and ds[0]["question"] == "g0" and ds[-1]["question"] == "g4"
    assert (cache.split_dir(sft_mixture.GSM8K_REPO, "main", "train") / "manifest.json").is_file()
    cache.load(sft_mixture.GSM8K_REPO, "main", "train")
    assert len(calls) == 1                                           # second load reads the cache
    order = np.random.default_rng(42).permutation(5)                 # the order `datasets` gives for seed 42
    sh = ds.shuffle(42)
    assert [sh[i]["question"] for i in range(5)] == [f"g{int(j)}" for j in order]
    with pytest.raises(IndexError):
        ds[5]
    # mixture: 1 x SmolTalk + 3 x MMLU + 4 x GSM8K, lazy rows, deterministic
    build = sft_mixture.MixtureBuilder(hub_data.hub_loader(cache))
    mix = build("train")
    assert len(mix) == 10 + 3 * 6 + 4 * 5
    again = build("train")
    assert [mix[i]["messages"][0]["content"] for i in range(len(mix))] == \
           [again[i]["messages"][0]["content"] for i in range(len(again))]
    kinds = [m["messages"][-1]["content"] for m in (mix[i] for i in range(len(mix)))]
    assert sum(isinstance(k, list) for k in kinds) == 20             # GSM8K answers are tool-call part lists
    demo = build("demo", limit=2)
    assert len(demo) == 6
    val = build("val")
    assert len(val) == 10 + 6 + 5                                    # caps above the fake sizes
    with pytest.raises(ValueError):
        build("nope")
    # a malformed conversation is reported with its index
    bad = hub_data.DatasetCache(tmp_path / "bad", fetch=lambda *a: iter([("00000.parquet", _parquet_bytes(
        [{"messages": [{"role": "assistant", "content": "x"}, {"role": "user", "content": "y"}]}]))]))
    with pytest.raises(ValueError, match="row 0"):
        sft_mixture.SmolTalk(bad.load, "train")[0]


def test_tiktoken_encoding_matches_the_native_tokenizer(data_dir):
    pytest.importorskip("tiktoken")
    from nanochat_cpp_b200.data.native import Tokenizer
    path = os.path.join(data_dir, "loader_tokenizer.nctoken")
    art = tiktoken_tok.read_nctoken1(path)
    nat = Tokenizer.load(path)
    tt = tiktoken_tok.TiktokenTokenizer(art)
    assert tt.get_vocab_size() == nat.vocab_size and tt.get_bos_token_id() == nat.bos_id
    texts = ["Hello world, it's 12345 days!\n\n  The café's naïve façade...   x", "def f(x):\n\treturn x**2 # ok\r\n",
             "日本語のテキスト 123 ünï", "a  b   c \n d", "", "I'LL we'Ve 0001"]
    for s in texts:
        assert tt.encode(s, prepend="<|bos|>") == nat.encode(s, prepend=nat.bos_id), s
        assert tt.decode(tt.encode(s)) == s
    assert tt.encode(texts, num_threads=2) == [nat.encode(s) for s in texts]
    lengths = tt.token_byte_lengths()
    assert len(lengths) == nat.vocab_size and lengths[65] == 1 and lengths[tt.get_bos_token_id()] == 0
    assert sum(lengths[i] for i in tt.encode(texts[0])) == len(texts[0].encode())


def test_guarded_execution_and_humaneval_injection():
    run = hub_data.code_executor(timeout=3.0)
    ok = run("print(6 * 7)")
    assert ok.success and ok.stdout.strip() == "42"
    assert not run("raise SystemExit(3)").success
    slow = run("while True: pass")
    assert slow.timed_out and not slow.success
    env = run("import os; print(sorted(k for k in os.environ if k.endswith('TOKEN') or 'SECRET' in k or k.startswith('HF_')))")
    assert env.success and env.stdout.strip() == "[]"
    big = hub_data.run_program("x = bytearray(3 << 30)", memory_bytes=1 << 30)
    assert not big.success and "MemoryError" in big.stderr
    from nanochat_cpp_b200.chat.tasks import HumanEval
    rows = [{"prompt": "def add(a, b):\n", "canonical_solution": "    return a + b\n", "entry_point": "add",
             "test": "def check(f):\n    assert f(2, 3) == 5\n"}]
    seen = []

    def spy(code):
        seen.append(code)
        return run(code)
    task = HumanEval(rows, executor=spy)
    conv = task[0]
    assert task.evaluate(conv, "```python\ndef add(a, b):\n    return a + b\n```")
    assert not task.evaluate(conv, "def add(a, b):\n    return a - b")
    assert len(seen) == 2 and "check(add)" in seen[0]


def test_missing_extra_names_the_feature():
    with pytest.raises(MissingExtra) as e:
        extras.need("a_package_that_is_not_installed", "for the test")
    assert e.value.package == "a_package_that_is_not_installed" and "for the test" in str(e.value)
    assert extras.EXTRAS["pyarrow"] == "hfdata"
