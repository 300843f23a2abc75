"""Native host runtime (C++) against the reference's own fixtures: tokenizer (rustbpe/tiktoken parity), loader
(upstream best-fit packing), checkpoint container v0/v1, plus round trips of what has no fixture."""
import os
import struct

import numpy as np
import pytest

from nanochat_cpp_b200.data import native
from nanochat_cpp_b200.data.record_file import read_records


def _strings(recs, prefix, offs_name, data_name):
    offs = recs[prefix + offs_name]
    data = bytes(recs[prefix + data_name])
    return [data[int(offs[i]):int(offs[i + 1])] for i in range(len(offs) - 1)]


def _fixture_tokenizer(recs, tmp_path):
    """Builds an NCTOKEN1 file from the fixture's merge table with our own writer, then loads it natively."""
    left, right = recs["merges/left"], recs["merges/right"]
    names = _strings(recs, "special/", "names_offsets", "names")
    ids = recs["special/ids"]
    pattern = bytes(recs["config/pattern"])
    path = str(tmp_path / "fixture.nctoken")
    with open(path, "wb") as f:
        f.write(b"NCTOKEN1" + struct.pack("<I", 1) + struct.pack("<I", len(pattern)) + pattern)
        f.write(struct.pack("<I", len(left)))
        for a, b in zip(left, right):
            f.write(struct.pack("<II", int(a), int(b)))
        f.write(struct.pack("<I", len(names)))
        for n, i in zip(names, ids):
            f.write(struct.pack("<I", len(n)) + n + struct.pack("<I", int(i)))
    return native.Tokenizer.load(path)


def test_tokenizer_fixture(data_dir, tmp_path):
    _, recs = read_records(os.path.join(data_dir, "tokenizer_fixture.bin"))
    tok = _fixture_tokenizer(recs, tmp_path)
    assert tok.vocab_size == int(recs["config/vocab_size"][0])
    # split pattern
    strings = _strings(recs, "split/", "strings_offsets", "strings")
    sp_off = recs["split/string_piece_offsets"]
    piece_off = recs["split/piece_offsets"]
    pieces_blob = bytes(recs["split/pieces"])
    for i, s in enumerate(strings):
        want = [pieces_blob[int(piece_off[k]):int(piece_off[k + 1])] for k in range(int(sp_off[i]), int(sp_off[i + 1]))]
        assert native.split_pattern(s) == want, (s, native.split_pattern(s), want)
    # encode
    inputs = _strings(recs, "encode/", "input_offsets", "inputs")
    id_off, ids = recs["encode/id_offsets"], recs["encode/ids"]
    for i, s in enumerate(inputs):
        want = ids[int(id_off[i]):int(id_off[i + 1])].tolist()
        got = tok.encode(s, int(recs["encode/prepend"][i]), int(recs["encode/append"][i]))
        assert got == want, (s, got, want)
    # decode (lossy UTF-8)
    d_off, d_ids = recs["decode/id_offsets"], recs["decode/ids"]
    outs = _strings(recs, "decode/", "output_offsets", "outputs")
    for i, want in enumerate(outs):
        assert tok.decode_bytes(d_ids[int(d_off[i]):int(d_off[i + 1])].tolist()) == want
    # save / load round trip
    path = str(tmp_path / "again.nctoken")
    tok.save(path)
    again = native.Tokenizer.load(path)
    assert again.encode("Hello, world! 12345") == tok.encode("Hello, world! 12345")


def test_reference_tokenizer_file_loads(data_dir):
    tok = native.Tokenizer.load(os.path.join(data_dir, "loader_tokenizer.nctoken"))
    assert 256 < tok.vocab_size <= 512 and tok.bos_id >= 256
    text = "The quick brown fox jumps over the lazy dog. [7]"
    assert tok.decode(tok.encode(text)) == text


def test_loader_parity(data_dir):
    blob = open(os.path.join(data_dir, "loader_parity.bin"), "rb").read()
    assert blob[:8] == b"NCLDRP01"
    ver, batch, seq, buffer, source_batch, doc_count = struct.unpack_from("<6I", blob, 8)
    off = 32
    docs = []
    for _ in range(doc_count):
        (n,) = struct.unpack_from("<I", blob, off)
        docs.append(blob[off + 4:off + 4 + n])
        off += 4 + n
    (steps,) = struct.unpack_from("<I", blob, off)
    off += 4
    tok = native.Tokenizer.load(os.path.join(data_dir, "loader_tokenizer.nctoken"))
    token_docs = [tok.encode(d, prepend=tok.bos_id) for d in docs]
    loader = native.DataLoader.from_documents(token_docs, batch, seq, buffer_docs=buffer, source_batch=source_batch)
    for _ in range(steps):
        want_tok = np.frombuffer(blob, dtype="<i4", count=batch * seq, offset=off).reshape(batch, seq)
        off += 4 * batch * seq
        want_tgt = np.frombuffer(blob, dtype="<i4", count=batch * seq, offset=off).reshape(batch, seq)
        off += 4 * batch * seq
        got_tok, got_tgt = loader.next()
        assert np.array_equal(got_tok, want_tok)
        assert np.array_equal(got_tgt, want_tgt)


def test_loader_cursor_and_sharding(tmp_path):
    docs = [[1000 + i] + list(range(i % 7 + 2)) for i in range(50)]
    a = native.DataLoader.from_documents(docs, 2, 8, buffer_docs=4)
    for _ in range(3):
        a.next()
    cur = str(tmp_path / "cursor")
    a.save_cursor(cur)
    want = [a.next() for _ in range(3)]
    b = native.DataLoader.from_documents(docs, 2, 8, buffer_docs=4)
    b.load_cursor(cur)
    got = [b.next() for _ in range(3)]
    for (t0, g0), (t1, g1) in zip(want, got):
        assert np.array_equal(t0, t1) and np.array_equal(g0, g1)
    r0 = native.DataLoader.from_documents(docs, 1, 64, buffer_docs=1, rank=0, world=2)
    r1 = native.DataLoader.from_documents(docs, 1, 64, buffer_docs=1, rank=1, world=2)
    firsts0 = {int(x) for x in r0.next()[0].ravel() if x >= 1000}
    firsts1 = {int(x) for x in r1.next()[0].ravel() if x >= 1000}
    assert all(v % 2 == 0 for v in firsts0) and all(v % 2 == 1 for v in firsts1)


def test_checkpoint_v0_and_v1(data_dir, tmp_path):
    recs, opt, meta = native.read_checkpoint(os.path.join(data_dir, "checkpoint_v0.ckpt"))
    assert list(recs) == ["fixture/weights", "fixture/bias"]
    assert recs["fixture/weights"][0] == 0 and recs["fixture/weights"][1].shape == (2, 3)
    assert recs["fixture/bias"][0] == 1 and recs["fixture/bias"][1].shape == (3,)

    def fnv(b):
        h = 0xcbf29ce484222325
        for x in b:
            h = ((h ^ x) * 0x100000001b3) & 0xFFFFFFFFFFFFFFFF
        return h
    assert fnv(recs["fixture/weights"][1].tobytes()) == 0x7610708711193cf0
    assert fnv(recs["fixture/bias"][1].tobytes()) == 0x702bf156049a2035
    assert meta["config"]["container_version"] == 0
    # a version 1 file written by the reference
    recs1, opt1, meta1 = native.read_checkpoint(os.path.join(data_dir, "sft_base_fixture.ckpt"))
    assert meta1["config"]["container_version"] == 1 and meta1["config"]["num_layers"] > 0
    assert "lm_head.weight" in recs1
    # our writer -> our reader, metadata included
    cfg = dict(num_layers=2, num_heads=4, num_kv_heads=2, hidden_dim=64, seq_len=32, vocab_size=96,
               padded_vocab_size=128, rope_base=10000.0, window_pattern="SL", value_embedding=True)
    path = str(tmp_path / "x.ckpt")
    w = np.arange(12, dtype=np.float32).reshape(3, 4)
    native.write_checkpoint(path, [("a.weight", 0, w)], [("optimizer/step", 0, np.array([7.0], np.float32))],
                            config=cfg, stage=1, step=42, world_size=8, precision=1, tokenizer_id="tok", notes="hello")
    r, o, m = native.read_checkpoint(path)
    assert np.array_equal(r["a.weight"][1], w) and float(o["optimizer/step"][1][0]) == 7.0
    assert m["stage"] == 1 and m["step"] == 42 and m["world_size"] == 8 and m["precision"] == 1
    assert m["tokenizer_id"] == "tok" and m["notes"] == ["hello"]
    assert {k: m["config"][k] for k in ("num_layers", "hidden_dim", "window_pattern")} == \
        {"num_layers": 2, "hidden_dim": 64, "window_pattern": "SL"}


def test_bpe_trainer_and_parquet(tmp_path):
    pa = pytest.importorskip("pyarrow")
    import pyarrow.parquet as pq
    docs = [f"the quick brown fox {i} jumps over the lazy dog, again and again and again" for i in range(200)]
    docs[5] = None
    for codec in ("NONE", "ZSTD"):
        path = str(tmp_path / f"d_{codec}.parquet")
        pq.write_table(pa.table({"text": docs, "n": list(range(200))}), path, compression=codec,
                       use_dictionary=False, data_page_version="1.0", row_group_size=64)
        rows = native.read_parquet_strings(path, "text")
        assert [r.decode() for r in rows] == [d for d in docs if d is not None]
    text = str(tmp_path / "corpus.txt")
    with open(text, "w") as f:
        f.write("\n".join(d for d in docs if d))
    tok = native.Tokenizer.train(text=text, vocab_size=300)
    assert tok.vocab_size == 300 and tok.bos_id == 300 - 9
    ids = tok.encode("the quick brown fox")
    assert len(ids) < len("the quick brown fox") and tok.decode(ids) == "the quick brown fox"
    tok2 = native.Tokenizer.train(parquet=path, text_column="text", vocab_size=300)
    assert tok2.vocab_size == 300


def test_sampler():
    logits = np.array([0.1, 5.0, 0.2, 4.9], dtype=np.float32)
    assert native.sample_token(logits, 0.0, 0, 1) == 1
    draws = {native.sample_token(logits, 1.0, 2, 7, row=r) for r in range(64)}
    assert draws <= {1, 3} and len(draws) == 2
    assert native.sample_token(logits, 1.0, 2, 7, row=3, step=2) == native.sample_token(logits, 1.0, 2, 7, row=3, step=2)


def test_fp8_host_codecs_match_torch():
    import torch
    from nanochat_cpp_b200.data.native import fp8_decode, fp8_encode
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(5000).astype(np.float32) * s for s in (1e-3, 0.1, 1, 30, 500, 1e5)] +
                       [np.array([0.0, -0.0, 448, 449, -1e9, 2 ** -9, 2 ** -10, 3 * 2 ** -10], dtype=np.float32)])
    for fmt, dt, mx in (("e4m3", torch.float8_e4m3fn, 448.0), ("e5m2", torch.float8_e5m2, 57344.0)):
        codes = fp8_encode(x, fmt)
        want = torch.from_numpy(np.clip(x, -mx, mx)).to(dt).float().numpy()
        assert np.array_equal(fp8_decode(codes, fmt), want)


def test_spec_profile_and_plan():
    import pytest
    from nanochat_cpp_b200.plan import ModelSpec, SpecError, build_plan, device_profiles, profile_for
    spec = ModelSpec.default()
    cfg = spec.to_config()
    assert (cfg.num_layers, cfg.hidden_dim, cfg.window_pattern, cfg.value_embedding) == (12, 768, "SSSL", True)
    assert [cfg.window_left(i) >= 0 for i in range(12)] == [b["attention"] == "sliding_window" for b in spec.blocks]
    profs = device_profiles()
    assert profile_for("NVIDIA B200").device == "b200" and profile_for("Xeon").device == "cpu"
    plan = build_plan(spec, profs["b200"])
    assert all(r.choice == "kernel" for r in plan.rows) and "fused families" in plan.line()
    cpu_plan = build_plan(spec, profs["cpu"], precision="fp32")
    assert all(r.choice == "composition" for r in cpu_plan.rows)
    assert {r.family for r in build_plan(spec, profs["b200"], graph="decode").rows} >= {"decode_attention"}
    with pytest.raises(SpecError):
        build_plan(spec, profs["cpu"], precision="bf16")
    bad = dict(spec_version=1, name="x", dimensions=dict(num_heads=2, hidden_dim=64), blocks=[dict(norm="layer_norm")])
    with pytest.raises(SpecError, match="layer_norm"):
        ModelSpec.from_json(bad)
    with pytest.raises(SpecError, match="unknown spec keys"):
        ModelSpec.from_json(dict(bad, colour="red"))
