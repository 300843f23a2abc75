"""MeshRuntime on CPU replicas (gloo): two replicas take the same steps as one."""
import numpy as np

from nanochat_cpp_b200.config import Config
from nanochat_cpp_b200.optim import OptimizerConfig
from nanochat_cpp_b200.runtime import MeshRuntime, fnv1a64
from nanochat_cpp_b200.train.loop import TrainConfig


def test_fnv():
    assert fnv1a64(b"") == 0xCBF29CE484222325 and fnv1a64(b"a") == 0xAF63DC4C8601EC8C


def test_two_replicas_match_one(tmp_path):
    cfg = Config(num_layers=2, num_heads=2, num_kv_heads=2, hidden_dim=64, seq_len=16, vocab_size=128,
                 padded_vocab_size=128)
    rng = np.random.default_rng(0)
    batches = [(rng.integers(0, 128, (4, 16)), rng.integers(0, 128, (4, 16))) for _ in range(3)]

    def run(devices):
        tc = TrainConfig(batch=4 // len(devices), num_iterations=3, dtype="fp32", optim=OptimizerConfig(adam_eps=1e-4))
        with MeshRuntime(cfg, devices, tc) as rt:
            losses = [rt.train_step(t, g) for t, g in batches]
            path = str(tmp_path / f"m{len(devices)}.ckpt")
            rt.save(path)
            m = rt.metrics()
            return losses, rt.param("lm_head.weight"), rt.digest(), m, path

    l1, p1, d1, m1, path1 = run(["cpu"])
    l2, p2, d2, m2, _ = run(["cpu", "cpu"])
    assert m1["step"] == m2["step"] == 3 and m2["world_size"] == 2
    assert np.allclose(l1, l2, atol=1e-5) and np.allclose(p1, p2, atol=1e-4)
    with MeshRuntime(cfg, ["cpu"], TrainConfig(batch=4, num_iterations=3, dtype="fp32")) as rt:
        assert rt.load(path1) == 3 and rt.digest() == d1


def test_bench_report_document_and_roofline_join(tmp_path):
    """`nanochat.bench.v3`: key order of a row, optional keys left out when unset, MFU against the stated peak,
    and the (family, phase) join with roofline rows."""
    import json
    from nanochat_cpp_b200.bench.report import SCHEMA, BenchReport, join_with_roofline
    rep = BenchReport(device="NVIDIA B200", precision="bf16", peak_flops=1.0e15)
    rep.set_row_identity("linear", "fwd")
    rep.add("gemm:fc.fwd", "M=65536 N=5120 K=1280", 0.57, 1.5e6, iterations=10)
    rep.add("misc", "n/a", 1.0, family="", phase="")
    rep.extras["preset"] = "d20"
    doc = json.loads(rep.json())
    assert doc["schema"] == SCHEMA == "nanochat.bench.v3" and list(doc)[:4] == ["schema", "device", "precision", "peak_flops"]
    r0, r1 = doc["rows"]
    assert list(r0) == ["name", "family", "phase", "precision", "shape", "ms", "gflops", "work_ratio", "mfu", "iterations"]
    assert abs(r0["mfu"] - 1.5) > 0 and r0["mfu"] == 1.0          # 1.5e15 / 1e15, clamped to 1
    assert "family" not in r1 and "iterations" not in r1 and r1["mfu"] == 0.0 and doc["preset"] == "d20"
    path = tmp_path / "bench.json"
    rep.write(str(path))
    assert json.loads(path.read_text()) == doc
    roof = {"schema": "nanochat.roofline.v3", "rows": [{"family": "linear", "phase": "fwd", "bound_ms": 0.38}]}
    joined = join_with_roofline(doc, roof)
    assert len(joined) == 1 and abs(joined[0]["attainment"] - 0.38 / 0.57) < 1e-12
    assert "gemm:fc.fwd" in rep.table()
