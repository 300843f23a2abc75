"""The native planning layer (csrc/host/plan.cc): training-run plans against the reference's recorded cases
(tests/data/plan_fixture.bin, produced by its Python planner), the operator plan against the Python planner of this
package, and the strict readers' rejections."""
import json
import os
import subprocess

import pytest

from nanochat_cpp_b200 import plan as P

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _fixture():
    raw = open(os.path.join(HERE, "data", "plan_fixture.bin"), "rb").read()
    assert raw[:8] == b"NANOPLAN"
    return json.loads(raw[12:].decode())


def _same(a, b, path=""):
    if isinstance(a, dict):
        assert set(a) == set(b), (path, set(a) ^ set(b))
        for k in a:
            _same(a[k], b[k], path + "/" + k)
    elif isinstance(a, float) or isinstance(b, float):
        assert abs(a - b) <= 1e-12 * max(1.0, abs(a)), (path, a, b)
    else:
        assert a == b, (path, a, b)


def test_training_run_plan_matches_the_recorded_cases():
    cases = _fixture()["cases"]
    assert len(cases) >= 3
    for case in cases:
        i = case["inputs"]
        got = P.compute_plan(i["depth"], vocab_size=i["vocab_size"], device_batch_size=i["device_batch_size"],
                             aspect_ratio=i["aspect_ratio"], head_dim=i["head_dim"], seq_len=i["seq_len"],
                             window_pattern=i["window_pattern"], total_batch_size=i["total_batch_size"],
                             num_iterations=i["num_iterations"], target_flops=i["target_flops"],
                             target_param_data_ratio=i["target_param_data_ratio"])
        _same(case["counts"], got["counts"], "counts")
        _same(case["plan"], got["plan"], "plan")
        assert got["flops_per_token"] == case["flops_per_token"]


def test_native_cli_prints_the_same_plan():
    exe = os.path.join(ROOT, "nanochat_cpp_b200", "nanochat_cli")
    if not os.path.exists(exe):
        pytest.skip("native CLI not built")
    case = _fixture()["cases"][0]
    i = case["inputs"]
    out = subprocess.run([exe, "train_plan", "--depth", str(i["depth"]), "--vocab", str(i["vocab_size"]), "--seq",
                          str(i["seq_len"]), "--device-batch", str(i["device_batch_size"])], capture_output=True,
                         text=True, check=True).stdout
    _same(case["plan"], json.loads(out)["plan"], "plan")


@pytest.mark.parametrize("device", ["b200", "cpu"])
@pytest.mark.parametrize("graph", ["train", "decode"])
def test_operator_plan_equals_the_python_planner(device, graph):
    caps = os.path.join(ROOT, "nanochat_cpp_b200", "caps", device + ".json")
    native = P.build_plan_native(caps_path=caps, precision="fp32" if device == "cpu" else "bf16", graph=graph)
    prof = P.device_profiles()[device]
    want = P.build_plan(P.ModelSpec.default(), prof, "fp32" if device == "cpu" else "bf16", graph)
    assert [(r.family, r.choice, r.detail) for r in native.rows] == [(r.family, r.choice, r.detail) for r in want.rows]
    assert native.model == want.model and native.device == want.device


def test_strict_readers_reject_what_they_do_not_know(tmp_path):
    spec = json.load(open(os.path.join(ROOT, "nanochat_cpp_b200", "model_specs", "nanochat-default.json")))
    caps = os.path.join(ROOT, "nanochat_cpp_b200", "caps", "b200.json")

    def plan_of(doc, caps_path=caps, precision="bf16"):
        path = tmp_path / "spec.json"
        path.write_text(json.dumps(doc))
        return P.build_plan_native(str(path), caps_path, precision)
    bad = dict(spec, surprise=1)
    with pytest.raises(P.SpecError, match="unknown keys"):
        plan_of(bad)
    bad = json.loads(json.dumps(spec))
    bad["blocks"][0]["mlp"] = "swiglu"
    with pytest.raises(P.SpecError, match="swiglu"):
        plan_of(bad)
    bad = dict(spec, requires=list(spec.get("requires", [])) + ["ring_attention"])
    with pytest.raises(P.SpecError, match="ring_attention"):
        plan_of(bad)
    with pytest.raises(P.SpecError, match="does not run"):
        plan_of(spec, os.path.join(ROOT, "nanochat_cpp_b200", "caps", "cpu.json"), "bf16")
