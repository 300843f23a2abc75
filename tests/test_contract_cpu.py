"""The per-record tolerance contract: both CPU engines conform, and the runner catches what it should."""
import json
import os

import numpy as np
import pytest

from nanochat_cpp_b200 import contract as K
from nanochat_cpp_b200.data.record_file import read_records


@pytest.mark.parametrize("engine", ["python", "native"])
@pytest.mark.parametrize("file", sorted(K.PRODUCERS))
def test_engine_conforms(file, engine, data_dir):
    assert K.run_fixture(file, engine, data_dir=data_dir) == []


def test_every_record_resolves_and_first_match_wins(data_dir):
    contracts = K.load_tolerances()
    for file, c in contracts.items():
        _, recs = read_records(os.path.join(data_dir, file))
        assert c.uncovered(recs) == [] and len(recs) == c.record_count
        assert c.verify_file(os.path.join(data_dir, file)) == []
    c = contracts["debug_state.bin"]
    assert c.bound_for("step/2/param/backout_lambda").atol == 2e-4          # the specific rule sits before the general one
    assert c.bound_for("step/2/param/lm_head.weight").atol == 1e-4
    assert c.bound_for("step/0/param/lm_head.weight").mode == "exact"
    assert c.bound_for("something/else") is None


def test_violations_are_reported_with_record_and_element(data_dir, tmp_path):
    c = K.load_tolerances()["debug_state.bin"]
    _, recs = read_records(os.path.join(data_dir, "debug_state.bin"))
    produced = K.produce_debug_state(K.ENGINES["native"], recs)
    skip = set(K.OPTIONAL["native"])
    wanted = {k: v for k, v in recs.items() if k not in skip}
    assert c.check(produced, wanted) == []
    # one element of one gradient off by 3e-5 (bound 1e-5)
    name = "grad/lm_head.weight"
    broken = dict(produced)
    broken[name] = produced[name].copy()
    broken[name].reshape(-1)[7] += 3e-5
    bad = c.check(broken, wanted)
    assert len(bad) == 1 and bad[0].startswith(name) and " at 7 " in bad[0]
    # a record that is not produced, a record without a bound
    del broken[name]
    assert any(b == f"{name}: not produced" for b in c.check(broken, wanted))
    assert any("no bound" in b for b in c.check(produced, dict(wanted, **{"extra/record": np.zeros(1)})))
    # a changed file is noticed
    path = tmp_path / "debug_state.bin"
    data = bytearray(open(os.path.join(data_dir, "debug_state.bin"), "rb").read())
    data[-1] ^= 1
    path.write_bytes(bytes(data))
    assert "sha256" in c.verify_file(str(path))[0]


def test_bound_modes():
    assert K.Bound("exact").violation([1, 2, 3], [1, 2, 3]) is None
    assert "differs at 1" in K.Bound("exact").violation([1, 5, 3], [1, 2, 3])
    assert K.Bound("absolute", atol=1e-3, rtol=1e-2).violation([100.9], [100.0]) is None
    assert K.Bound("absolute", atol=1e-3, rtol=1e-2).violation([101.1], [100.0]) is not None
    assert K.Bound("norm", rtol=1e-3).violation([3.0, 4.0], [4.0, 3.0]) is None          # same norm, other elements
    assert K.Bound("norm", rtol=1e-3).violation([3.0, 4.1], [4.0, 3.0]) is not None
    assert K.Bound("absolute", atol=1.0).violation([float("nan")], [0.0]) == "non-finite values"
    assert K.Bound("input").violation([1], [2]) is None
    assert "size" in K.Bound("exact").violation([1, 2], [1, 2, 3])
