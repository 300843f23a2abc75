"""The measured half of the optimisation loop, on saved measurements and a fake bench command (no GPU)."""
import json
import os
import sys

import pytest

from nanochat_cpp_b200.perf import pgo

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

HEADER = ('"ID","Process ID","Process Name","Host Name","Kernel Name","Context","Stream","Block Size","Grid Size",'
          '"Device","CC","Section Name","Metric Name","Metric Unit","Metric Value"')


def _row(i, kernel, ns, unit="ns"):
    return (f'"{i}","529","python3.12","127.0.0.1","{kernel}","1","7","(320, 1, 1)","(8, 10, 32)","0","10.0",'
            f'"Command line profiler metrics","gpu__time_duration.sum","{unit}","{ns}"')


def _launch_list(path):
    rows = ["==PROF== Connected to process 529 (/usr/bin/python3.12)", HEADER]
    kernels = [("void nc::unnamed>::gemm_pair_kernel<1, 2>(CUtensorMap_st, nc::GemmArgs)", 30_000_000),
               ("void unnamed>::attention_bwd_kernel<128, 1>(CUtensorMap_st, BwdParams)", 10_000_000),
               ("void unnamed>::attention_fwd2_kernel<128>(CUtensorMap_st)", 4_000_000),
               ("nc::classifier_smem_kernel<false>(__nv_bfloat16*, long long)", "2,000,000"),
               ("nc::rmsnorm_bwd_kernel(float*)", 1_000_000),
               ("nc::adamw_kernel(float*)", 500_000), ("something_else(int)", 500_000)]
    for step in range(2):                       # the list covers two steps
        for k, (name, ns) in enumerate(kernels):
            rows.append(_row(step * 10 + k, name, ns))
    rows.append(_row(99, "nc::sumsq_kernel(float const*)", 2, unit="ms"))
    path.write_text("\n".join(rows) + "\n")


def _fake_bench(values):
    it = iter(values)
    return lambda cmd: "warm-up noise\n" + json.dumps({"metric": "tok/s", "value": 1.0, "unit": "tok/s",
                                                        "ms_per_step": next(it), "clocks": {"reasons": ["sw_power_cap"]}})


def test_families():
    assert pgo.family_of("void nc::gemm_pair_kernel<1>(...)") == "gemm"
    assert pgo.family_of("attention_bwd_kernel<128, 1>") == "attention_bwd"
    assert pgo.family_of("nc::grad_push_kernel") == "comm"
    assert pgo.family_of("ncclDevKernel_AllReduce_Sum_f32") == "comm"
    assert pgo.family_of("linear_dgrad_relu2_act") == "gemm"
    assert pgo.family_of("muon_update") == "optimizer"
    assert pgo.family_of("paged_decode_kernel") == "decode"
    assert pgo.family_of("mystery") == "other"
    assert pgo.short_kernel_name("void nc::unnamed>::gemm_pair_kernel<1, 2>(CUtensorMap_st, nc::GemmArgs)") == "gemm_pair_kernel"


def test_one_iteration_of_the_loop(tmp_path):
    t = pgo.init(tmp_path, "d20-base", "python bench.py --steps 8 --warmup 3", runs=3)
    before = pgo.measure(t, "before", runner=_fake_bench([100.0, 101.0, 100.5]))
    assert before["median_ms"] == 100.5 and abs(before["spread_rel"] - 1.0 / 100.5) < 1e-12
    csv_path = tmp_path / "launches.csv"
    _launch_list(csv_path)
    rows = pgo.read_launch_list(csv_path)
    assert len(rows) == 15 and rows[3]["ns"] == 2_000_000 and rows[-1]["ns"] == 2_000_000      # thousands separators, units
    pgo.trace(t, launches=csv_path, steps=2)
    a = pgo.analyze(t)
    sig = {s["id"]: s for s in a["signatures"]}
    assert abs(sig["launches:gemm"]["ms"] - 30.0) < 1e-9 and abs(sig["launches:gemm"]["share"] - 30.0 / 100.5) < 1e-9
    assert abs(sig["launches:optimizer"]["ms"] - 1.5) < 1e-9                       # adamw per step + sumsq / 2 steps
    assert abs(sig["launches:idle"]["ms"] - (100.5 - 49.0)) < 1e-6                 # the launch-bound share
    assert a["candidates"] == ["launches:idle", "launches:gemm"]
    assert sig["launches:gemm"]["top_kernels"][0][0] == "gemm_pair_kernel"
    # an idea against attention backward (ceiling 10 / 100.5): a 6 % gain is accepted, a 30 % gain is flagged
    t.write([{"id": "dkv-pairs", "signature": "launches:attention_bwd", "text": "share B operands across a CTA pair"}],
            t.iter_dir(), "ideas.json")
    pgo.measure(t, "after", runner=_fake_bench([94.0, 94.5, 94.2]))
    v = pgo.compare(t, idea="dkv-pairs")
    assert v["verdict"] == "improved" and v["flags"] == [] and abs(v["gain"] - (1 - 94.2 / 100.5)) < 1e-12
    pgo.measure(t, "after", runner=_fake_bench([70.0, 70.0, 70.0]))
    v = pgo.compare(t, idea="dkv-pairs")
    assert v["verdict"] == "improved" and "exceeds the ceiling" in v["flags"][0]
    # within noise: no change; slower: regressed
    pgo.measure(t, "after", runner=_fake_bench([100.0, 100.2, 100.4]))
    assert pgo.compare(t)["verdict"] == "no change"
    pgo.measure(t, "after", runner=_fake_bench([104.0, 104.2, 104.4]))
    assert pgo.compare(t)["verdict"] == "regressed"
    # apply an improvement: the loop advances and the new baseline is carried over
    pgo.measure(t, "after", runner=_fake_bench([94.0, 94.5, 94.2]))
    pgo.compare(t, idea="dkv-pairs", apply=True)
    assert t.loop["iteration"] == 2 and t.loop["history"][0]["verdict"] == "improved"
    assert t.read("iter-02", "before.json")["median_ms"] == 94.2
    text = pgo.report(t)
    assert "| 1 | dkv-pairs | 100.50 | 94.20 |" in text and "## Iteration 2" in text
    assert (tmp_path / "d20-base" / "RESULT.md").read_text() == text


def test_one_step_is_cut_out_of_a_longer_launch_list(tmp_path):
    rows = ["==PROF== banner", HEADER]
    seq = ["warm_kernel(int)"] * 3
    for step in range(3):
        seq += ["nc::finish_norm_kernel(double const*)", "nc::adamw_kernel(float*)", "void nc::gemm_pair_kernel<1>(int)",
                "nc::sumsq_kernel(float const*)"]
    for i, k in enumerate(seq):
        rows.append(_row(i, k, 1000 * (i + 1)))
    src = tmp_path / "long.csv"
    src.write_text("\n".join(rows) + "\n")
    assert pgo.cut_one_period(src, "finish_norm", tmp_path / "one.csv") == 4
    kept = pgo.read_launch_list(tmp_path / "one.csv")
    assert [pgo.short_kernel_name(r["kernel"]) for r in kept] == ["adamw_kernel", "gemm_pair_kernel", "sumsq_kernel",
                                                                   "finish_norm_kernel"]
    assert kept[0]["ns"] == 1000 * (3 + 4 + 1 + 1)          # the second step's first kernel after the marker
    t = pgo.init(tmp_path, "cut", "cmd")
    rec = pgo.trace(t, launches=src, between="finish_norm")
    assert rec["steps_in_launch_list"] == 1 and len(pgo.read_launch_list(t.path("iter-01", "trace", "launches.csv"))) == 4
    with pytest.raises(ValueError, match="fewer than two"):
        pgo.cut_one_period(src, "no_such_kernel", tmp_path / "x.csv")


def test_throttled_runs_and_missing_lines_are_rejected(tmp_path):
    t = pgo.init(tmp_path, "x", "cmd", runs=1)
    with pytest.raises(SystemExit, match="no JSON line"):
        pgo.measure(t, "before", runner=lambda cmd: "nothing here\n")
    hot = json.dumps({"ms_per_step": 10.0, "clocks": {"reasons": ["sw_power_cap", "hw_thermal_slowdown"]}})
    with pytest.raises(SystemExit, match="throttled"):
        pgo.measure(t, "before", runner=lambda cmd: hot)
    with pytest.raises(SystemExit, match="needs both"):
        pgo.compare(t)


def test_operator_table_of_the_committed_step_profile(tmp_path):
    path = os.path.join(ROOT, "profiles", "step_profile_d20_batch32.txt")
    tab = pgo.read_operator_table(path)
    head = next(l for l in open(path) if "fwd+bwd" in l and "optimizer" in l)
    nums = [float(x) for x in __import__("re").findall(r"([0-9]+\.[0-9]+) ms", head)]
    assert abs(tab["step_ms"] - (nums[0] + nums[1])) < 1e-6 and 200 < tab["step_ms"] < 300
    assert tab["operators"]["attention_bwd"]["calls"] == 20
    t = pgo.init(tmp_path, "d20", "cmd")
    pgo.trace(t, operators=path)
    a = pgo.analyze(t)
    sig = {s["id"]: s for s in a["signatures"]}
    gemm = sum(tab["operators"][k]["ms"] for k in ("linear_wgrad", "linear_fwd", "linear_dgrad", "linear_dgrad_relu2_act",
                                                   "linear_relu2_act_fwd"))
    assert abs(sig["operators:gemm"]["ms"] - gemm) < 1e-3
    assert a["candidates"] == ["operators:gemm", "operators:attention_bwd"]
    assert 0.14 < sig["operators:attention_bwd"]["ceiling"] < 0.17


def test_command_line_end_to_end(tmp_path):
    fake = tmp_path / "fake_bench.py"
    fake.write_text("import json; print(json.dumps({'ms_per_step': 50.0, 'metric': 'm', 'value': 2.0, 'unit': 'u'}))\n")
    root = str(tmp_path / "targets")
    assert pgo.main(["init", "--root", root, "--name", "t", "--measure-cmd", f"{sys.executable} {fake}", "--runs", "2"]) == 0
    assert pgo.main(["measure", "--root", root, "--name", "t", "--before"]) == 0
    assert pgo.main(["measure", "--root", root, "--name", "t", "--after"]) == 0
    assert pgo.main(["compare", "--root", root, "--name", "t"]) == 0
    assert json.loads((tmp_path / "targets" / "t" / "iter-01" / "verdict.json").read_text())["verdict"] == "no change"
    assert pgo.main(["report", "--root", root, "--name", "t"]) == 0
