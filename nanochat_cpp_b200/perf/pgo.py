#!/usr/bin/env python3
"""The measured half of a profile-guided optimisation loop: measure, trace, analyse, compare, record.

    pgo init    --root DIR --name TARGET --measure-cmd "python bench.py --steps 8 --warmup 3" \\
                [--trace-cmd "..."] [--runs 2] [--stage base] [--device b200]
    pgo measure --root DIR --name TARGET --before | --after
    pgo trace   --root DIR --name TARGET            # runs the trace command, or: --launches FILE [--between KERNEL] / --operators FILE
    pgo analyze --root DIR --name TARGET
    pgo compare --root DIR --name TARGET [--idea ID] [--apply]
    pgo report  --root DIR --name TARGET

Optimising a training step has a part that needs judgement (which idea the profile supports, how to write it) and a
part that must be exact: the step time before and after, the share of the step each cost owns, whether a change was
a gain beyond the run-to-run noise. This module is the exact part; it only reads files and runs the commands the
target names, with the standard library, so it works on a machine without a GPU on saved measurements.

  measure   runs the target's command `runs` times; each run must print one JSON line with `ms_per_step` (the
            contract of the repository's `bench.py`). Stores every sample, the median and the spread.
  trace     two kinds of evidence, either or both: a *launch list* (the CSV that
            `ncu --metrics gpu__time_duration.sum --csv` writes: one row per kernel launch with its device time) and
            an *operator table* (the text `bench/step_profile.py` writes: operator, milliseconds, calls).
  analyze   groups kernels into families (GEMM, attention forward / backward, classifier, row kernels, optimizer,
            communication, decode, other) and writes one *signature* per family: its device time, its share of the
            step, and its *ceiling*: the most the step could gain if that cost vanished (Amdahl's bound). Device
            idle time (step time minus kernel time, when the launch list covers whole steps) is a signature too:
            the launch-bound share. The two largest ceilings are the candidates.
  compare   after ÷ before with the noise of both; verdict `improved`, `regressed` or `no change` (threshold: the
            larger of 1 % and twice the relative spread). A gain larger than the ceiling of the signature the idea
            named is flagged: the measurement, not the idea, is then suspect. `--apply` closes the iteration: the
            after-measurement becomes the next baseline.
  report    RESULT.md: the state of the target from the files alone.

Where the reference's loop (python/nanochat_cpp/pgo.py) reads Nsight Systems CSVs from a cloud run, this one reads
Nsight Compute launch lists and CUDA-event operator tables, which are what this package's benches produce.
"""
from __future__ import annotations

import argparse
import csv
import datetime
import json
import os
import re
import shlex
import statistics
import subprocess
import sys
from pathlib import Path
from typing import Dict, List, Optional

# kernel / operator name -> family, first match wins
FAMILIES = (
    ("comm", r"grad_push|grad_reduce|reduce_pull|adamw_push|muon_apply_push|ncclDevKernel|nccl|all_?gather|reduce_?scatter"),
    ("attention_bwd", r"attention_bwd|attention_dq|attn_delta|attention_delta"),
    ("attention_fwd", r"attention_fwd|attention_fwd2"),
    ("decode", r"paged_decode|decode_prep|kv_append|gemm_skinny|decode_"),
    ("classifier", r"classifier"),
    ("gemm", r"gemm_|linear_|cutlass|cublas|sgemm|gemv|fp8_mx|mxfp8"),
    ("optimizer", r"adamw|muon|newton|sumsq|grad_norm|clip|polar"),
    ("rows", r"rmsnorm|norm_blend|blend|qk_prep|value_gate|smear|backout|embedding|relu|add_cols|rope|flat_kernel|\badd\b"),
    ("framework", r"at::native|vectorized_elementwise|elementwise_kernel|CatArray|copy_kernel|launch_clamp|where_kernel|"
                  r"reduce_kernel|fill|index_"),
)


def family_of(name: str) -> str:
    for fam, pat in FAMILIES:
        if re.search(pat, name, re.I):
            return fam
    return "other"


def now() -> str:
    return datetime.datetime.now(datetime.timezone.utc).isoformat(timespec="seconds")


# ------------------------------------------------------------------------------------------------ state
class Target:
    def __init__(self, root, name: str):
        self.dir = Path(root) / name
        self.name = name

    def path(self, *parts) -> Path:
        return self.dir.joinpath(*parts)

    def read(self, *parts, default=None):
        try:
            return json.loads(self.path(*parts).read_text())
        except (OSError, ValueError):
            return default

    def write(self, obj, *parts) -> None:
        p = self.path(*parts)
        p.parent.mkdir(parents=True, exist_ok=True)
        tmp = p.with_suffix(p.suffix + ".tmp")
        tmp.write_text(json.dumps(obj, indent=1, sort_keys=True) + "\n")
        os.replace(tmp, p)

    @property
    def spec(self) -> dict:
        s = self.read("target.json")
        if s is None:
            raise SystemExit(f"no target '{self.name}' under {self.dir.parent} (run `pgo init` first)")
        return s

    @property
    def loop(self) -> dict:
        return self.read("loop.json", default={"iteration": 1, "history": []})

    def iter_dir(self, k: Optional[int] = None) -> str:
        return f"iter-{(k or self.loop['iteration']):02d}"


def init(root, name, measure_cmd, trace_cmd="", runs=2, stage="base", device="b200") -> Target:
    t = Target(root, name)
    t.write({"name": name, "stage": stage, "device": device, "measure_cmd": measure_cmd, "trace_cmd": trace_cmd,
             "runs": int(runs), "created_utc": now()}, "target.json")
    if t.read("loop.json") is None:
        t.write({"iteration": 1, "history": []}, "loop.json")
    return t


# ------------------------------------------------------------------------------------------------ measure
def parse_bench_line(text: str) -> Optional[dict]:
    """The last line of `text` that is a JSON object with `ms_per_step`."""
    for line in reversed(text.splitlines()):
        line = line.strip()
        if line.startswith("{") and "ms_per_step" in line:
            try:
                obj = json.loads(line)
            except ValueError:
                continue
            if isinstance(obj.get("ms_per_step"), (int, float)):
                return obj
    return None


def summarize(samples: List[float]) -> dict:
    med = statistics.median(samples)
    return {"samples_ms": samples, "median_ms": med, "spread_rel": (max(samples) - min(samples)) / med if med else 0.0}


def measure(t: Target, which: str, runner=None) -> dict:
    """`runner(cmd) -> stdout text`; the default runs the command in a shell-free subprocess."""
    spec = t.spec
    runner = runner or (lambda cmd: subprocess.run(shlex.split(cmd), capture_output=True, text=True, check=True).stdout)
    samples, last = [], None
    for _ in range(spec["runs"]):
        obj = parse_bench_line(runner(spec["measure_cmd"]))
        if obj is None:
            raise SystemExit("the measure command printed no JSON line with ms_per_step")
        clocks = obj.get("clocks") or {}
        bad = [r for r in clocks.get("reasons", []) if "thermal" in r or r == "hw_slowdown"]
        if bad:
            raise SystemExit(f"run rejected: throttled ({', '.join(bad)}); measure again")
        samples.append(float(obj["ms_per_step"]))
        last = obj
    rec = dict(summarize(samples), which=which, at_utc=now(), metric=last.get("metric"), value=last.get("value"),
               unit=last.get("unit"), config=last.get("config"))
    t.write(rec, t.iter_dir(), f"{which}.json")
    return rec


# ------------------------------------------------------------------------------------------------ trace readers
def read_launch_list(path) -> List[dict]:
    """Rows of an `ncu --csv` launch list: [{"id", "kernel", "ns"}]; lines before the header (ncu banners) are skipped."""
    lines = Path(path).read_text(errors="replace").splitlines()
    start = next((i for i, l in enumerate(lines) if l.startswith('"ID"')), None)
    if start is None:
        raise ValueError(f"{path}: no ncu CSV header")
    out = []
    for row in csv.DictReader(lines[start:]):
        if row.get("Metric Name") != "gpu__time_duration.sum":
            continue
        value = float(row["Metric Value"].replace(",", ""))
        unit = row.get("Metric Unit", "ns")
        ns = value * {"ns": 1.0, "us": 1e3, "ms": 1e6, "s": 1e9}.get(unit, 1.0)
        out.append({"id": int(row["ID"]), "kernel": row["Kernel Name"], "ns": ns})
    return out


def cut_one_period(path, marker: str, out_path) -> int:
    """Writes to `out_path` the part of an `ncu --csv` launch list between the last two launches whose kernel name
    contains `marker` (exclusive of the first, inclusive of the second): one step of a loop that launches the marker
    kernel once per iteration. Returns the number of launches kept."""
    lines = Path(path).read_text(errors="replace").splitlines()
    start = next((i for i, l in enumerate(lines) if l.startswith('"ID"')), None)
    if start is None:
        raise ValueError(f"{path}: no ncu CSV header")
    body = lines[start + 1:]
    names = [row.get("Kernel Name", "") for row in csv.DictReader(lines[start:])]
    hits = [i for i, n in enumerate(names) if marker in n]
    if len(hits) < 2:
        raise ValueError(f"{path}: fewer than two launches of a kernel named like '{marker}'")
    a, b = hits[-2], hits[-1]
    Path(out_path).write_text("\n".join([lines[start]] + body[a + 1:b + 1]) + "\n")
    return b - a


def short_kernel_name(full: str) -> str:
    m = re.search(r"([A-Za-z_][A-Za-z0-9_]*)\s*(<[^()]*>)?\s*\(", full)
    return m.group(1) if m else full[:60]


def read_operator_table(path) -> Dict[str, dict]:
    """`operator   ms   calls` rows of a step-profile text; comment lines may carry `fwd+bwd X ms, optimizer Y ms`."""
    ops, step_ms = {}, None
    for line in Path(path).read_text().splitlines():
        m = re.search(r"fwd\+bwd\s+([0-9.]+)\s*ms,\s*optimizer\s+([0-9.]+)\s*ms", line)
        if m and step_ms is None:          # the first such line heads the table; later ones may quote older runs
            step_ms = float(m.group(1)) + float(m.group(2))
        m = re.match(r"^([A-Za-z_][\w+() ]*?)\s+([0-9.]+)\s+([0-9]+)\s*$", line)
        if m and not line.startswith("#"):
            ops[m.group(1).strip()] = {"ms": float(m.group(2)), "calls": int(m.group(3))}
    return {"operators": ops, "step_ms": step_ms}


def trace(t: Target, launches=None, operators=None, steps: int = 1, runner=None, between: Optional[str] = None) -> dict:
    d = t.path(t.iter_dir(), "trace")
    d.mkdir(parents=True, exist_ok=True)
    spec = t.spec
    if launches and between:
        cut_one_period(launches, between, d / "launches.csv")
        launches, steps = d / "launches.csv", 1
    if not launches and not operators:
        if not spec.get("trace_cmd"):
            raise SystemExit("the target has no trace command; pass --launches and / or --operators")
        env = dict(os.environ, NANOCHAT_PGO_TRACE_DIR=str(d))
        (runner or (lambda cmd: subprocess.run(shlex.split(cmd), check=True, env=env)))(spec["trace_cmd"])
        launches = d / "launches.csv" if (d / "launches.csv").exists() else None
        operators = d / "operators.txt" if (d / "operators.txt").exists() else None
        if not launches and not operators:
            raise SystemExit(f"the trace command wrote neither launches.csv nor operators.txt into {d}")
    rec = {"steps_in_launch_list": int(steps), "at_utc": now()}
    for key, src, name in (("launches", launches, "launches.csv"), ("operators", operators, "operators.txt")):
        if src:
            if Path(src).resolve() != (d / name).resolve():
                (d / name).write_bytes(Path(src).read_bytes())
            rec[key] = name
    t.write(rec, t.iter_dir(), "trace", "trace.json")
    return rec


# ------------------------------------------------------------------------------------------------ analyze
def analyze(t: Target) -> dict:
    it = t.iter_dir()
    tr = t.read(it, "trace", "trace.json")
    if tr is None:
        raise SystemExit("no trace in this iteration")
    before = t.read(it, "before.json")
    step_ms = before["median_ms"] if before else None
    sigs, notes = [], []
    if "launches" in tr:
        rows = read_launch_list(t.path(it, "trace", tr["launches"]))
        steps = max(1, tr.get("steps_in_launch_list", 1))
        fam: Dict[str, dict] = {}
        for r in rows:
            f = fam.setdefault(family_of(r["kernel"]), {"ms": 0.0, "launches": 0, "kernels": {}})
            f["ms"] += r["ns"] / 1e6 / steps
            f["launches"] += 1
            k = short_kernel_name(r["kernel"])
            f["kernels"][k] = f["kernels"].get(k, 0.0) + r["ns"] / 1e6 / steps
        busy = sum(f["ms"] for f in fam.values())
        # under the profiler kernels run serialised and cold: compare shares, and scale to the measured step
        denom = step_ms if step_ms else busy
        for name, f in fam.items():
            top = sorted(f["kernels"].items(), key=lambda kv: -kv[1])[:3]
            sigs.append({"id": f"launches:{name}", "source": "launch list", "family": name, "ms": round(f["ms"], 4),
                         "launches_per_step": f["launches"] / steps, "share": f["ms"] / denom,
                         "ceiling": min(1.0, f["ms"] / denom), "top_kernels": [[k, round(v, 4)] for k, v in top]})
        if step_ms and busy < step_ms:
            idle = step_ms - busy
            sigs.append({"id": "launches:idle", "source": "launch list", "family": "idle", "ms": round(idle, 4),
                         "launches_per_step": len(rows) / steps, "share": idle / step_ms, "ceiling": idle / step_ms,
                         "top_kernels": []})
        elif step_ms:
            notes.append(f"kernel time under the profiler ({busy:.1f} ms) exceeds the measured step ({step_ms:.1f} ms): "
                         "kernels overlap in the real step or ran cold here; shares are relative to the step")
    if "operators" in tr:
        tab = read_operator_table(t.path(it, "trace", tr["operators"]))
        denom = step_ms or tab["step_ms"] or sum(o["ms"] for o in tab["operators"].values())
        fam = {}
        for op, o in tab["operators"].items():
            if op.startswith("sum of"):
                continue
            f = fam.setdefault(family_of(op), {"ms": 0.0, "calls": 0, "ops": {}})
            f["ms"] += o["ms"]
            f["calls"] += o["calls"]
            f["ops"][op] = o["ms"]
        for name, f in fam.items():
            top = sorted(f["ops"].items(), key=lambda kv: -kv[1])[:3]
            sigs.append({"id": f"operators:{name}", "source": "operator table", "family": name, "ms": round(f["ms"], 4),
                         "launches_per_step": f["calls"], "share": f["ms"] / denom, "ceiling": min(1.0, f["ms"] / denom),
                         "top_kernels": [[k, round(v, 4)] for k, v in top]})
    sigs.sort(key=lambda s: -s["ceiling"])
    seen, candidates = set(), []
    for s in sigs:                       # the two largest ceilings over distinct families
        if s["family"] not in seen:
            seen.add(s["family"])
            candidates.append(s["id"])
        if len(candidates) == 2:
            break
    out = {"step_ms": step_ms, "signatures": sigs, "candidates": candidates, "notes": notes, "at_utc": now()}
    t.write(out, it, "analysis.json")
    return out


# ------------------------------------------------------------------------------------------------ compare
def compare(t: Target, idea: Optional[str] = None, apply: bool = False) -> dict:
    it = t.iter_dir()
    before, after = t.read(it, "before.json"), t.read(it, "after.json")
    if not before or not after:
        raise SystemExit("compare needs both measure --before and measure --after in this iteration")
    gain = 1.0 - after["median_ms"] / before["median_ms"]           # fraction of the step removed
    noise = max(before["spread_rel"], after["spread_rel"])
    threshold = max(0.01, 2.0 * noise)
    verdict = "improved" if gain > threshold else "regressed" if gain < -threshold else "no change"
    out = {"before_ms": before["median_ms"], "after_ms": after["median_ms"], "gain": gain, "noise": noise,
           "threshold": threshold, "verdict": verdict, "speedup": before["median_ms"] / after["median_ms"],
           "flags": [], "at_utc": now()}
    if idea:
        ideas = {i["id"]: i for i in (t.read(it, "ideas.json", default=[]) or [])}
        analysis = t.read(it, "analysis.json", default={"signatures": []})
        sig_id = ideas.get(idea, {}).get("signature", idea)
        sig = next((s for s in analysis["signatures"] if s["id"] == sig_id), None)
        out["idea"], out["signature"] = idea, sig_id
        if sig is None:
            out["flags"].append(f"the idea names signature '{sig_id}', which the analysis does not have")
        elif gain > sig["ceiling"] + threshold:
            out["flags"].append(f"gain {gain:.3f} exceeds the ceiling {sig['ceiling']:.3f} of {sig_id}: "
                                "the measurement is suspect (different clocks, skipped work?)")
    t.write(out, it, "verdict.json")
    if apply:
        loop = t.loop
        loop["history"].append({"iteration": loop["iteration"], "verdict": verdict, "gain": gain,
                                "before_ms": out["before_ms"], "after_ms": out["after_ms"], "idea": idea})
        loop["iteration"] += 1
        t.write(loop, "loop.json")
        if verdict == "improved":                           # the gain becomes the next baseline
            t.write(dict(after, which="before", carried_from=it), t.iter_dir(loop["iteration"]), "before.json")
    return out


# ------------------------------------------------------------------------------------------------ report
def report(t: Target) -> str:
    spec, loop = t.spec, t.loop
    out = [f"# {spec['name']}", "", f"stage `{spec['stage']}` on `{spec['device']}`; measure: `{spec['measure_cmd']}`", ""]
    if loop["history"]:
        out += ["| iteration | idea | before ms | after ms | gain | verdict |", "|---|---|---|---|---|---|"]
        out += [f"| {h['iteration']} | {h.get('idea') or ''} | {h['before_ms']:.2f} | {h['after_ms']:.2f} | "
                f"{100 * h['gain']:+.1f} % | {h['verdict']} |" for h in loop["history"]]
        out.append("")
    it = t.iter_dir()
    out.append(f"## Iteration {loop['iteration']}")
    for which in ("before", "after"):
        m = t.read(it, f"{which}.json")
        if m:
            out.append(f"- {which}: {m['median_ms']:.2f} ms/step (spread {100 * m['spread_rel']:.1f} %, "
                       f"{len(m['samples_ms'])} runs)")
    a = t.read(it, "analysis.json")
    if a:
        out += ["", "| signature | ms/step | launches | share | ceiling | top |", "|---|---|---|---|---|---|"]
        for s in a["signatures"]:
            top = ", ".join(f"{k} {v:.2f}" for k, v in s["top_kernels"])
            mark = " **candidate**" if s["id"] in a["candidates"] else ""
            out.append(f"| {s['id']}{mark} | {s['ms']:.2f} | {s['launches_per_step']:.0f} | {100 * s['share']:.1f} % | "
                       f"{100 * s['ceiling']:.1f} % | {top} |")
        out += [""] + [f"note: {n}" for n in a["notes"]]
    v = t.read(it, "verdict.json")
    if v:
        out += ["", f"verdict: **{v['verdict']}** ({100 * v['gain']:+.2f} % of the step, threshold "
                f"{100 * v['threshold']:.2f} %)"] + [f"flag: {f}" for f in v["flags"]]
    text = "\n".join(out) + "\n"
    t.path("RESULT.md").write_text(text)
    return text


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="pgo", description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="verb", required=True)

    def common(p):
        p.add_argument("--root", default=os.environ.get("NANOCHAT_PGO_DIR", "pgo_targets"))
        p.add_argument("--name", required=True)
        return p
    p = common(sub.add_parser("init"))
    p.add_argument("--measure-cmd", required=True)
    p.add_argument("--trace-cmd", default="")
    p.add_argument("--runs", type=int, default=2)
    p.add_argument("--stage", default="base")
    p.add_argument("--device", default="b200")
    p = common(sub.add_parser("measure"))
    g = p.add_mutually_exclusive_group(required=True)
    g.add_argument("--before", action="store_true")
    g.add_argument("--after", action="store_true")
    p = common(sub.add_parser("trace"))
    p.add_argument("--launches", default=None)
    p.add_argument("--operators", default=None)
    p.add_argument("--steps", type=int, default=1, help="training steps the launch list covers")
    p.add_argument("--between", default=None, metavar="KERNEL",
                   help="keep only the launches between the last two launches of this kernel (one step of the loop)")
    common(sub.add_parser("analyze"))
    p = common(sub.add_parser("compare"))
    p.add_argument("--idea", default=None)
    p.add_argument("--apply", action="store_true")
    common(sub.add_parser("report"))
    a = ap.parse_args(argv)
    if a.verb == "init":
        init(a.root, a.name, a.measure_cmd, a.trace_cmd, a.runs, a.stage, a.device)
        print(f"target {a.name} in {Path(a.root) / a.name}")
        return 0
    t = Target(a.root, a.name)
    if a.verb == "measure":
        rec = measure(t, "before" if a.before else "after")
        print(f"{rec['which']}: {rec['median_ms']:.2f} ms/step over {len(rec['samples_ms'])} runs "
              f"(spread {100 * rec['spread_rel']:.1f} %)")
    elif a.verb == "trace":
        print(json.dumps(trace(t, a.launches, a.operators, a.steps, between=a.between)))
    elif a.verb == "analyze":
        res = analyze(t)
        for s in res["signatures"][:8]:
            print(f"{s['id']:<28} {s['ms']:9.2f} ms  share {100 * s['share']:5.1f} %  ceiling {100 * s['ceiling']:5.1f} %")
        print("candidates: " + ", ".join(res["candidates"]))
    elif a.verb == "compare":
        v = compare(t, a.idea, a.apply)
        print(f"{v['verdict']}: {v['before_ms']:.2f} -> {v['after_ms']:.2f} ms ({100 * v['gain']:+.2f} %; "
              f"threshold {100 * v['threshold']:.2f} %)")
        for f in v["flags"]:
            print("flag: " + f)
    if a.verb in ("measure", "analyze", "compare", "report"):
        text = report(t)
        if a.verb == "report":
            print(text, end="")
    return 0


if __name__ == "__main__":
    sys.exit(main())
