"""Workflow sub-commands of the command line: build, test, check, devices, doctor, verify, bench, profile, attain,
seam, prune, and the process boundary: run (sandbox), gpuq / gpu (GPU queue), session, client, sim (stand-in CUDA
runtime), fixtures, lint, shutdown.

The reference's `tools/nanochat` front end offers the same verbs around Bazel, a sandbox and a GPU queue
(python/nanochat_cpp/cli.py: build, test, check, devices, doctor, verify, bench, profile, attain). Here they run in
the calling process or as one child `python -m ...`: the extension is built by nvcc in-tree, tests are pytest tiers
(`cpu` = everything not marked gpu, `gpu` = the rest), and benchmarks are the modules under `nanochat_cpp_b200.bench`.
"""
from __future__ import annotations

import importlib
import json
import os
import shutil
import subprocess
import sys
from typing import Dict, List

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

BENCHES: Dict[str, str] = {
    "gemm": "gemm_bench", "attention": "attn_bench", "optimizer": "optim_bench", "rows": "row_bench",
    "fp8": "fp8_bench", "decode": "decode_bench", "comm": "dp_comm_bench", "cpu": "cpu_config",
}


def cmd_build(a) -> int:
    """Compile every CUDA source for sm_100a and the host runtime, link them in-tree, import the result."""
    from . import build as b
    b.build_all(verbose=not a.quiet)
    importlib.import_module("nanochat_cpp_b200")
    print(json.dumps({"extension": b.EXT_PATH, "exists": os.path.exists(b.EXT_PATH)}))
    return 0 if os.path.exists(b.EXT_PATH) else 1


def _pytest(tier: str, extra: List[str]) -> int:
    marker = {"cpu": "not gpu", "gpu": "gpu"}[tier]
    cmd = [sys.executable, "-m", "pytest", os.path.join(ROOT, "tests"), "-q", "-m", marker] + extra
    return subprocess.call(cmd, cwd=ROOT)


def cmd_test(a) -> int:
    """One test tier: `cpu` needs no GPU (multi-process paths use gloo), `gpu` needs one B200."""
    return _pytest(a.tier, a.rest)


def cmd_check(a) -> int:
    """Build, then the CPU tier, then (when a GPU is present) the hardware gate: what a change must pass."""
    rc = cmd_build(a)
    if rc:
        return rc
    rc = _pytest("cpu", ["-x"])
    if rc:
        return rc
    import torch
    return cmd_verify(a) if torch.cuda.is_available() else 0


def device_table() -> List[dict]:
    """CPU entry first, then one entry per visible GPU (name, SMs, memory, compute capability, peer access)."""
    import torch
    out = [{"index": -1, "kind": "cpu", "name": "host", "threads": os.cpu_count()}]
    if torch.cuda.is_available():
        n = torch.cuda.device_count()
        for i in range(n):
            p = torch.cuda.get_device_properties(i)
            peers = [j for j in range(n) if j != i and torch.cuda.can_device_access_peer(i, j)]
            out.append({"index": i, "kind": "cuda", "name": p.name, "sms": p.multi_processor_count,
                        "memory_gib": round(p.total_memory / 2 ** 30, 1), "cc": f"{p.major}.{p.minor}",
                        "native": (p.major, p.minor) == (10, 0), "peers": peers})
    return out


def cmd_devices(a) -> int:
    for d in device_table():
        print(json.dumps(d))
    return 0


def doctor_report() -> dict:
    """What the framework needs and whether it is there: interpreter, torch, CUDA toolchain, the built extension and
    host library, collective backends, measured peaks."""
    import torch
    from . import build as b
    rep = {
        "python": sys.version.split()[0],
        "torch": torch.__version__,
        "torch_cuda": torch.version.cuda,
        "gpu_visible": torch.cuda.is_available(),
        "nvcc": shutil.which("nvcc") or (os.path.exists("/usr/local/cuda/bin/nvcc") and "/usr/local/cuda/bin/nvcc") or None,
        "extension_built": os.path.exists(b.EXT_PATH),
        "host_library_built": os.path.exists(os.path.join(os.path.dirname(b.EXT_PATH), "libnanochat_core.so")),
        "native_cli_built": os.path.exists(os.path.join(os.path.dirname(b.EXT_PATH), "nanochat_cli")),
        "nccl": bool(torch.distributed.is_available() and torch.distributed.is_nccl_available()),
        "gloo": bool(torch.distributed.is_available() and torch.distributed.is_gloo_available()),
        "measured_peaks": os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")),
    }
    if rep["gpu_visible"]:
        cc = torch.cuda.get_device_capability(0)
        rep["gpu0"] = torch.cuda.get_device_name(0)
        rep["gpu0_is_sm100"] = cc == (10, 0)
    problems = []
    if not rep["extension_built"]:
        problems.append("CUDA extension not built: run `build`")
    if not rep["host_library_built"]:
        problems.append("host runtime library not built: run `build`")
    if rep["nvcc"] is None:
        problems.append("nvcc not found: the extension cannot be rebuilt here")
    if rep["gpu_visible"] and not rep.get("gpu0_is_sm100", False):
        problems.append("GPU 0 is not sm_100: the kernels are compiled for sm_100a only")
    rep["problems"] = problems
    return rep


def cmd_doctor(a) -> int:
    rep = doctor_report()
    print(json.dumps(rep, indent=1))
    return 1 if rep["problems"] and a.strict else 0


def cmd_verify(a) -> int:
    """The start-up correctness gate on GPU `--device` (kernels against the PyTorch definitions)."""
    import torch
    if not torch.cuda.is_available():
        print(json.dumps({"ok": False, "error": "no GPU visible"}))
        return 1
    from .hwgate import run_hardware_gate
    ok, report = run_hardware_gate(getattr(a, "device", "cuda:0") or "cuda:0")
    for r in report:
        print(json.dumps(r))
    print(json.dumps({"ok": ok, "checks": len(report)}))
    return 0 if ok else 1


def cmd_bench(a) -> int:
    """`bench list`, `bench step [bench.py flags]` (the headline training step) or `bench <name> [flags]`."""
    if a.name == "list":
        print(json.dumps({"step": "bench.py (d20 training step, tokens/s)",
                          **{k: f"nanochat_cpp_b200.bench.{v}" for k, v in BENCHES.items()}}, indent=1))
        return 0
    if a.name == "step":
        return subprocess.call([sys.executable, os.path.join(ROOT, "bench.py")] + a.rest, cwd=ROOT)
    if a.name not in BENCHES:
        print(f"bench: unknown benchmark {a.name!r}; try `bench list`", file=sys.stderr)
        return 2
    return subprocess.call([sys.executable, "-m", f"nanochat_cpp_b200.bench.{BENCHES[a.name]}"] + a.rest, cwd=ROOT)


def cmd_profile(a) -> int:
    """Per-operator device time of one training step (CUDA events around every operator)."""
    return subprocess.call([sys.executable, "-m", "nanochat_cpp_b200.bench.step_profile"] + a.rest, cwd=ROOT)


def cmd_attain(a) -> int:
    """Measured phase times against the roofline model (fraction of the attainable time per phase)."""
    return subprocess.call([sys.executable, "-m", "nanochat_cpp_b200.perf.attain"] + a.rest, cwd=ROOT)


def seam_table() -> List[dict]:
    """Every operator of the seam with where it is implemented: the PyTorch definition and, when the extension is
    built, the sm_100a kernel (the reference's `seam` verb lists kernels.h entry points per backend)."""
    from . import ops
    try:
        cuda_mod = ops.cuda_module()
    except Exception:                      # extension not built: definitions only
        cuda_mod = None
    rows = []
    for name in ops._NAMES:
        has_kernel = False
        if cuda_mod is not None:
            try:
                has_kernel = callable(getattr(cuda_mod, name))
            except AttributeError:
                has_kernel = False
        rows.append({"operator": name, "definition": hasattr(ops.ref, name), "kernel": has_kernel})
    return rows


def cmd_seam(a) -> int:
    rows = seam_table()
    for r in rows:
        print(json.dumps(r))
    missing = [r["operator"] for r in rows if not r["definition"]]
    return 1 if missing else 0


def prune_checkpoints(directory: str, keep: int, pattern: str = "*.ckpt") -> List[str]:
    """Delete all but the `keep` newest checkpoints matching `pattern` in `directory`, with their cursor sidecars
    (files that start with the checkpoint's name). Returns the deleted paths."""
    import glob
    paths = sorted(glob.glob(os.path.join(directory, pattern)), key=os.path.getmtime, reverse=True)
    removed = []
    for path in paths[max(0, keep):]:
        for victim in [path] + [q for q in glob.glob(path + "*") if q != path]:
            os.remove(victim)
            removed.append(victim)
    return removed


def cmd_prune(a) -> int:
    """Remove stale native build objects (those no current source hashes to) and, with --checkpoints, old checkpoints."""
    from . import build as b
    before = set(os.listdir(b.BUILD_DIR)) if os.path.isdir(b.BUILD_DIR) else set()
    if a.build:
        b.build_all(verbose=False)         # compiling nothing new; its prune step drops objects of changed sources
    after = set(os.listdir(b.BUILD_DIR)) if os.path.isdir(b.BUILD_DIR) else set()
    removed = prune_checkpoints(a.checkpoints, a.keep) if a.checkpoints else []
    print(json.dumps({"build_objects_removed": len(before - after), "checkpoints_removed": removed}))
    return 0



# ------------------------------------------------------------------------------------------------ process boundary
def _after_dashes(rest: List[str]) -> List[str]:
    return rest[1:] if rest[:1] == ["--"] else rest


def cmd_run(a) -> int:
    """`run <profile> -- cmd`: the command under that resource profile (process/sandbox.py)."""
    from .process import sandbox
    return sandbox.launch(a.profile, _after_dashes(a.rest), a.backend)


def cmd_gpuq(a) -> int:
    from .process import gpu_queue
    return gpu_queue.main(a.rest)


def cmd_gpu(a) -> int:
    """`gpu [--gpus N] [--profile P] -- cmd`: submit to the GPU queue, start a worker if none is live, follow the
    log, return the job's exit code."""
    from .process import gpu_queue as q
    cmd = _after_dashes(a.rest)
    if not cmd:
        print("gpu: no command", file=sys.stderr)
        return 2
    conn = q.open_db()
    if not q.live_workers(conn):
        subprocess.Popen([sys.executable, "-m", "nanochat_cpp_b200.process.gpu_queue", "worker", "--idle-exit", "600"],
                         start_new_session=True, stdin=subprocess.DEVNULL, stdout=subprocess.DEVNULL,
                         stderr=subprocess.DEVNULL)
    job = q.submit(conn, cmd, a.gpus, a.profile)
    print(f"[gpuq] job {job}", file=sys.stderr)
    return q.wait_for(conn, job, follow=sys.stdout)


def cmd_session(a) -> int:
    from .process import supervisor
    return supervisor.main(a.rest)


def cmd_client(a) -> int:
    """`client [--device cuda:N|cpu] [--profile P] -- cmd`: a program that uses the C ABI, started in the sandbox with
    the device selected through NANOCHAT_DEVICE."""
    from .process import sandbox
    env = dict(os.environ, NANOCHAT_DEVICE=a.device)
    return sandbox.launch(a.profile, _after_dashes(a.rest), "auto", env=env)


def cmd_sim(a) -> int:
    """`sim -- cmd`: the command with the stand-in CUDA runtime preloaded; prints the summary of its trace."""
    from . import build as b
    lib = b.build_sim()
    cmd = _after_dashes(a.rest)
    if not lib or not cmd:
        print("sim: the stand-in runtime is not built, or no command", file=sys.stderr)
        return 2
    trace = a.trace or os.path.join(os.getcwd(), "cudart_sim_trace.jsonl")
    env = dict(os.environ, LD_PRELOAD=lib, NANOCHAT_SIM_TRACE=trace, NANOCHAT_SIM_STRICT="1" if a.strict else "0")
    rc = subprocess.run(cmd, env=env).returncode
    try:
        rows = [json.loads(line) for line in open(trace)]
        summary = rows[-1] if rows and rows[-1].get("call") == "summary" else {}
        for v in [r for r in rows if r.get("call") == "violation"][:20]:
            print(f"[sim] {v['in']}: {v['what']}", file=sys.stderr)
        print(json.dumps({k: summary.get(k) for k in ("launches", "tensor_maps", "violations", "live_allocations",
                                                      "live_bytes")}))
        if summary.get("violations"):
            rc = rc or 1
    except OSError:
        pass
    return rc


def cmd_fixtures(a) -> int:
    from .fixtures import generate
    return generate.main((["--check"] if a.check else []) + a.names)


LINT_NOTES = ("SURVEY" + ".md", "VERDICT" + ".md", "ADVICE" + ".md", "DESIGN" + ".md", "BASELINE" + ".md")


def lint_findings(root: str = ROOT) -> List[str]:
    """House rules that a compiler does not check: every Python file byte-compiles; GPU tests carry the gpu marker;
    profiler commands in profiles/ leave the clocks alone; sources do not point at working notes or at paths of one
    machine; nothing stops processes by name pattern."""
    import re
    out = []
    skip = {"_work", "gpurun_out", ".git", "_build", "__pycache__", "_ref"}
    for dirpath, dirs, files in os.walk(root):
        dirs[:] = [d for d in dirs if d not in skip]
        for f in files:
            path = os.path.join(dirpath, f)
            rel = os.path.relpath(path, root)
            if f.endswith(".py"):
                try:
                    compile(open(path, errors="replace").read(), path, "exec")
                except SyntaxError as e:
                    out.append(f"{rel}: does not compile: line {e.lineno}: {e.msg}")
            if f.endswith((".py", ".cu", ".cuh", ".cc", ".cpp", ".h")):
                text = open(path, errors="replace").read()
                for note in LINT_NOTES:
                    if note in text:
                        out.append(f"{rel}: names the working note {note}")
                if re.search(r"\bpkill\s+-f\b|\bkillall\b", text) and rel != os.path.relpath(__file__, root):
                    out.append(f"{rel}: stops processes by name pattern")
                if re.match(r"tests/test_.*_gpu\.py$", rel.replace(os.sep, "/")) and "pytest.mark.gpu" not in text:
                    out.append(f"{rel}: a GPU test file without the gpu marker")
            if rel.startswith("profiles") and f.endswith((".md", ".txt")):
                for line in open(path, errors="replace"):
                    if re.search(r"(^|\s)ncu\s+-", line) and "--clock-control none" not in line and " -i " not in line:
                        out.append(f"{rel}: an ncu command without --clock-control none: {line.strip()[:80]}")
    return out


def cmd_lint(a) -> int:
    found = lint_findings()
    for line in found:
        print(line)
    print(f"lint: {len(found)} finding(s)")
    return 1 if found else 0


def cmd_shutdown(a) -> int:
    """Stop what outlives a command: live queue workers and session supervisors (each by the pid in its own record)."""
    import signal
    from .process import gpu_queue as q, supervisor as v
    stopped = {"workers": 0, "sessions": 0}
    conn = q.open_db()
    for w in q.live_workers(conn):
        if q.pid_alive(w["pid"]):
            os.kill(w["pid"], signal.SIGTERM)
            stopped["workers"] += 1
    for rec in v.status():
        if rec["state"] == "live" and v.stop(rec["name"]):
            stopped["sessions"] += 1
    print(json.dumps(stopped))
    return 0


def register(sub) -> None:
    import argparse
    ap = sub.add_parser("build", help="compile the CUDA extension and the host runtime in-tree")
    ap.add_argument("--quiet", action="store_true")
    ap.set_defaults(fn=cmd_build)
    ap = sub.add_parser("test", help="run a test tier")
    ap.add_argument("tier", choices=["cpu", "gpu"])
    ap.add_argument("rest", nargs=argparse.REMAINDER, help="extra pytest arguments")
    ap.set_defaults(fn=cmd_test)
    ap = sub.add_parser("check", help="build + CPU tier (+ hardware gate when a GPU is present)")
    ap.add_argument("--quiet", action="store_true")
    ap.set_defaults(fn=cmd_check)
    ap = sub.add_parser("devices", help="list the CPU and the visible GPUs")
    ap.set_defaults(fn=cmd_devices)
    ap = sub.add_parser("doctor", help="environment report")
    ap.add_argument("--strict", action="store_true", help="exit 1 when a problem is listed")
    ap.set_defaults(fn=cmd_doctor)
    ap = sub.add_parser("verify", help="hardware correctness gate")
    ap.add_argument("--device", default="cuda:0")
    ap.set_defaults(fn=cmd_verify)
    ap = sub.add_parser("bench", help="run a benchmark: list | step | " + " | ".join(BENCHES))
    ap.add_argument("name")
    ap.add_argument("rest", nargs=argparse.REMAINDER)
    ap.set_defaults(fn=cmd_bench)
    ap = sub.add_parser("profile", help="per-operator step profile")
    ap.add_argument("rest", nargs=argparse.REMAINDER)
    ap.set_defaults(fn=cmd_profile)
    ap = sub.add_parser("seam", help="operators of the seam and where each is implemented")
    ap.set_defaults(fn=cmd_seam)
    ap = sub.add_parser("prune", help="drop stale build objects and old checkpoints")
    ap.add_argument("--build", action="store_true", help="prune the native build cache")
    ap.add_argument("--checkpoints", default="", help="directory of *.ckpt files")
    ap.add_argument("--keep", type=int, default=3)
    ap.set_defaults(fn=cmd_prune)
    ap = sub.add_parser("attain", help="attainment report against the roofline model")
    ap.add_argument("rest", nargs=argparse.REMAINDER)
    ap.set_defaults(fn=cmd_attain)
    ap = sub.add_parser("run", help="run <profile> -- cmd: a command under a resource profile")
    ap.add_argument("profile")
    ap.add_argument("--backend", default="auto", choices=["auto", "cgroup", "rlimit", "none"])
    ap.add_argument("rest", nargs=argparse.REMAINDER)
    ap.set_defaults(fn=cmd_run)
    ap = sub.add_parser("gpuq", help="GPU job queue: submit | worker | list | status | cancel | logs | wait | prune")
    ap.add_argument("rest", nargs=argparse.REMAINDER)
    ap.set_defaults(fn=cmd_gpuq)
    ap = sub.add_parser("gpu", help="gpu [--gpus N] [--profile P] -- cmd: run a command through the GPU queue")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--profile", default="gpu-test")
    ap.add_argument("rest", nargs=argparse.REMAINDER)
    ap.set_defaults(fn=cmd_gpu)
    ap = sub.add_parser("session", help="session start | send | status | stop")
    ap.add_argument("rest", nargs=argparse.REMAINDER)
    ap.set_defaults(fn=cmd_session)
    ap = sub.add_parser("client", help="client [--device D] [--profile P] -- cmd: a C-ABI program in the sandbox")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--profile", default="train")
    ap.add_argument("rest", nargs=argparse.REMAINDER)
    ap.set_defaults(fn=cmd_client)
    ap = sub.add_parser("sim", help="sim -- cmd: run with the stand-in CUDA runtime preloaded (no GPU needed)")
    ap.add_argument("--trace", default="")
    ap.add_argument("--strict", action="store_true")
    ap.add_argument("rest", nargs=argparse.REMAINDER)
    ap.set_defaults(fn=cmd_sim)
    ap = sub.add_parser("fixtures", help="produce (or --check) the package's own fixtures")
    ap.add_argument("--check", action="store_true")
    ap.add_argument("names", nargs="*")
    ap.set_defaults(fn=cmd_fixtures)
    ap = sub.add_parser("lint", help="house rules no compiler checks")
    ap.set_defaults(fn=cmd_lint)
    ap = sub.add_parser("gates", help="consistency gates: C ABI header / library / callers, stdlib isolation, fixtures, lint")
    ap.set_defaults(fn=lambda a: __import__("nanochat_cpp_b200.gates", fromlist=["main"]).main([]))
    ap = sub.add_parser("pgo", help="pgo init | measure | trace | analyze | compare | report: the measured half of the optimisation loop")
    ap.add_argument("rest", nargs=argparse.REMAINDER)
    ap.set_defaults(fn=lambda a: __import__("nanochat_cpp_b200.perf.pgo", fromlist=["main"]).main(a.rest))
    ap = sub.add_parser("contract", help="contract verify [--engine E] | table: per-record tolerance contract of the parity fixtures")
    ap.add_argument("rest", nargs=argparse.REMAINDER)
    ap.set_defaults(fn=lambda a: __import__("nanochat_cpp_b200.contract", fromlist=["main"]).main(a.rest or ["verify"]))
    ap = sub.add_parser("shutdown", help="stop live queue workers and session supervisors")
    ap.set_defaults(fn=cmd_shutdown)
