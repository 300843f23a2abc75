"""Consistency gates: facts that several files state and nothing else keeps in step.

    python -m nanochat_cpp_b200.cli gates

  capi        every function declared in include/nanochat/capi.h is exported by libnanochat_core.so, and every
              `nanochat_*` symbol the Python bindings look up is declared in the header (the C ABI is the contract
              of three parties: the header, the library, the ctypes callers);
  isolation   the process-boundary modules (sandbox, GPU queue, supervisor) import only the standard library: they
              must start on a machine where the package's native parts are not built yet;
  fixtures    the committed fixtures of this package are what its producers give today (fixtures/generate.py --check);
  contract    both CPU engines (PyTorch operators, native C++) stay inside the per-record bounds of
              model_specs/nanochat-default.tolerances.json on the reference's fp32 fixtures, the files have the recorded
              SHA-256, and every record of each file resolves to a bound;
  lint        the house rules of `tools_cli.lint_findings`.

The reference keeps the same kind of facts in step with generators and gates of its own (tools/gen_capi_mirrors.py,
tools/isolation_gate.py, tools/doc_facts.py); the mirrors here are hand-written, so the gate checks them instead of
generating them.
"""
from __future__ import annotations

import ast
import ctypes
import os
import re
import sys
from typing import Dict, List

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.dirname(os.path.abspath(__file__))


def header_functions(path: str = os.path.join(ROOT, "include", "nanochat", "capi.h")) -> List[str]:
    text = re.sub(r"/\*.*?\*/", " ", open(path).read(), flags=re.S)
    text = re.sub(r"//[^\n]*", " ", text)
    names = re.findall(r"\b(nanochat_[a-z0-9_]+)\s*\(", text)
    seen, out = set(), []
    for n in names:
        if n not in seen:
            seen.add(n)
            out.append(n)
    return out


def capi_findings() -> List[str]:
    out = []
    declared = header_functions()
    lib_path = os.path.join(PKG, "libnanochat_core.so")
    if not os.path.exists(lib_path):
        return [f"{lib_path} is not built"]
    lib = ctypes.CDLL(lib_path)
    for name in declared:
        if not hasattr(lib, name):
            out.append(f"capi: {name} is declared in capi.h but not exported by libnanochat_core.so")
    known = set(declared)
    for rel in ("cpu_engine.py", "native_mesh.py", os.path.join("data", "native.py"), "runtime.py", "api.py"):
        path = os.path.join(PKG, rel)
        if not os.path.exists(path):
            continue
        for name in set(re.findall(r"\b(nanochat_[a-z0-9_]+)\b", open(path).read())):
            if name.startswith("nanochat_cpp") or name in ("nanochat_cli", "nanochat_core", "nanochat_gpu"):
                continue
            if hasattr(lib, name) and name not in known:
                out.append(f"capi: {rel} calls {name}, which the library exports but capi.h does not declare")
    return out


STDLIB = set(getattr(sys, "stdlib_module_names", ()))


def isolation_findings() -> List[str]:
    out = []
    d = os.path.join(PKG, "process")
    for f in sorted(os.listdir(d)):
        if not f.endswith(".py"):
            continue
        tree = ast.parse(open(os.path.join(d, f)).read())
        for node in ast.walk(tree):
            mods = []
            if isinstance(node, ast.Import):
                mods = [a.name.split(".")[0] for a in node.names]
            elif isinstance(node, ast.ImportFrom) and node.level == 0 and node.module:
                mods = [node.module.split(".")[0]]
            for m in mods:
                if m not in STDLIB and m != "nanochat_cpp_b200":
                    out.append(f"isolation: process/{f} imports {m}")
    return out


def fixture_findings() -> List[str]:
    from .fixtures import generate as G
    out = []
    data = os.path.join(ROOT, "tests", "data")
    for name, (fname, fn) in G.PRODUCERS.items():
        path = os.path.join(data, fname)
        if not os.path.exists(path):
            out.append(f"fixtures: {fname} is missing")
            continue
        bad = G.compare(fn(), path)
        if bad:
            out.append(f"fixtures: {fname} differs from its producer in {', '.join(bad[:4])}")
    return out


def contract_findings() -> List[str]:
    from . import contract as K
    contracts = K.load_tolerances()
    out = []
    for file in K.PRODUCERS:
        for engine in K.ENGINES:
            out += [f"contract: {file} [{engine}] {b}" for b in K.run_fixture(file, engine, contracts=contracts)]
    return out


def run_all(skip_fixtures: bool = False) -> Dict[str, List[str]]:
    from .tools_cli import lint_findings
    res = {"capi": capi_findings(), "isolation": isolation_findings(), "lint": lint_findings()}
    if not skip_fixtures:
        res["fixtures"] = fixture_findings()
        res["contract"] = contract_findings()
    return res


def main(argv=None) -> int:
    res = run_all()
    total = 0
    for gate, found in res.items():
        print(f"{gate}: {'ok' if not found else str(len(found)) + ' finding(s)'}")
        for line in found:
            print("  " + line)
        total += len(found)
    return 1 if total else 0


if __name__ == "__main__":
    sys.exit(main())
