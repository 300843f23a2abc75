"""Per-record tolerance contract for the parity fixtures, and the runner that holds an engine to it.

    python -m nanochat_cpp_b200.contract verify [--engine python|native|both] [--json]
    python -m nanochat_cpp_b200.contract table

`model_specs/nanochat-default.tolerances.json` lists, for every fixture an engine is judged against, the file's
SHA-256 and record count and an ordered list of (name pattern -> bound). The first matching pattern wins and every
record of the file must resolve to a bound, so a fixture cannot grow a record that nothing checks. Bounds:

    exact       equal arrays (inputs, configuration, token ids)
    absolute    every element: |got - want| <= atol + rtol * |want|
    norm        the L2 norms: | ||got|| - ||want|| | <= atol + rtol * ||want||
    input       the record feeds the engine and is not an output of it (its integrity is the file's SHA-256)

An *engine* here is a function from the fixture's records to a dict of produced records with the same names; the
runner (`run_fixture`) applies the bounds and reports every violation with the record name, the worst element and
its bound. Engines for the fp32 debug-state fixture (forward, backward, three optimizer steps) exist for the PyTorch
operator path and for the native C++ engine through its C ABI; a new backend joins by adding one producer.

Same role as the reference's models/nanochat-default/tolerances.json (per-record bounds, first match wins, coverage
of every record) and the isolation gate that reads it; the numbers for the reference's own fixtures are the
reference's (tests/oracle_test.cc:83-95).
"""
from __future__ import annotations

import argparse
import dataclasses
import fnmatch
import hashlib
import json
import os
import sys
from typing import Callable, Dict, List, Optional

import numpy as np

PKG = os.path.dirname(os.path.abspath(__file__))
DEFAULT_PATH = os.path.join(PKG, "model_specs", "nanochat-default.tolerances.json")
DATA_DIR = os.path.join(os.path.dirname(PKG), "tests", "data")


@dataclasses.dataclass
class Bound:
    mode: str
    atol: float = 0.0
    rtol: float = 0.0
    source: str = ""

    def violation(self, got, want) -> Optional[str]:
        """None when `got` is within the bound of `want`, else a one-line description."""
        if self.mode == "input":
            return None
        g, w = np.asarray(got), np.asarray(want)
        if g.size != w.size:
            return f"size {g.size} != {w.size}"
        g, w = g.reshape(-1), w.reshape(-1)
        if self.mode == "exact":
            if np.array_equal(g, w):
                return None
            i = int(np.flatnonzero(g != w)[0])
            return f"differs at {i}: got {g[i]!r} want {w[i]!r}"
        g, w = g.astype(np.float64), w.astype(np.float64)
        if not np.isfinite(g).all():
            return "non-finite values"
        if self.mode == "absolute":
            over = np.abs(g - w) - (self.atol + self.rtol * np.abs(w))
            i = int(np.argmax(over))
            return None if over[i] <= 0 else (f"|err| {abs(g[i] - w[i]):.3e} at {i} > "
                                              f"{self.atol + self.rtol * abs(w[i]):.3e} (got {g[i]:.8g} want {w[i]:.8g})")
        if self.mode == "norm":
            a, b = float(np.linalg.norm(g)), float(np.linalg.norm(w))
            lim = self.atol + self.rtol * b
            return None if abs(a - b) <= lim else f"norm {a:.8g} vs {b:.8g}: off by {abs(a - b):.3e} > {lim:.3e}"
        return f"unknown bound mode '{self.mode}'"


@dataclasses.dataclass
class FixtureContract:
    file: str
    sha256: str
    record_count: int
    precision: str
    rules: List[tuple]          # (pattern, Bound), in order

    def bound_for(self, name: str) -> Optional[Bound]:
        for pat, b in self.rules:
            if fnmatch.fnmatchcase(name, pat):
                return b
        return None

    def uncovered(self, names) -> List[str]:
        return sorted(n for n in names if self.bound_for(n) is None)

    def verify_file(self, path: str) -> List[str]:
        out = []
        with open(path, "rb") as f:
            digest = hashlib.sha256(f.read()).hexdigest()
        if digest != self.sha256:
            out.append(f"{self.file}: sha256 {digest} is not the contract's {self.sha256}")
        return out

    def check(self, produced: Dict[str, np.ndarray], recorded: Dict[str, np.ndarray]) -> List[str]:
        """Violations of every produced record against the file's, plus output records nothing produced."""
        bad = []
        for name, want in recorded.items():
            b = self.bound_for(name)
            if b is None:
                bad.append(f"{name}: no bound in the contract")
            elif b.mode != "input":
                if name not in produced:
                    bad.append(f"{name}: not produced")
                else:
                    v = b.violation(produced[name], want)
                    if v:
                        bad.append(f"{name}: {v}  [{b.mode} atol={b.atol:g} rtol={b.rtol:g}; {b.source}]")
        return bad


def load_tolerances(path: str = DEFAULT_PATH) -> Dict[str, FixtureContract]:
    doc = json.load(open(path))
    if doc.get("schema_version") != 1:
        raise ValueError(f"{path}: unknown schema_version")
    out = {}
    for fx in doc["fixtures"]:
        rules = [(r["match"], Bound(r["mode"], float(r.get("atol", 0.0)), float(r.get("rtol", 0.0)), r.get("source", "")))
                 for r in fx["records"]]
        out[fx["file"]] = FixtureContract(fx["file"], fx["sha256"], int(fx["record_count"]), fx.get("precision", "fp32"),
                                          rules)
    return out


# ------------------------------------------------------------------------------------------------ producers
def _config_of(recs):
    from .config import Config
    g = lambda k: int(recs["config/" + k][0])
    return Config(num_layers=g("layers"), num_heads=g("heads"), num_kv_heads=g("kv_heads"), hidden_dim=g("embd"),
                  seq_len=g("seq"), vocab_size=g("vocab"), padded_vocab_size=g("padded_vocab"), rope_base=100000.0,
                  window_pattern=bytes(recs["config/window_pattern"]).decode())


def _optim_fields(recs) -> dict:
    """Optimizer and schedule fields of a fixture; absent schedule fields mean a constant schedule."""
    o = lambda k, d: float(recs["config/opt/" + k][0]) if "config/opt/" + k in recs else d
    s = lambda k, d: float(recs["config/sched/" + k][0]) if "config/sched/" + k in recs else d
    return dict(unembedding_lr=o("unembedding_lr", 0.0), embedding_lr=o("embedding_lr", 0.0),
                matrix_lr=o("matrix_lr", 0.0), scalar_lr=o("scalar_lr", 0.0), weight_decay=o("weight_decay", 0.0),
                clip=o("clip", 0.0), adam_eps=o("adam_eps", 1e-10),
                num_iterations=int(s("num_iterations", 0)), warmup_steps=int(s("warmup_steps", 0)),
                warmdown_ratio=s("warmdown_ratio", 0.0), final_lr_frac=s("final_lr_frac", 0.0),
                weight_decay_base=s("weight_decay_base", 0.0),
                muon_momentum_warmup_steps=s("muon_momentum_warmup_steps", 0.0),
                muon_momentum_start=s("muon_momentum_start", 0.95), muon_momentum_peak=s("muon_momentum_peak", 0.95),
                muon_momentum_final=s("muon_momentum_final", 0.95))


class _PythonEngine:
    """The PyTorch operator path in fp32."""
    name = "python"

    def __init__(self, recs, prefix):
        import torch
        from .models import GPT
        self.torch, self.cfg = torch, _config_of(recs)
        self.m = GPT(self.cfg, "cpu", torch.float32, init=False)
        self.m.load_state_dict({n: torch.from_numpy(np.array(recs[prefix + n])).reshape(
            self.m.params.m(n).shape) for n in self.m.params.names()})
        self.opt = None

    def names(self):
        return self.m.params.names()

    def _t(self, a):
        return self.torch.from_numpy(np.array(a)).long()

    def raw_logits(self, tok):
        return self.m.logits(self._t(tok)).numpy()

    def loss(self, tok, tgt) -> float:
        return self.m.forward_loss(self._t(tok), self._t(tgt)).item()

    def forward_backward(self, tok, tgt) -> float:
        self.m.zero_grad()
        return self.m.forward_backward(self._t(tok), self._t(tgt)).item()

    def grad(self, n):
        return self.m.params.g(n).detach().numpy().copy()

    def param(self, n):
        return self.m.params.m(n).detach().numpy().copy()

    def make_optimizer(self, fields):
        from .optim import Optimizer, OptimizerConfig, SchedulerConfig
        oc = {k: fields[k] for k in ("unembedding_lr", "embedding_lr", "matrix_lr", "scalar_lr", "weight_decay", "clip",
                                     "adam_eps")}
        sc = {k: v for k, v in fields.items() if k not in oc}
        self.opt = Optimizer(self.m.params, OptimizerConfig(**oc), SchedulerConfig(**sc))

    def step(self, k):
        self.opt.step(k)

    def grad_norm(self) -> float:
        return float(self.opt.grad_norm())


class _NativeEngine:
    """The C++ CPU engine through the C ABI. It exposes losses, parameters and parameter gradients (not logits)."""
    name = "native"

    def __init__(self, recs, prefix):
        from .cpu_engine import CpuModel
        self.cfg = _config_of(recs)
        self.m = CpuModel(self.cfg)
        for n in self.m.names():
            self.m.write(n, np.array(recs[prefix + n]))
        self.opt = None

    def names(self):
        return self.m.names()

    def loss(self, tok, tgt) -> float:
        return self.m.forward_loss(np.array(tok), np.array(tgt))

    def forward_backward(self, tok, tgt) -> float:
        self.m.zero_grad()
        loss = self.m.forward_loss(np.array(tok), np.array(tgt))
        self.m.backward()
        return loss

    def grad(self, n):
        return self.m.read(n, grad=True)

    def param(self, n):
        return self.m.read(n)

    def make_optimizer(self, fields):
        from .cpu_engine import CpuOptimizer
        self.opt = CpuOptimizer(self.m, **fields)

    def step(self, k):
        self.opt.step(k)

    def grad_norm(self) -> float:
        return float(self.opt.grad_norm())


ENGINES = {"python": _PythonEngine, "native": _NativeEngine}


def produce_debug_state(engine_cls, recs) -> Dict[str, np.ndarray]:
    """Forward, backward and a short optimizer trajectory on one fixed batch."""
    tok, tgt = recs["input/tokens"], recs["input/targets"]
    out = {}
    e = engine_cls(recs, "param/")
    if hasattr(e, "raw_logits"):
        full = np.array(recs["forward/raw_logits"]).copy()       # padded vocabulary columns are not produced
        full[..., :e.cfg.vocab_size] = e.raw_logits(tok)
        out["forward/raw_logits"] = full
    out["forward/loss"] = np.array([e.forward_backward(tok, tgt)])
    for n in e.names():
        out["grad/" + n] = e.grad(n)
    e = engine_cls(recs, "step/0/param/")
    e.make_optimizer(_optim_fields(recs))
    out["step/0/loss"] = np.array([e.loss(tok, tgt)])
    for n in e.names():
        out["step/0/param/" + n] = e.param(n)
    for k in range(1, int(recs["config/steps"][0]) + 1):
        e.forward_backward(tok, tgt)
        e.step(k)
        out[f"step/{k}/loss"] = np.array([e.loss(tok, tgt)])
        for n in e.names():
            out[f"step/{k}/param/{n}"] = e.param(n)
    return out


def produce_train_parity(engine_cls, recs) -> Dict[str, np.ndarray]:
    """A 20-step training run on recorded batches: per step the loss of the batch re-scored after the update, the
    global gradient norm, and the L2 norm of every gradient and parameter."""
    out = {}
    e = engine_cls(recs, "param/")
    e.make_optimizer(_optim_fields(recs))
    norm = lambda a: np.array([float(np.linalg.norm(np.asarray(a, dtype=np.float64)))])
    for n in e.names():
        out[f"step/0/param_l2/{n}"] = norm(e.param(n))
    for k in range(1, int(recs["config/steps"][0]) + 1):
        tok, tgt = recs[f"batch/{k - 1}/tokens"], recs[f"batch/{k - 1}/targets"]
        loss = e.forward_backward(tok, tgt)
        if k == 1:
            out["step/0/loss"] = np.array([loss])
        for n in e.names():
            out[f"step/{k}/grad_l2/{n}"] = norm(e.grad(n))
        e.step(k)
        out[f"step/{k}/grad_norm"] = np.array([e.grad_norm()])
        out[f"step/{k}/loss"] = np.array([e.loss(tok, tgt)])
        for n in e.names():
            out[f"step/{k}/param_l2/{n}"] = norm(e.param(n))
    return out


# records an engine may leave out: intermediate activations that only a graph-level engine can expose
OPTIONAL = {"python": ("forward/logits", "grad/raw_logits", "grad/logits"),
            "native": ("forward/raw_logits", "forward/logits", "grad/raw_logits", "grad/logits")}
PRODUCERS: Dict[str, Callable] = {"debug_state.bin": produce_debug_state, "train_parity.bin": produce_train_parity}


def run_fixture(file: str, engine: str, data_dir: str = DATA_DIR, contracts=None) -> List[str]:
    """All violations of one engine on one fixture (file integrity, coverage, bounds). Empty = the engine conforms."""
    from .data.record_file import read_records
    contracts = contracts or load_tolerances()
    c = contracts[file]
    path = os.path.join(data_dir, file)
    bad = c.verify_file(path)
    _, recs = read_records(path)
    if len(recs) != c.record_count:
        bad.append(f"{file}: {len(recs)} records, the contract says {c.record_count}")
    bad += [f"{n}: no bound in the contract" for n in c.uncovered(recs)]
    produced = PRODUCERS[file](ENGINES[engine], recs)
    skip = set(OPTIONAL.get(engine, ()))
    bad += [b for b in c.check(produced, {k: v for k, v in recs.items() if k not in skip})
            if "no bound in the contract" not in b]
    return bad


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="contract", description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="verb", required=True)
    v = sub.add_parser("verify")
    v.add_argument("--engine", default="both", choices=["python", "native", "both"])
    v.add_argument("--json", action="store_true")
    sub.add_parser("table")
    a = ap.parse_args(argv)
    contracts = load_tolerances()
    if a.verb == "table":
        for c in contracts.values():
            print(f"{c.file}  ({c.precision}, {c.record_count} records)")
            for pat, b in c.rules:
                print(f"   {pat:<28} {b.mode:<9} atol={b.atol:<8g} rtol={b.rtol:<8g} {b.source}")
        return 0
    report, rc = {}, 0
    for file in PRODUCERS:
        for e in (list(ENGINES) if a.engine == "both" else [a.engine]):
            bad = run_fixture(file, e, contracts=contracts)
            report[f"{file}:{e}"] = bad
            rc |= 1 if bad else 0
            if not a.json:
                print(f"{file} [{e}]: " + ("conforms" if not bad else f"{len(bad)} violation(s)"))
                for b in bad[:20]:
                    print("   " + b)
    if a.json:
        print(json.dumps(report, indent=1))
    return rc


if __name__ == "__main__":
    sys.exit(main())
