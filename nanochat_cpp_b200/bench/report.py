"""`nanochat.bench.v3` documents: the report every micro-benchmark can write besides its own lines.

One document per benchmark run: device, precision, the peak rate used as the MFU denominator, and one row per
measured feature with the join identity (family, phase, precision) that the attainment report matches against
`nanochat.roofline.v3` rows. Field names and their order follow the reference's writer
(include/nanochat/bench.h:84-109, 230-274) so that a reader of either tree's reports needs one parser.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Dict, List, Optional

SCHEMA = "nanochat.bench.v3"
ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def measured_peak_flops(precision: str = "bf16", sustained: bool = False) -> float:
    """Dense FLOP/s measured on this machine's GPU (cuBLAS, `MEASURED_PEAKS.json`), 0 when no measurement exists.
    fp8 has no measured figure: twice the bf16 one is used, as the hardware's nominal ratio."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if not os.path.exists(path):
        return 0.0
    peaks = json.load(open(path))
    tf = float(peaks.get("bf16_tflops_sustained" if sustained else "bf16_tflops", 0.0))
    return tf * 1e12 * (2.0 if precision.startswith("fp8") else 1.0)


@dataclass
class BenchRow:
    name: str
    shape: str
    ms: float
    gflops: float = 0.0          # achieved GFLOP/s over the necessary operation count
    work_ratio: float = 0.0      # issued / necessary work, 0 = not reported
    mfu: float = 0.0             # share of the report's peak rate, filled by the report
    family: str = ""
    phase: str = ""
    precision: str = ""
    iterations: int = 0
    occupancy: int = 0


class BenchReport:
    def __init__(self, device: str = "", precision: str = "", peak_flops: float = 0.0):
        self.device, self.precision, self.peak_flops = device, precision, float(peak_flops)
        self.family, self.phase = "", ""
        self.rows: List[BenchRow] = []
        self.extras: Dict[str, object] = {}

    def use_device_peak(self, precision: str = "bf16", sustained: bool = False) -> "BenchReport":
        import torch
        self.precision = precision
        if torch.cuda.is_available():
            self.device = torch.cuda.get_device_name(torch.cuda.current_device())
        self.peak_flops = measured_peak_flops(precision, sustained)
        return self

    def set_row_identity(self, family: str, phase: str) -> None:
        self.family, self.phase = family, phase

    def add(self, name: str, shape: str, ms: float, gflops: float = 0.0, work_ratio: float = 0.0,
            iterations: int = 0, occupancy: int = 0, family: Optional[str] = None, phase: Optional[str] = None,
            precision: Optional[str] = None) -> BenchRow:
        row = BenchRow(name, shape, float(ms), float(gflops), float(work_ratio), 0.0,
                       self.family if family is None else family, self.phase if phase is None else phase,
                       self.precision if precision is None else precision, int(iterations), int(occupancy))
        self.rows.append(row)
        return row

    def _mfu(self, gflops: float) -> float:
        if self.peak_flops <= 0.0 or gflops <= 0.0:
            return 0.0
        return min(1.0, gflops * 1e9 / self.peak_flops)

    def document(self) -> dict:
        doc: Dict[str, object] = {"schema": SCHEMA}
        if self.device:
            doc["device"] = self.device
        if self.precision:
            doc["precision"] = self.precision
        if self.peak_flops > 0.0:
            doc["peak_flops"] = self.peak_flops
        rows = []
        for r in self.rows:
            d: Dict[str, object] = {"name": r.name}
            for key in ("family", "phase", "precision"):
                if getattr(r, key):
                    d[key] = getattr(r, key)
            d.update(shape=r.shape, ms=r.ms, gflops=r.gflops, work_ratio=r.work_ratio, mfu=self._mfu(r.gflops))
            if r.iterations > 0:
                d["iterations"] = r.iterations
            if r.occupancy > 0:
                d["occupancy"] = r.occupancy
            rows.append(d)
        doc["rows"] = rows
        doc.update(self.extras)
        return doc

    def json(self) -> str:
        return json.dumps(self.document(), separators=(",", ":"))

    def write(self, path: str) -> None:
        with open(path, "w") as f:
            f.write(self.json() + "\n")

    def table(self) -> str:
        lines = [f"{'name':32s} {'shape':34s} {'ms':>10s} {'GFLOP/s':>12s} {'mfu':>6s}"]
        for d in self.document()["rows"]:
            lines.append(f"{d['name']:32s} {d['shape']:34s} {d['ms']:10.4f} {d['gflops']:12.1f} {d['mfu']:6.3f}")
        return "\n".join(lines)


def join_with_roofline(bench_doc: dict, roofline_doc: dict) -> List[dict]:
    """Rows of a bench document matched with roofline rows on (family, phase): measured ms, bound ms and their ratio
    (the attainment of that family); bench rows without identity, or without a partner, take part in no join."""
    bounds = {(r.get("family"), r.get("phase")): r for r in roofline_doc.get("rows", [])}
    out = []
    for r in bench_doc.get("rows", []):
        key = (r.get("family"), r.get("phase"))
        b = bounds.get(key)
        if not r.get("family") or b is None:
            continue
        bound_ms = float(b.get("bound_ms", b.get("ms", 0.0)))
        out.append({"family": key[0], "phase": key[1], "name": r["name"], "measured_ms": r["ms"], "bound_ms": bound_ms,
                    "attainment": (bound_ms / r["ms"]) if r["ms"] > 0 and bound_ms > 0 else 0.0})
    return out
