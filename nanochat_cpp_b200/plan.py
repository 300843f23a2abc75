"""Model specification, device profile and the planner that maps one onto the other.

The reference keeps three small contracts apart (include/nanochat/model_spec.h, device_profile.h, plan.h): a closed
JSON description of the model's blocks, a per-device declaration of capabilities and rates, and a pure function that
decides, per operation family, whether the device's fused kernel or the composition of primitive operators runs.
Same split here: `ModelSpec` (strict reader: unknown keys and unknown block kinds are errors), `DeviceProfile`
(`caps/*.json`; the B200 rates are replaced by the measured ones when `MEASURED_PEAKS.json` exists) and
`build_plan`. The plan is what `ops` executes: "kernel" rows run `ops.cuda`, "composition" rows run `ops.ref`.
"""
from __future__ import annotations

import glob
import json
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

from .config import Config

_HERE = os.path.dirname(os.path.abspath(__file__))

BLOCK_KEYS = {"norm", "attention", "attention_variant", "position", "mlp", "residual", "dtype", "value_embedding"}
BLOCK_VOCAB = {"norm": {"rms_norm"}, "attention": {"causal", "sliding_window"},
               "attention_variant": {"mha", "gqa"}, "position": {"rope"}, "mlp": {"relu_square"},
               "residual": {"blend"}, "dtype": {"build_default", "fp32", "bf16", "fp8"}}
SPEC_KEYS = {"spec_version", "name", "requires", "dimensions", "blocks", "head", "embedding", "backout_layer"}
DIM_KEYS = {"num_heads", "num_kv_heads", "hidden_dim", "seq_len", "rope_base", "vocab_size", "padded_vocab_size"}


class SpecError(ValueError):
    pass


@dataclass
class ModelSpec:
    name: str
    requires: List[str]
    dimensions: Dict[str, float]
    blocks: List[Dict[str, object]]
    head: Dict[str, object] = field(default_factory=dict)
    embedding: Dict[str, object] = field(default_factory=dict)
    backout_layer: Optional[int] = None

    @classmethod
    def from_json(cls, source) -> "ModelSpec":
        d = json.load(open(source)) if isinstance(source, (str, os.PathLike)) else dict(source)
        extra = set(d) - SPEC_KEYS
        if extra:
            raise SpecError(f"unknown spec keys: {sorted(extra)}")
        if d.get("spec_version") != 1:
            raise SpecError(f"unsupported spec_version {d.get('spec_version')!r}")
        for k in ("name", "dimensions", "blocks"):
            if k not in d:
                raise SpecError(f"spec lacks {k!r}")
        extra = set(d["dimensions"]) - DIM_KEYS
        if extra:
            raise SpecError(f"unknown dimension keys: {sorted(extra)}")
        if not d["blocks"]:
            raise SpecError("a model needs at least one block")
        for i, b in enumerate(d["blocks"]):
            extra = set(b) - BLOCK_KEYS
            if extra:
                raise SpecError(f"block {i}: unknown keys {sorted(extra)}")
            for key, allowed in BLOCK_VOCAB.items():
                if key in b and b[key] not in allowed:
                    raise SpecError(f"block {i}: {key} = {b[key]!r} is not one of {sorted(allowed)}")
        return cls(d["name"], list(d.get("requires", [])), dict(d["dimensions"]), [dict(b) for b in d["blocks"]],
                   dict(d.get("head", {})), dict(d.get("embedding", {})), d.get("backout_layer"))

    @classmethod
    def default(cls) -> "ModelSpec":
        return cls.from_json(os.path.join(_HERE, "model_specs", "nanochat-default.json"))

    def to_config(self) -> Config:
        dm = self.dimensions
        pattern = "".join("S" if b.get("attention") == "sliding_window" else "L" for b in self.blocks)
        # the shortest repeating prefix describes the pattern (the last layer is always full context)
        body = pattern[:-1] + ("L" if pattern[-1] == "L" else pattern[-1])
        period = next((p for p in range(1, len(body) + 1)
                       if all(body[i] == body[i % p] for i in range(len(body) - 1))), len(body))
        vocab = int(dm.get("vocab_size", 32768))
        return Config(num_layers=len(self.blocks), num_heads=int(dm["num_heads"]),
                      num_kv_heads=int(dm.get("num_kv_heads", dm["num_heads"])), hidden_dim=int(dm["hidden_dim"]),
                      seq_len=int(dm.get("seq_len", 2048)), vocab_size=vocab,
                      padded_vocab_size=int(dm.get("padded_vocab_size", (vocab + 63) // 64 * 64)),
                      rope_base=float(dm.get("rope_base", 100000.0)), window_pattern=body[:period],
                      value_embedding=any(b.get("value_embedding") for b in self.blocks))


@dataclass
class DeviceProfile:
    device: str
    match: List[str]
    features: List[str]
    precisions: List[str]
    peaks: Dict[str, float]
    raw: Dict[str, object] = field(default_factory=dict)

    def has(self, feature: str) -> bool:
        return feature in self.features


def device_profiles() -> Dict[str, DeviceProfile]:
    out = {}
    for path in sorted(glob.glob(os.path.join(_HERE, "caps", "*.json"))):
        d = json.load(open(path))
        peaks = {k: v for k, v in d.get("peaks", {}).items() if isinstance(v, (int, float))}
        if d["device"] == "b200":
            from .train.mfu import measured_peaks
            m = measured_peaks()
            if m.get("source") == "measured":
                peaks.update(bf16_flops=m["bf16_tflops"] * 1e12, fp8_flops=2 * m["bf16_tflops"] * 1e12,
                             hbm_bytes_per_s=m["hbm_gbs"] * 1e9)
        out[d["device"]] = DeviceProfile(d["device"], d.get("match", []), d.get("features", []),
                                         d.get("precisions", []), peaks, d)
    return out


def profile_for(device_name: str) -> DeviceProfile:
    """Profile whose `match` strings occur in the device name (e.g. "NVIDIA B200"); falls back to cpu."""
    profs = device_profiles()
    for p in profs.values():
        if any(m.lower() in device_name.lower() for m in p.match):
            return p
    return profs["cpu"]


# operation family -> (feature that grants the fused kernel, kernel name)
FAMILIES = [
    ("linear", "fused_gemm_epilogue", "gemm_tcgen05 (pair tiles, fused residual / relu^2 / accumulate epilogues)"),
    ("blend_rms_norm", "fused_blend_rms_norm", "rowops.blend_norm"),
    ("qk_prep", "fused_qk_prep", "rowops.qk_prep (norm + rope + scale, q and k in one launch)"),
    ("attention_forward", "fused_attention_forward", "attention_fwd2 (tcgen05 flash, window-aware)"),
    ("attention_backward", "fused_attention_backward", "attention_bwd (dQ and dK/dV kernels)"),
    ("classifier", "fused_classifier", "rowops.classifier_smem (softcap + CE forward/backward in place)"),
    ("muon", "fused_muon", "optim.muon_* + batched tcgen05 Newton-Schulz"),
    ("adamw", "fused_adamw", "optim.adamw / comm.adamw_push"),
    ("decode_attention", "paged_kv_decode", "decode.paged_decode (split-KV)"),
    ("gradient_sync", "peer_reduce_scatter", "comm.grad_push + grad_reduce_local + update-and-push"),
]


@dataclass
class PlanRow:
    family: str
    choice: str      # "kernel" | "composition"
    detail: str


@dataclass
class Plan:
    model: str
    device: str
    precision: str
    rows: List[PlanRow]

    def line(self) -> str:
        k = sum(r.choice == "kernel" for r in self.rows)
        return f"[nanochat] plan {self.model} on {self.device} ({self.precision}): {k} fused families, " \
               f"{len(self.rows) - k} compositions"


def build_plan(spec: ModelSpec, profile: DeviceProfile, precision: str = "bf16", graph: str = "train") -> Plan:
    missing = [r for r in spec.requires if not profile.has(r)]
    if missing:
        raise SpecError(f"device {profile.device} lacks required capabilities {missing}")
    if precision not in profile.precisions and not (precision == "fp8" and "fp8_e4m3" in profile.precisions):
        raise SpecError(f"device {profile.device} does not run {precision}")
    rows = []
    for family, feature, kernel in FAMILIES:
        if graph in ("prefill", "decode", "generate", "eval") and family in ("attention_backward", "muon", "adamw",
                                                                               "gradient_sync"):
            continue
        if graph == "train" and family == "decode_attention":
            continue
        rows.append(PlanRow(family, "kernel", kernel) if profile.has(feature)
                    else PlanRow(family, "composition", "PyTorch operators of ops.ref"))
    return Plan(spec.name, profile.device, precision, rows)


# ---------------------------------------------------------------------------------------------------------
# Native planning layer (csrc/host/plan.cc, behind the C ABI): the same operator plan computed in C++, and the
# training-run plan (horizon, batch size, learning-rate and weight-decay scaling for a depth).
# ---------------------------------------------------------------------------------------------------------
def _native_text(call) -> str:
    import ctypes
    from .data import native
    lib = native.lib()
    buf = ctypes.create_string_buffer(1 << 16)
    n = call(lib, buf, len(buf))
    if n < 0:
        lib.nanochat_last_error.restype = ctypes.c_char_p
        raise SpecError(lib.nanochat_last_error().decode())
    return buf.value.decode()


def build_plan_native(spec_path: Optional[str] = None, caps_path: Optional[str] = None, precision: str = "bf16",
                      graph: str = "train") -> Plan:
    """`build_plan` through `ncb_plan_json`: the C++ reader and planner on the same two JSON files."""
    import ctypes
    spec_path = spec_path or os.path.join(_HERE, "model_specs", "nanochat-default.json")
    caps_path = caps_path or os.path.join(_HERE, "caps", "b200.json")

    def call(lib, buf, cap):
        lib.ncb_plan_json.restype = ctypes.c_int64
        lib.ncb_plan_json.argtypes = [ctypes.c_char_p] * 4 + [ctypes.c_char_p, ctypes.c_int64]
        return lib.ncb_plan_json(spec_path.encode(), caps_path.encode(), precision.encode(), graph.encode(), buf, cap)
    d = json.loads(_native_text(call))
    return Plan(d["model"], d["device"], d["precision"], [PlanRow(r["family"], r["choice"], r["detail"]) for r in d["rows"]])


def compute_plan(depth: int, *, vocab_size: int, device_batch_size: int, aspect_ratio: int = 64, head_dim: int = 128,
                 seq_len: int = 2048, window_pattern: str = "SSSL", total_batch_size: int = -1, num_iterations: int = 0,
                 target_flops: float = 0.0, target_param_data_ratio: int = 12) -> dict:
    """Training-run plan of a depth (reference python/nanochat_cpp/plan.py `compute_plan`, which mirrors upstream
    `scripts/base_train.py`): the model shape, the parameter counts, and from them the token horizon
    (`target_param_data_ratio` x scaling parameters), the batch size (power of two nearest to 2^19 x (tokens /
    tokens at depth 12)^0.383 unless given), the sqrt batch scaling of the learning rates, the weight decay
    scaled by sqrt(batch ratio) x (depth-12 tokens / tokens), the iteration count and the gradient accumulation.
    Computed natively (`ncb_train_plan_json`); returns the decoded document (`counts`, `flops_per_token`, `config`,
    `inputs`, `plan`)."""
    import ctypes

    def call(lib, buf, cap):
        lib.ncb_train_plan_json.restype = ctypes.c_int64
        lib.ncb_train_plan_json.argtypes = [ctypes.c_int] * 6 + [ctypes.c_char_p, ctypes.c_int64, ctypes.c_int64,
                                                                 ctypes.c_double, ctypes.c_int, ctypes.c_char_p,
                                                                 ctypes.c_int64]
        return lib.ncb_train_plan_json(depth, aspect_ratio, head_dim, seq_len, vocab_size, device_batch_size,
                                       window_pattern.encode(), int(total_batch_size), int(num_iterations),
                                       float(target_flops), target_param_data_ratio, buf, cap)
    return json.loads(_native_text(call))
