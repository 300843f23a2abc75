"""Operator entry points used by the model, the optimizer and the inference engine.

Every operator has two implementations with one signature:

* `ops.ref`  - plain PyTorch, the numerical definition, and the path for CPU tensors;
* `ops.cuda` - the hand-written sm_100a kernels of `csrc/cuda`, the path for CUDA tensors.

A CUDA tensor never falls back silently: if the extension is not built, the first call
raises. Setting `NANOCHAT_B200_OPS=torch` routes CUDA tensors through `ops.ref` (cuBLAS and
eager PyTorch); that arm exists only so benchmarks and tests can compare against it.
"""
from __future__ import annotations

import os
from typing import Callable

import torch

from . import ref

_MODE = os.environ.get("NANOCHAT_B200_OPS", "kernels")


def set_mode(mode: str) -> None:
    """`kernels` (default) or `torch` (comparison arm)."""
    global _MODE
    if mode not in ("kernels", "torch"):
        raise ValueError(mode)
    _MODE = mode


def get_mode() -> str:
    return _MODE


_cuda_mod = None


def cuda_module():
    """The module wrapping the compiled extension; raises if it cannot be loaded."""
    global _cuda_mod
    if _cuda_mod is None:
        from . import cuda as _c  # noqa: WPS433  (import here: needs the built .so)
        _cuda_mod = _c
    return _cuda_mod


def _first_tensor(args, kwargs):
    """The tensor that decides where an operator runs; looks inside list / tuple arguments too (gradient lists)."""
    for a in list(args) + list(kwargs.values()):
        if isinstance(a, torch.Tensor):
            return a
        if isinstance(a, (list, tuple)):
            for b in a:
                if isinstance(b, torch.Tensor):
                    return b
    return None


class OpProfile:
    """Per-operator device time, measured with CUDA events around every operator call.

    `with ops.profile() as prof: step()` then `prof.table()` gives milliseconds and call counts per
    operator. Events are recorded on the current stream, so the numbers are what the stream spent
    between the two records (launch gaps included)."""

    def __init__(self):
        self.events = []

    def __enter__(self):
        global _PROFILE
        _PROFILE = self
        return self

    def __exit__(self, *exc):
        global _PROFILE
        _PROFILE = None

    def table(self):
        torch.cuda.synchronize()
        agg = {}
        for name, a, b in self.events:
            ms = a.elapsed_time(b)
            t = agg.setdefault(name, [0.0, 0])
            t[0] += ms
            t[1] += 1
        return sorted(((k, v[0], v[1]) for k, v in agg.items()), key=lambda r: -r[1])


_PROFILE = None


def profile() -> OpProfile:
    return OpProfile()


def _dispatch(name: str) -> Callable:
    ref_fn = getattr(ref, name)

    def fn(*args, **kwargs):
        t = _first_tensor(args, kwargs)
        if t is not None and t.is_cuda and _MODE == "kernels":
            impl = getattr(cuda_module(), name)
            if _PROFILE is not None:
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                out = impl(*args, **kwargs)
                b.record()
                _PROFILE.events.append((name, a, b))
                return out
            return impl(*args, **kwargs)
        return ref_fn(*args, **kwargs)

    fn.__name__ = name
    fn.__doc__ = ref_fn.__doc__
    return fn


_NAMES = [
    "linear_fwd", "linear_relu2_fwd", "linear_relu2_act_fwd", "linear_dgrad_relu2_act", "linear_dgrad", "linear_dgrad_relu2", "linear_wgrad",
    "linear_wgrad_relu2", "rmsnorm_fwd", "rmsnorm_apply", "rmsnorm_bwd", "add", "add_cols", "concat_qkv",
    "backout_fwd", "backout_bwd", "blend_norm_fwd", "blend_bwd", "norm_blend_bwd", "qk_prep_fwd", "qk_prep_bwd",
    "attention_fwd", "attention_bwd", "value_gate_fwd", "value_gate_bwd", "smear_fwd", "smear_bwd",
    "embedding_fwd", "embedding_bwd", "embedding_order", "classifier_fwd_bwd", "adamw_update", "muon_update",
    "grad_norm_and_clip", "kv_append", "paged_decode_attention", "quantize_fp8", "gemm_scaled_fp8",
]
for _n in _NAMES:
    globals()[_n] = _dispatch(_n)

build_rope = ref.build_rope
paged_gather = ref.paged_gather

__all__ = _NAMES + ["profile", "OpProfile", "build_rope", "ref", "set_mode", "get_mode", "cuda_module"]
