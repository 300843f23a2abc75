"""Parameter storage: one flat fp32 master, one flat compute copy, one flat gradient.

Registration order and names follow the reference graph (`src/model.cc:213-339`):
`lm_head.weight`, `transformer.wte.weight`, `value_embeds.<i>.weight` for every
layer that carries one, `resid_lambdas`, `x0_lambdas`, `smear_gate.weight`,
`smear_lambda`, `backout_lambda`, then per block `attn.c_q/c_k/c_v/c_proj`,
`attn.ve_gate` (when present), `mlp.c_fc`, `mlp.c_proj`.

Flat storage is what the data-parallel path wants: gradients of a bucket are one
contiguous span, owner shards are slices, and the optimizer kernels walk spans
instead of Python lists of tensors. `c_q`, `c_k`, `c_v` of a block are adjacent, so
one `[q_dim + 2*kv_dim, hidden]` view serves a single fused QKV GEMM.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from ..config import SMEAR_CHANNELS, VE_GATE_CHANNELS, Config

ALIGN = 64  # elements; keeps every bf16 parameter 128-byte aligned for TMA


@dataclass
class ParamSpec:
    name: str
    shape: Tuple[int, ...]
    rows: int  # 0 for scalars/vectors (reference ParamView.rows/cols)
    cols: int
    kind: str  # lm_head | wte | value_embed | resid | x0 | smear | matrix
    offset: int = 0
    layer: int = -1

    @property
    def count(self) -> int:
        return int(math.prod(self.shape))


def param_specs(cfg: Config) -> List[ParamSpec]:
    L, C = cfg.num_layers, cfg.hidden_dim
    V = cfg.padded_vocab_size
    specs: List[ParamSpec] = [
        ParamSpec("lm_head.weight", (V, C), V, C, "lm_head"),
        ParamSpec("transformer.wte.weight", (V, C), V, C, "wte"),
    ]
    for i in range(L):
        if cfg.has_value_embedding(i):
            specs.append(ParamSpec(f"value_embeds.{i}.weight", (V, cfg.kv_dim), V, cfg.kv_dim,
                                   "value_embed", layer=i))
    specs += [
        ParamSpec("resid_lambdas", (L,), 0, 0, "resid"),
        ParamSpec("x0_lambdas", (L,), 0, 0, "x0"),
        ParamSpec("smear_gate.weight", (1, SMEAR_CHANNELS), 1, SMEAR_CHANNELS, "smear"),
        ParamSpec("smear_lambda", (1,), 0, 0, "smear"),
        ParamSpec("backout_lambda", (1,), 0, 0, "smear"),
    ]
    for i in range(L):
        p = f"transformer.h.{i}."
        specs.append(ParamSpec(p + "attn.c_q.weight", (cfg.query_dim, C), cfg.query_dim, C, "matrix", layer=i))
        specs.append(ParamSpec(p + "attn.c_k.weight", (cfg.kv_dim, C), cfg.kv_dim, C, "matrix", layer=i))
        specs.append(ParamSpec(p + "attn.c_v.weight", (cfg.kv_dim, C), cfg.kv_dim, C, "matrix", layer=i))
        specs.append(ParamSpec(p + "attn.c_proj.weight", (C, C), C, C, "matrix", layer=i))
        if cfg.has_value_embedding(i):
            specs.append(ParamSpec(p + "attn.ve_gate.weight", (cfg.num_kv_heads, VE_GATE_CHANNELS),
                                   cfg.num_kv_heads, VE_GATE_CHANNELS, "matrix", layer=i))
        specs.append(ParamSpec(p + "mlp.c_fc.weight", (cfg.mlp_dim, C), cfg.mlp_dim, C, "matrix", layer=i))
        specs.append(ParamSpec(p + "mlp.c_proj.weight", (C, cfg.mlp_dim), C, cfg.mlp_dim, "matrix", layer=i))
    off = 0
    for s in specs:
        s.offset = off
        off += ((s.count + ALIGN - 1) // ALIGN) * ALIGN
    return specs


class ParamStore:
    """Flat buffers plus named views. `value` aliases `master` when the compute dtype is fp32."""

    def __init__(self, cfg: Config, device, dtype: torch.dtype = torch.bfloat16,
                 grad_dtype: torch.dtype = torch.float32, allocator=None):
        """`allocator(numel, dtype) -> zeroed 1-D tensor` lets the data-parallel engine place the gradient
        and the compute copy in symmetric (peer-mapped) memory."""
        self.cfg = cfg
        self.device = torch.device(device)
        self.dtype = dtype
        self.specs = param_specs(cfg)
        last = self.specs[-1]
        self.total = last.offset + ((last.count + ALIGN - 1) // ALIGN) * ALIGN
        self.master = torch.zeros(self.total, dtype=torch.float32, device=self.device)
        alloc = allocator or (lambda n, dt: torch.zeros(n, dtype=dt, device=self.device))
        self.value = self.master if dtype == torch.float32 else alloc(self.total, dtype)
        self.grad = alloc(self.total, grad_dtype)
        self.by_name: Dict[str, ParamSpec] = {s.name: s for s in self.specs}
        self._v: Dict[str, torch.Tensor] = {}
        self._g: Dict[str, torch.Tensor] = {}
        self._m: Dict[str, torch.Tensor] = {}
        for s in self.specs:
            sl = slice(s.offset, s.offset + s.count)
            self._v[s.name] = self.value[sl].view(s.shape)
            self._g[s.name] = self.grad[sl].view(s.shape)
            self._m[s.name] = self.master[sl].view(s.shape)

    # named access -------------------------------------------------------
    def v(self, name: str) -> torch.Tensor:
        return self._v[name]

    def g(self, name: str) -> torch.Tensor:
        return self._g[name]

    def m(self, name: str) -> torch.Tensor:
        return self._m[name]

    def names(self) -> List[str]:
        return [s.name for s in self.specs]

    def qkv_view(self, layer: int, which: str = "v") -> Optional[torch.Tensor]:
        """[q_dim+2*kv_dim, hidden] view over c_q|c_k|c_v of `layer`, or None when padding
        separates them."""
        cfg = self.cfg
        sq = self.by_name[f"transformer.h.{layer}.attn.c_q.weight"]
        sk = self.by_name[f"transformer.h.{layer}.attn.c_k.weight"]
        sv = self.by_name[f"transformer.h.{layer}.attn.c_v.weight"]
        if sk.offset != sq.offset + sq.count or sv.offset != sk.offset + sk.count:
            return None
        buf = {"v": self.value, "g": self.grad, "m": self.master}[which]
        n = cfg.query_dim + 2 * cfg.kv_dim
        return buf[sq.offset: sq.offset + n * cfg.hidden_dim].view(n, cfg.hidden_dim)

    def sync_compute(self) -> None:
        """Refresh the compute copy from the fp32 master."""
        if self.value is not self.master:
            self.value.copy_(self.master)

    def zero_grad(self) -> None:
        self.grad.zero_()

    def num_params(self) -> int:
        return sum(s.count for s in self.specs)


# ---------------------------------------------------------------------------
# Initialisation. The distributions are the reference's (`src/model.cc:427-497`):
# wte N(0, 0.8), lm_head N(0, 0.001), s = sqrt(3)/sqrt(hidden), c_q/c_k/c_v U(-s, s),
# both c_proj 0, c_fc U(-0.4s, 0.4s), resid 1.15 - 0.10 i/(L-1), x0 0.20 - 0.15 i/(L-1),
# smear_lambda 0, backout 0.2, smear_gate / ve_gate U(0, 0.02), value_embeds U(-s, s).
# The stream is torch's Philox generator seeded per parameter, not the reference's
# xorshift64*: bit-equal weights are obtained by loading a checkpoint instead.
# ---------------------------------------------------------------------------
def init_weights(store: ParamStore, seed: int = 0) -> None:
    cfg = store.cfg
    C, L = cfg.hidden_dim, cfg.num_layers
    s = math.sqrt(3.0) / math.sqrt(float(C))
    denom = float(max(L - 1, 1))
    dev = store.device
    gen = torch.Generator(device="cpu")

    def normal(t, std, k):
        gen.manual_seed(seed * 1000003 + k)
        chunk = 1 << 24
        flat = t.view(-1)
        for a in range(0, flat.numel(), chunk):
            b = min(a + chunk, flat.numel())
            flat[a:b] = (torch.randn(b - a, generator=gen, dtype=torch.float32) * std).to(dev)

    def uniform(t, lo, hi, k):
        gen.manual_seed(seed * 1000003 + k)
        chunk = 1 << 24
        flat = t.view(-1)
        for a in range(0, flat.numel(), chunk):
            b = min(a + chunk, flat.numel())
            flat[a:b] = (torch.rand(b - a, generator=gen, dtype=torch.float32) * (hi - lo) + lo).to(dev)

    store.master.zero_()
    for k, sp in enumerate(store.specs):
        t = store.m(sp.name)
        n = sp.name
        if n == "transformer.wte.weight":
            normal(t, 0.8, k)
        elif n == "lm_head.weight":
            normal(t, 0.001, k)
        elif n.startswith("value_embeds."):
            uniform(t, -s, s, k)
        elif n == "resid_lambdas":
            t.copy_(torch.tensor([1.15 - 0.10 * i / denom for i in range(L)], dtype=torch.float32))
        elif n == "x0_lambdas":
            t.copy_(torch.tensor([0.20 - 0.15 * i / denom for i in range(L)], dtype=torch.float32))
        elif n == "smear_gate.weight" or n.endswith("ve_gate.weight"):
            uniform(t, 0.0, 0.02, k)
        elif n == "smear_lambda":
            t.fill_(0.0)
        elif n == "backout_lambda":
            t.fill_(0.2)
        elif n.endswith("c_q.weight") or n.endswith("c_k.weight") or n.endswith("c_v.weight"):
            uniform(t, -s, s, k)
        elif n.endswith("c_fc.weight"):
            uniform(t, -0.4 * s, 0.4 * s, k)
        elif n.endswith("c_proj.weight"):
            t.zero_()
        else:
            raise AssertionError(n)
    store.sync_compute()
