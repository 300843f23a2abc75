"""Checkpoint conversion between an upstream PyTorch nanochat `state_dict` and the `NCHKPT01` container.

Upstream saves `model_<step>.pt` (a state_dict whose keys carry the names this engine uses:
`transformer.wte.weight`, `transformer.h.<i>.attn.c_q.weight`, `value_embeds.<i>.weight`, `lm_head.weight`,
`resid_lambdas`, `x0_lambdas`, ...) possibly prefixed by `_orig_mod.` from torch.compile. The reference converts with
python/nanochat_cpp/checkpoint.py and nanochat_cpp_bridge/torch_checkpoint.py; this module does both directions.

    python -m nanochat_cpp_b200.train.convert model_000650.pt base.ckpt
    python -m nanochat_cpp_b200.train.convert base.ckpt model.pt --to-torch
"""
from __future__ import annotations

import argparse
from typing import Dict

import numpy as np
import torch

from ..config import Config
from ..data import native
from ..models.params import param_specs

PREFIXES = ("_orig_mod.", "module.")


def clean_names(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    out = {}
    for k, v in sd.items():
        for p in PREFIXES:
            while k.startswith(p):
                k = k[len(p):]
        out[k] = v
    return out


def config_from_state_dict(sd: Dict[str, torch.Tensor], seq_len: int = 2048, head_dim: int = 128,
                           window_pattern: str = "SSSL", vocab_size: int = 0) -> Config:
    padded, hidden = sd["lm_head.weight"].shape
    layers = sum(1 for k in sd if k.endswith("attn.c_q.weight"))
    q_dim = sd["transformer.h.0.attn.c_q.weight"].shape[0]
    kv_dim = sd["transformer.h.0.attn.c_k.weight"].shape[0]
    gates = [k for k in sd if k.endswith("attn.ve_gate.weight")]
    kv_heads = sd[gates[0]].shape[0] if gates else max(1, kv_dim // head_dim)
    hd = kv_dim // kv_heads
    return Config(num_layers=layers, num_heads=q_dim // hd, num_kv_heads=kv_heads, hidden_dim=hidden, seq_len=seq_len,
                  vocab_size=vocab_size or padded, padded_vocab_size=padded, window_pattern=window_pattern,
                  value_embedding=bool(gates))


def torch_to_container(pt_path: str, out_path: str, *, step: int = 0, stage: int = 0, **config_kw) -> Config:
    sd = torch.load(pt_path, map_location="cpu", weights_only=True)
    if "model" in sd and isinstance(sd["model"], dict):
        sd = sd["model"]
    sd = clean_names(sd)
    cfg = config_from_state_dict(sd, **config_kw)
    records = []
    for s in param_specs(cfg):
        if s.name not in sd:
            raise KeyError(f"the state_dict has no tensor {s.name!r}")
        t = sd[s.name].detach().to(torch.float32).reshape(s.shape).contiguous().numpy()
        records.append((s.name, 0, t))
    native.write_checkpoint(out_path, records, [], config=dict(
        num_layers=cfg.num_layers, num_heads=cfg.num_heads, num_kv_heads=cfg.num_kv_heads, hidden_dim=cfg.hidden_dim,
        seq_len=cfg.seq_len, vocab_size=cfg.vocab_size, padded_vocab_size=cfg.padded_vocab_size,
        rope_base=cfg.rope_base, window_pattern=cfg.window_pattern, value_embedding=cfg.value_embedding),
        stage=stage, step=step, world_size=1, precision=0, notes="converted from a PyTorch state_dict")
    return cfg


def container_to_torch(ckpt_path: str, out_path: str) -> None:
    records, _, _ = native.read_checkpoint(ckpt_path)
    sd = {}
    for name, (code, arr, _) in records.items():
        if code == 1:
            arr = (arr.astype(np.uint32) << 16).view(np.float32)
        sd[name] = torch.from_numpy(np.asarray(arr, dtype=np.float32).copy())
    torch.save(sd, out_path)


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("src")
    ap.add_argument("dst")
    ap.add_argument("--to-torch", action="store_true")
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--vocab-size", type=int, default=0)
    ap.add_argument("--window-pattern", default="SSSL")
    a = ap.parse_args()
    if a.to_torch:
        container_to_torch(a.src, a.dst)
    else:
        cfg = torch_to_container(a.src, a.dst, seq_len=a.seq_len, vocab_size=a.vocab_size,
                                 window_pattern=a.window_pattern)
        print(f"converted {cfg.num_layers} layers, hidden {cfg.hidden_dim}, vocab {cfg.vocab_size}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
