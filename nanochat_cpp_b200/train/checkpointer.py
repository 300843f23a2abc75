"""Checkpoint save / load in the reference's `NCHKPT01` container (native writer and reader).

Layout and record names follow the reference (`src/train.cc:266-430`, `src/optim.cc:310-329, 801-828`,
docs/checkpoint-format.md): parameter records under their model names (fp32 canonical), then the optimizer
section: `adamw.<kind>.m` / `.v` (the moments of a group concatenated in parameter order),
`muon.<rows>x<cols>.buf1` / `.buf2` (stacked over the matrices of a shape group) and `optimizer/step`.
Rank 0 writes one canonical file whatever the world size; with an owner-sharded optimizer the shards are
gathered first, so a run can resume on a different number of GPUs. The data-loader cursor goes to the
sidecar `<path>.cursor`.
"""
from __future__ import annotations

import os

from typing import Dict, Optional

import numpy as np
import torch

from ..config import Config
from ..data import native
from ..models import GPT
from ..optim import Optimizer

STAGES = {"base": 0, "sft": 1, "rl": 2}
# AdamW group names as they appear in record names (reference src/optim.cc:75-90)
RECORD_KIND = {"wte": "embedding", "value_embed": "value_embedding"}


def _kind(g) -> str:
    return RECORD_KIND.get(g.kind, g.kind)


def _np(t: torch.Tensor) -> np.ndarray:
    return t.detach().to("cpu", torch.float32).contiguous().numpy()


def _gather_state(opt: Optimizer, dp) -> Dict[str, np.ndarray]:
    """Optimizer records (numpy, fp32) for the canonical file; gathers owner shards when `dp` is given."""
    store = opt.store
    out: Dict[str, np.ndarray] = {}

    def full_adamw(spec, key):
        local = opt.state.get(spec.name)
        a, b = opt.adamw_slices.get(spec.name, (0, spec.count))
        buf = torch.zeros(spec.count, dtype=torch.float32, device=store.device)
        if local is not None and b > a:
            buf[a:b] = local[key].view(-1)
        if dp is not None and dp.world_size > 1:
            import torch.distributed as dist
            dist.all_reduce(buf, group=dp.group)
        return buf

    for g in opt.adamw_groups:
        if not g.params:
            continue
        for key in ("m", "v"):
            out[f"adamw.{_kind(g)}.{key}"] = np.concatenate([_np(full_adamw(s, key)) for s in g.params])
    for g in opt.muon_groups:
        lines = g.rows if g.rows >= g.cols else g.cols
        b1, b2 = [], []
        for s in g.params:
            st = opt.state.get(s.name)
            t1 = st["buf1"] if st is not None else torch.zeros(s.shape, dtype=torch.float32, device=store.device)
            t2 = st["buf2"] if st is not None else torch.zeros(lines, dtype=torch.float32, device=store.device)
            if dp is not None and dp.world_size > 1:
                import torch.distributed as dist
                t1, t2 = t1.clone(), t2.clone()
                dist.all_reduce(t1, group=dp.group)
                dist.all_reduce(t2, group=dp.group)
            b1.append(_np(t1))
            b2.append(_np(t2))
        out[f"muon.{g.rows}x{g.cols}.buf1"] = np.stack(b1)
        out[f"muon.{g.rows}x{g.cols}.buf2"] = np.stack(b2)
    out["optimizer/step"] = np.array([float(opt.step_count)], dtype=np.float32)
    return out


def _gather_master(model: GPT, dp) -> torch.Tensor:
    """fp32 master weights of every parameter on every rank (non-owners hold stale masters under sharding)."""
    store = model.params
    if dp is None or dp.world_size == 1:
        return store.master
    import torch.distributed as dist
    buf = torch.zeros_like(store.master)
    for s in store.specs:
        o = dp.owners[s.name]
        if o == dp.rank:
            buf[s.offset:s.offset + s.count] = store.master[s.offset:s.offset + s.count]
        elif o == -1:
            a, b = dp.slices[s.name]
            buf[s.offset + a:s.offset + b] = store.master[s.offset + a:s.offset + b]
    dist.all_reduce(buf, group=dp.group)
    return buf


def save_checkpoint(path: str, model: GPT, optimizer: Optional[Optimizer] = None, *, step: int = 0,
                    stage: str = "base", dp=None, tokenizer_id: str = "", notes: str = "",
                    loader: Optional[native.DataLoader] = None) -> None:
    master = _gather_master(model, dp)
    opt_records = _gather_state(optimizer, dp) if optimizer is not None else {}
    rank = 0 if dp is None else dp.rank
    if rank != 0:
        return
    cfg = model.cfg
    records = []
    for s in model.params.specs:
        records.append((s.name, 0, _np(master[s.offset:s.offset + s.count]).reshape(s.shape)))
    precision = 1 if model.dtype == torch.bfloat16 else 0
    # Both files are written beside their final names and renamed into place, so a run that is stopped in the
    # middle of a save leaves the previous checkpoint and cursor intact.
    final_path, path = path, path + ".tmp"
    native.write_checkpoint(path, records, [(k, 0, v) for k, v in opt_records.items()],
                            config=dict(num_layers=cfg.num_layers, num_heads=cfg.num_heads,
                                        num_kv_heads=cfg.num_kv_heads, hidden_dim=cfg.hidden_dim,
                                        seq_len=cfg.seq_len, vocab_size=cfg.vocab_size,
                                        padded_vocab_size=cfg.padded_vocab_size, rope_base=cfg.rope_base,
                                        window_pattern=cfg.window_pattern, value_embedding=cfg.value_embedding),
                            stage=STAGES[stage], step=step, world_size=1 if dp is None else dp.world_size,
                            precision=precision, tokenizer_id=tokenizer_id, notes=notes)
    if loader is not None:
        loader.save_cursor(final_path + ".cursor.tmp")
    os.replace(path, final_path)
    if loader is not None:
        os.replace(final_path + ".cursor.tmp", final_path + ".cursor")


def config_from_metadata(meta: dict) -> Config:
    c = meta["config"]
    return Config(num_layers=c["num_layers"], num_heads=c["num_heads"], num_kv_heads=c["num_kv_heads"],
                  hidden_dim=c["hidden_dim"], seq_len=c["seq_len"], vocab_size=c["vocab_size"],
                  padded_vocab_size=c["padded_vocab_size"], rope_base=c["rope_base"],
                  window_pattern=c["window_pattern"], value_embedding=bool(c["value_embedding"]))


def infer_config(records, meta: dict) -> Config:
    """Model shape from the record shapes (files written through the plain C ABI carry default metadata)."""
    base = config_from_metadata(meta)
    lm = records["lm_head.weight"][1]
    padded, hidden = lm.shape
    layers = sum(1 for k in records if k.endswith("attn.c_q.weight"))
    q_dim = records["transformer.h.0.attn.c_q.weight"][1].shape[0]
    kv_dim = records["transformer.h.0.attn.c_k.weight"][1].shape[0]
    gates = [k for k in records if k.endswith("attn.ve_gate.weight")]
    if gates:
        kv_heads = records[gates[0]][1].shape[0]
        head_dim = kv_dim // kv_heads
    else:
        head_dim = 128 if q_dim % 128 == 0 else 64 if q_dim % 64 == 0 else base.head_dim
        kv_heads = kv_dim // head_dim
    consistent = (base.hidden_dim == hidden and base.padded_vocab_size == padded and base.num_layers == layers and
                  base.query_dim == q_dim and base.kv_dim == kv_dim)
    if consistent:
        return base
    vocab = base.vocab_size if base.vocab_size <= padded and base.padded_vocab_size == padded else padded
    return Config(num_layers=layers, num_heads=q_dim // head_dim, num_kv_heads=kv_heads, hidden_dim=hidden,
                  seq_len=base.seq_len, vocab_size=vocab, padded_vocab_size=padded, rope_base=base.rope_base,
                  window_pattern=base.window_pattern, value_embedding=bool(gates))


def _decode(code: int, arr: np.ndarray) -> torch.Tensor:
    if code == 1:  # bf16 bit patterns
        return torch.from_numpy((arr.astype(np.uint32) << 16).view(np.float32).copy())
    return torch.from_numpy(np.asarray(arr, dtype=np.float32).copy())


def load_checkpoint(path: str, model: Optional[GPT] = None, optimizer: Optional[Optimizer] = None, *,
                    device="cpu", dtype: torch.dtype = torch.float32, strict_config: bool = True):
    """Loads weights (and optimizer state when `optimizer` is given). Without `model` a new one is built from the
    recorded configuration (version 1 files). Returns (model, metadata)."""
    records, opt_records, meta = native.read_checkpoint(path)
    if model is None:
        model = GPT(infer_config(records, meta), device, dtype, init=False)
    elif strict_config and meta["config"].get("container_version", 1) == 1:
        want = infer_config(records, meta)
        got = model.cfg
        for k in ("num_layers", "num_heads", "num_kv_heads", "hidden_dim", "vocab_size", "padded_vocab_size"):
            if getattr(want, k) != getattr(got, k):
                raise ValueError(f"checkpoint config mismatch on {k}: file {getattr(want, k)} vs model {getattr(got, k)}")
    sd = {}
    for s in model.params.specs:
        if s.name not in records:
            raise KeyError(f"checkpoint has no record {s.name!r}")
        code, arr, _ = records[s.name]
        sd[s.name] = _decode(code, arr).reshape(s.shape)
    model.load_state_dict({k: v.to(model.device) for k, v in sd.items()})
    if optimizer is not None and opt_records:
        _restore_state(optimizer, {k: _decode(c, a) for k, (c, a, _) in opt_records.items()})
    return model, meta


def _restore_state(opt: Optimizer, recs: Dict[str, torch.Tensor]) -> None:
    dev = opt.store.device
    for g in opt.adamw_groups:
        for key in ("m", "v"):
            name = f"adamw.{_kind(g)}.{key}"
            if name not in recs:
                continue
            flat = recs[name].reshape(-1)
            off = 0
            for s in g.params:
                a, b = opt.adamw_slices.get(s.name, (0, s.count))
                if s.name in opt.state and b > a:
                    opt.state[s.name][key].view(-1).copy_(flat[off + a:off + b].to(dev))
                off += s.count
    for g in opt.muon_groups:
        n1, n2 = f"muon.{g.rows}x{g.cols}.buf1", f"muon.{g.rows}x{g.cols}.buf2"
        P = len(g.params)
        b1 = recs[n1].reshape(P, g.rows, g.cols) if n1 in recs else None
        b2 = recs[n2].reshape(P, -1) if n2 in recs else None
        for k, s in enumerate(g.params):
            if s.name in opt.state:
                if b1 is not None:
                    opt.state[s.name]["buf1"].copy_(b1[k].to(dev))
                if b2 is not None:
                    opt.state[s.name]["buf2"].copy_(b2[k].to(dev))
    if "optimizer/step" in recs:
        opt.step_count = int(recs["optimizer/step"].reshape(-1)[0].item())
