"""A straight autograd statement of the nanochat graph, used as the test oracle.

It shares no code with `models.gpt` beyond the parameter names: the forward below is
written with ordinary differentiable PyTorch operations, and gradients come from
`torch.autograd`. Tests compare the hand-written backward of `models.gpt.GPT` against
it, and the upstream-PyTorch fixtures (`tests/data/debug_state.bin`) pin both.
Graph definition: reference `src/model.cc:894-1003` and `src/ops.cc:1454-1564`.
"""
from __future__ import annotations

import math
from typing import Dict

import torch
import torch.nn.functional as F

from ..config import LOGIT_SOFTCAP, QK_SCALE, RMS_EPS, SMEAR_CHANNELS, VE_GATE_CHANNELS, Config


def _norm(x):
    return x * torch.rsqrt(x.square().mean(-1, keepdim=True) + RMS_EPS)


def _rope(x, cos, sin):
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    return torch.cat([x1 * c + x2 * s, -x1 * s + x2 * c], -1)


def forward_logits(cfg: Config, p: Dict[str, torch.Tensor], tokens: torch.Tensor) -> torch.Tensor:
    """tokens [B,T] -> raw logits [B,T,padded_vocab]."""
    B, T = tokens.shape
    H, KV, D, C = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.hidden_dim
    dev = tokens.device
    half = D // 2
    inv = 1.0 / (cfg.rope_base ** (torch.arange(half, device=dev, dtype=torch.float32) * 2.0 / D))
    ang = torch.arange(T, device=dev, dtype=torch.float32)[:, None] * inv[None, :]
    cos, sin = torch.cos(ang).to(p["lm_head.weight"].dtype), torch.sin(ang).to(p["lm_head.weight"].dtype)
    tok = tokens.long()
    e = _norm(p["transformer.wte.weight"][tok])
    gate = torch.sigmoid(e[..., :SMEAR_CHANNELS] @ p["smear_gate.weight"].view(-1))
    prev = torch.cat([torch.zeros_like(e[:, :1]), e[:, :-1]], 1)
    gate = torch.cat([torch.zeros_like(gate[:, :1]), gate[:, 1:]], 1)
    x = e + (p["smear_lambda"] * gate).unsqueeze(-1) * prev
    x0 = x
    xb = None
    for i in range(cfg.num_layers):
        pre = f"transformer.h.{i}."
        xr = p["resid_lambdas"][i] * x + p["x0_lambdas"][i] * x0
        h = _norm(xr)
        q = (h @ p[pre + "attn.c_q.weight"].t()).view(B, T, H, D)
        k = (h @ p[pre + "attn.c_k.weight"].t()).view(B, T, KV, D)
        v = (h @ p[pre + "attn.c_v.weight"].t()).view(B, T, KV, D)
        if cfg.has_value_embedding(i):
            ve = p[f"value_embeds.{i}.weight"][tok].view(B, T, KV, D)
            g = 3.0 * torch.sigmoid(h[..., :VE_GATE_CHANNELS] @ p[pre + "attn.ve_gate.weight"].t())
            v = v + g.unsqueeze(-1) * ve
        q = _rope(_norm(q), cos, sin) * QK_SCALE
        k = _rope(_norm(k), cos, sin) * QK_SCALE
        wl = cfg.window_left(i)
        qpos = torch.arange(T, device=dev)[:, None]
        j = torch.arange(T, device=dev)[None, :]
        ok = j <= qpos
        if wl >= 0:
            ok = ok & ((qpos - j) <= wl)
        group = H // KV
        kk = k.permute(0, 2, 1, 3).repeat_interleave(group, 1)
        vv = v.permute(0, 2, 1, 3).repeat_interleave(group, 1)
        s = (q.permute(0, 2, 1, 3) @ kk.transpose(-1, -2)) / math.sqrt(D)
        s = s.masked_fill(~ok, float("-inf"))
        a = (torch.softmax(s, -1) @ vv).permute(0, 2, 1, 3).reshape(B, T, H * D)
        x_mid = xr + a @ p[pre + "attn.c_proj.weight"].t()
        h2 = _norm(x_mid)
        x = x_mid + torch.relu(h2 @ p[pre + "mlp.c_fc.weight"].t()).square() @ p[pre + "mlp.c_proj.weight"].t()
        if i == cfg.backout_layer:
            xb = x
    x = x - p["backout_lambda"] * xb
    return _norm(x) @ p["lm_head.weight"].t()


def loss_fn(cfg: Config, p: Dict[str, torch.Tensor], tokens, targets) -> torch.Tensor:
    logits = forward_logits(cfg, p, tokens)[..., : cfg.vocab_size]
    z = LOGIT_SOFTCAP * torch.tanh(logits / LOGIT_SOFTCAP)
    return F.cross_entropy(z.reshape(-1, cfg.vocab_size).float(), targets.reshape(-1).long(),
                           ignore_index=-1, reduction="mean")
