"""Parameter and FLOP counting, MFU.

Same counting rules as the reference performance model (`src/performance_model.cc:233-350`):
flops per token = 6 * matmul parameters + 12 * heads * head_dim * window per layer, where the matmul
parameters are the block matrices, the LM head and the two kinds of gate (embeddings are gathers, not matmuls) and the window
of a sliding layer is min(short_window, seq). Muon's Newton-Schulz FLOPs are reported separately and
never added to the model FLOPs (reference `src/train.cc:917-925`).
"""
from __future__ import annotations

import json
import os

from ..config import SMEAR_CHANNELS, VE_GATE_CHANNELS, Config


def num_matmul_params(cfg: Config) -> int:
    C = cfg.hidden_dim
    per_layer = cfg.query_dim * C + 2 * cfg.kv_dim * C + C * C + 2 * C * cfg.mlp_dim
    value_layers = sum(1 for i in range(cfg.num_layers) if cfg.has_value_embedding(i))
    # the value gates ([kv_heads, 12] each) and the smear gate ([1, 24]) are linear maps of the token stream too
    return (cfg.num_layers * per_layer + cfg.padded_vocab_size * C + value_layers * cfg.num_kv_heads * VE_GATE_CHANNELS
            + SMEAR_CHANNELS)


def count_params(cfg: Config) -> int:
    from ..models.params import param_specs
    return sum(s.count for s in param_specs(cfg))


def flops_per_token(cfg: Config, seq: int = 0) -> float:
    seq = seq or cfg.seq_len
    attn = 0
    for i in range(cfg.num_layers):
        attn += 12 * cfg.num_heads * cfg.head_dim * cfg.effective_window(i, seq)
    return 6.0 * num_matmul_params(cfg) + float(attn)


def muon_flops_per_step(cfg: Config, ns_steps: int = 5) -> float:
    total = 0.0
    C = cfg.hidden_dim
    shapes = [(cfg.query_dim, C), (cfg.kv_dim, C), (cfg.kv_dim, C), (C, C), (cfg.mlp_dim, C), (C, cfg.mlp_dim)]
    for r, c in shapes:
        k, n = min(r, c), max(r, c)
        total += cfg.num_layers * ns_steps * (4.0 * k * k * n + 2.0 * k * k * k)
    return total


def measured_peaks() -> dict:
    """bf16 / HBM peaks measured on this pool's B200s when the file exists, else the documented fallback."""
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            return {"bf16_tflops": float(d["bf16_tflops"]), "bf16_tflops_sustained": float(d["bf16_tflops_sustained"]),
                    "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
        except Exception:
            pass
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


def mfu(tokens_per_s: float, cfg: Config, peak_tflops: float, seq: int = 0) -> float:
    return tokens_per_s * flops_per_token(cfg, seq) / (peak_tflops * 1e12)
