"""Bandwidth benchmark of the memory-bound kernels on the d20 training shapes: achieved bytes/s of the bytes each
operator has to move, as a fraction of the measured copy bandwidth. Counterpart of the reference's `row_benchmark`
(backends/cuda/kernels/row_benchmark.cc).

    python -m nanochat_cpp_b200.bench.row_bench [--tokens 65536] [--json out.json]

Timing: CUDA events, 3 warm-up calls, L2 flushed before every timed call, median of 10 (bench/timing.py).
"""
from __future__ import annotations

import argparse
import json

import torch

from .timing import time_cuda


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=65536)
    ap.add_argument("--json", default="")
    a = ap.parse_args()
    from ..config import preset
    from ..ops import cuda as K
    from ..train import mfu
    cfg = preset("d20")
    dev = "cuda"
    M, C, H, KV, D, V = a.tokens, cfg.hidden_dim, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.padded_vocab_size
    T = cfg.seq_len
    B = M // T
    hbm = mfu.measured_peaks()["hbm_gbs"]
    bf = lambda *s: torch.randn(*s, device=dev).to(torch.bfloat16)
    x, x0, dy = bf(M, C), bf(M, C), bf(M, C)
    lam_r, lam_0 = torch.tensor(0.9, device=dev), torch.tensor(0.1, device=dev)
    xr, h, rstd = K.blend_norm_fwd(x, x0, lam_r, lam_0)
    qkv = bf(M, (H + 2 * KV) * D)
    q_pre = qkv[:, :H * D].view(B, T, H, D)
    k_pre = qkv[:, H * D:(H + KV) * D].view(B, T, KV, D)
    from .. import ops
    cos, sin = ops.build_rope(T, D, cfg.rope_base, torch.device(dev))
    dq, dk = bf(B, T, H, D), bf(B, T, KV, D)
    ve, v = bf(M, KV * D), bf(M, KV * D)
    gate_w = bf(KV, 12)
    v_out, gate = K.value_gate_fwd(h, ve, gate_w, v.clone(), D)
    ids = torch.randint(0, V, (M,), device=dev, dtype=torch.int32)
    table = bf(V, C)
    dtable = torch.zeros(V, C, device=dev, dtype=torch.float32)
    order = K.embedding_order(ids)
    rows = 8192
    logits = bf(rows, V)
    targets = torch.randint(0, cfg.vocab_size, (rows,), device=dev, dtype=torch.int32)
    n_opt = 64 * 1024 * 1024
    master, grad = torch.randn(n_opt, device=dev), torch.randn(n_opt, device=dev) * 1e-3
    m1, m2 = torch.zeros(n_opt, device=dev), torch.zeros(n_opt, device=dev)
    value = master.to(torch.bfloat16)
    big = torch.randn(256 * 1024 * 1024, device=dev)
    e = 2  # bytes per bf16
    cases = [
        ("blend_norm_fwd", lambda: K.blend_norm_fwd(x, x0, lam_r, lam_0), M * C * e * 4),
        ("rmsnorm_fwd", lambda: K.rmsnorm_fwd(x), M * C * e * 2),
        ("rmsnorm_bwd (+residual)", lambda: K.rmsnorm_bwd(xr, dy, rstd, residual=x), M * C * e * 4),
        ("blend_bwd", lambda: K.blend_bwd(dy, x, x0, lam_r, lam_0), M * C * e * 5),
        ("qk_prep_fwd", lambda: K.qk_prep_fwd(q_pre, k_pre, cos, sin), M * (H + KV) * D * e * 2),
        ("qk_prep_bwd", lambda: K.qk_prep_bwd(q_pre, k_pre, dq, dk, cos, sin), M * (H + KV) * D * e * 3),
        ("value_gate_fwd", lambda: K.value_gate_fwd(h, ve, gate_w, v, D), M * KV * D * e * 3),
        ("value_gate_bwd", lambda: K.value_gate_bwd(h, ve, gate_w, gate, v, D), M * KV * D * e * 3),
        ("embedding_fwd", lambda: K.embedding_fwd(ids, table), M * C * e * 2),
        ("embedding_bwd (atomic)", lambda: K.embedding_bwd(ids, dy, dtable), M * C * (e + 8)),
        ("embedding_bwd (sorted)", lambda: K.embedding_bwd(ids, dy, dtable, order=order), M * C * (e + 8)),
        ("classifier_fwd_bwd (8192 rows)", lambda: K.classifier_fwd_bwd(logits, targets, cfg.vocab_size, dlogit_scale=1e-4),
         rows * V * e * 2),
        ("adamw_update (64M)", lambda: K.adamw_update(master, value, grad, m1, m2, lr=1e-3, beta1=0.8, beta2=0.95,
                                                      eps=1e-10, weight_decay=0.0, step=3), n_opt * 30),
        ("grad_norm_and_clip (256M)", lambda: K.grad_norm_and_clip([big], 1.0), big.numel() * 4),
    ]
    out = []
    print(f"# measured copy bandwidth {hbm:.0f} GB/s; tokens {M}")
    print(f"{'kernel':34s} {'ms':>8s} {'GB moved':>9s} {'GB/s':>8s} {'of measured':>12s}")
    for name, fn, nbytes in cases:
        t = time_cuda(fn)["median_ms"]
        gbs = nbytes / (t * 1e-3) / 1e9
        out.append({"kernel": name, "ms": t, "bytes": nbytes, "gbs": gbs, "fraction_of_measured_hbm": gbs / hbm})
        print(f"{name:34s} {t:8.4f} {nbytes / 1e9:9.3f} {gbs:8.0f} {gbs / hbm:12.2f}")
    K.check_status()
    if a.json:
        with open(a.json, "w") as f:
            json.dump(out, f)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
