"""Start-up correctness gate on the real device.

The reference refuses to train when its kernels disagree with the host definition on the installed GPU
(`src/hw_gate.cc:437` RunHardwareCorrectnessGate: conversions, scaled GEMMs in three layouts, attention forward and
backward, two training steps). This gate does the same for this engine's kernels: each check runs a kernel and the
plain PyTorch definition of the same operator (`ops.ref`) on small inputs and compares; the last check runs two
training steps of a small model through both operator sets. It takes well under a second on a B200.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch


def _rel(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-6))


def run_hardware_gate(device) -> Tuple[bool, List[Dict]]:
    from . import ops
    from .config import Config
    from .models import GPT
    from .ops import ref
    device = torch.device(device)
    report: List[Dict] = []

    def check(name: str, err: float, tol: float) -> None:
        report.append(dict(name=name, err=err, tol=tol, ok=bool(err <= tol)))

    if device.type != "cuda":
        return True, report
    from .ops import cuda as K
    g = torch.Generator(device=device).manual_seed(1)
    rn = lambda *s: (torch.randn(*s, device=device, generator=g) * 0.5).to(torch.bfloat16)
    # GEMM: forward (K-major both), dgrad (MN-major B), wgrad (MN-major both, fp32 accumulate), fused epilogues
    x, w, dy = rn(512, 384), rn(640, 384), rn(512, 640)
    check("gemm.forward", _rel(K.linear_fwd(x, w), ref.linear_fwd(x, w)), 2e-2)
    check("gemm.relu2", _rel(K.linear_relu2_fwd(x, w)[1], ref.linear_relu2_fwd(x, w)[1]), 2e-2)
    check("gemm.dgrad", _rel(K.linear_dgrad(dy, w), ref.linear_dgrad(dy, w)), 2e-2)
    acc_k = torch.zeros(640, 384, device=device)
    acc_r = torch.zeros(640, 384, device=device)
    K.linear_wgrad(dy, x, acc_k)
    ref.linear_wgrad(dy, x, acc_r)
    check("gemm.wgrad", _rel(acc_k, acc_r), 2e-2)
    # fp8: the quantizer bit for bit, then the block-scaled product on three shapes (ragged M, both tile widths)
    xq = rn(300, 512) * 4
    qk_, ek_ = K.quantize_fp8(xq)
    qr_, er_ = ref.quantize_fp8(xq)
    check("fp8.quantize.codes", float((qk_.float() != qr_.float()).float().mean()), 0.0)
    check("fp8.quantize.scales", float((ek_ != er_).float().mean()), 0.0)
    for m_, n_, k_ in ((512, 640, 384), (257, 3840, 256), (1024, 1280, 1280)):
        a_, b_ = rn(m_, k_), rn(n_, k_)
        check(f"fp8.scaled_gemm.{m_}x{n_}x{k_}", _rel(K.gemm_scaled_fp8(a_, b_), ref.gemm_scaled_fp8(a_, b_)), 2e-2)
    # attention forward / backward, GQA + window
    B, T, H, KV, D = 2, 384, 4, 2, 128
    q, k, v, do = rn(B, T, H, D), rn(B, T, KV, D), rn(B, T, KV, D), rn(B, T, H, D)
    o_k, lse_k = K.attention_fwd(q, k, v, window_left=200, scale=D ** -0.5)
    o_r, lse_r = ref.attention_fwd(q, k, v, window_left=200, scale=D ** -0.5)
    check("attention.forward", _rel(o_k, o_r), 3e-2)
    gk = K.attention_bwd(q, k, v, o_k, lse_k, do, window_left=200, scale=D ** -0.5)
    gr = ref.attention_bwd(q, k, v, o_r, lse_r, do, window_left=200, scale=D ** -0.5)
    for n, a, b in zip(("dq", "dk", "dv"), gk, gr):
        check("attention.backward." + n, _rel(a, b), 4e-2)
    # two training steps of a small model: kernels against the PyTorch operators
    cfg = Config(num_layers=2, num_heads=2, num_kv_heads=1, hidden_dim=256, seq_len=256, vocab_size=512,
                 padded_vocab_size=512, window_pattern="SL", short_window_override=128)
    from .optim import Optimizer
    tok = torch.randint(0, 512, (2, 256), device=device, generator=g)
    tgt = torch.roll(tok, -1, 1)
    losses = {}
    for mode in ("kernels", "torch"):
        ops.set_mode(mode)
        try:
            m = GPT(cfg, device, torch.bfloat16, seed=3)
            opt = Optimizer(m.params)
            ls = []
            for s in (1, 2):
                m.zero_grad()
                ls.append(float(m.forward_backward(tok, tgt)))
                opt.step(s)
            ls.append(float(m.forward_loss(tok, tgt)))
            losses[mode] = ls
        finally:
            ops.set_mode("kernels")
    check("train.two_steps", max(abs(a - b) for a, b in zip(losses["kernels"], losses["torch"])), 3e-2)
    K.check_status(device)
    return all(r["ok"] for r in report), report
