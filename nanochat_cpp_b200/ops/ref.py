"""Plain-PyTorch statements of every operator of the model and the optimizer.

These functions are the numerical definition the CUDA kernels are tested
against, and the execution path for CPU tensors. They restate the arithmetic of
the reference CPU backend (`backends/cpu/kernels.cc`): RMSNorm :652-700,
QkPrep :708-839, attention :879-1127, classifier :1370-1510, embedding
:1511-1540, AdamW :1557-1580, Muon :1614-1810, value gate :1964-2033, smear
:2034-2109. Reductions run in fp32 (fp64 when the inputs are fp32/fp64 so that
the fp32 oracle fixtures hold to 1e-5), and every output is rounded once to the
dtype of its input.
"""
from __future__ import annotations

import math

import torch

from ..config import LOGIT_SOFTCAP, QK_SCALE, RMS_EPS, SMEAR_CHANNELS, VE_GATE_CHANNELS

POLAR_COEFFS = (
    (8.156554524902461, -22.48329292557795, 15.878769915207462),
    (4.042929935166739, -2.808917465908714, 0.5000178451051316),
    (3.8916678022926607, -2.772484153217685, 0.5060648178503393),
    (3.285753657755655, -2.3681294933425376, 0.46449024233003106),
    (2.3465413258596377, -1.7097828382687081, 0.42323551169305323),
)


def _acc(x: torch.Tensor) -> torch.dtype:
    return torch.float64 if x.dtype in (torch.float32, torch.float64) else torch.float32


# --------------------------------------------------------------------------
# GEMMs (weights are [out, in]; y = x @ w.T)
# --------------------------------------------------------------------------
def linear_fwd(x, w, *, out=None, residual=None):
    y = torch.matmul(x, w.t())
    if residual is not None:
        y = (y.float() + residual.float()).to(x.dtype)
    if out is not None:
        out.copy_(y)
        return out
    return y


def linear_relu2_fwd(x, w):
    """Returns (pre, act) with act = relu(pre)^2 computed from the rounded pre."""
    pre = torch.matmul(x, w.t())
    act = torch.relu(pre.float()).square().to(x.dtype)
    return pre, act


def quantize_fp8(x):
    """MXFP8 of x [R, K] (K % 32 == 0): (E4M3 values as float8_e4m3fn [R, K], biased power-of-two exponents uint8
    [R, K/32]); the value of element (r, k) is q[r, k] * 2^(e[r, k // 32] - 127). The seam's QuantizeFp8
    (reference: include/nanochat/kernels.h:138-175, per-tensor scale there)."""
    from .fp8 import ref_mx_quantize
    return ref_mx_quantize(x)


def gemm_scaled_fp8(x, w, relu2: bool = False):
    """y = Q(x) @ Q(w)^T in the compute dtype, Q = MXFP8 quantize-dequantize; with `relu2` returns (y, relu(y)^2).
    The seam's QuantizeFp8 + GemmScaledFp8 composition (reference: src/ops.cc:551-706, fp8 linear forward)."""
    from .fp8 import ref_mx_dequantize, ref_mx_quantize
    y = (ref_mx_dequantize(*ref_mx_quantize(x)) @ ref_mx_dequantize(*ref_mx_quantize(w)).t()).to(x.dtype)
    if relu2:
        return y, torch.relu(y.float()).square().to(x.dtype)
    return y


def linear_relu2_act_fwd(x, w):
    """act = relu(pre)^2 with pre = x @ w^T rounded to the compute dtype first (as `linear_relu2_fwd`)."""
    return linear_relu2_fwd(x, w)[1]


def linear_dgrad_relu2_act(dy, w, act):
    """d(pre) = (dy @ w) * 2 sqrt(act): relu(pre) recovered from the saved activation."""
    dact = torch.matmul(dy, w).float()
    return (dact * 2.0 * torch.sqrt(act.float().clamp_min(0.0))).to(dy.dtype)


def linear_dgrad(dy, w, *, residual=None):
    dx = torch.matmul(dy, w)
    if residual is not None:
        dx = (dx.float() + residual.float()).to(dy.dtype)
    return dx


def linear_dgrad_relu2(dy, w, pre):
    """d(pre) = (dy @ w) * 2*relu(pre): the backward of act = relu(pre)^2."""
    dact = torch.matmul(dy, w).float()
    return (dact * 2.0 * torch.relu(pre.float())).to(dy.dtype)


def linear_wgrad_relu2(dy, pre, grad, *, accumulate=True):
    """grad[N,K] (+)= dy[M,N]^T @ relu(pre[M,K])^2 (the activation is recomputed, not saved)."""
    act = torch.relu(pre.float()).square().to(pre.dtype)
    return linear_wgrad(dy, act, grad, accumulate=accumulate)


def linear_wgrad(dy, x, grad, *, accumulate=True):
    """grad[N,K] (+)= dy[M,N]^T @ x[M,K]; grad is fp32."""
    g = torch.matmul(dy.t(), x).float()
    if accumulate:
        grad.add_(g)
    else:
        grad.copy_(g)
    return grad


# --------------------------------------------------------------------------
# RMSNorm (no learned gain)
# --------------------------------------------------------------------------
def rmsnorm_fwd(x, eps=RMS_EPS):
    xf = x.to(_acc(x))
    ms = xf.square().sum(-1, keepdim=True).float() * (1.0 / x.shape[-1])
    rstd = 1.0 / torch.sqrt(ms + eps)
    y = (x.float() * rstd).to(x.dtype)
    return y, rstd.squeeze(-1)


def rmsnorm_apply(x, rstd):
    """Recompute y = x * rstd from the saved statistic."""
    return (x.float() * rstd.unsqueeze(-1)).to(x.dtype)


def rmsnorm_bwd(x, dy, rstd, residual=None):
    """dx = rstd*dy - rstd^3 * mean(x*dy) * x  (+ residual, added before the rounding)."""
    dim = x.shape[-1]
    acc = _acc(x)
    dot = (x.to(acc) * dy.to(acc)).sum(-1, keepdim=True).float()
    r = rstd.unsqueeze(-1)
    coeff = r * r * r * dot * (1.0 / dim)
    dx = r * dy.float() - coeff * x.float()
    if residual is not None:
        dx = dx + residual.float()
    return dx.to(x.dtype)


def add(a, b):
    return (a.float() + b.float()).to(a.dtype)


def add_cols(dh, extra):
    """dh[:, :n] += extra (fp32 [M, n]); returns dh."""
    n = extra.shape[1]
    dh[:, :n] = (dh[:, :n].float() + extra.float()).to(dh.dtype)
    return dh


def concat_qkv(dq, dk, dv):
    return torch.cat([dq, dk, dv], dim=1)


def backout_fwd(x, x_backout, lam):
    return (x.float() - lam.float() * x_backout.float()).to(x.dtype)


def backout_bwd(dy, x_backout, lam):
    """Returns (dx, dx_backout, dlam)."""
    acc = _acc(dy)
    dlam = -(dy.to(acc) * x_backout.to(acc)).sum().float()
    return dy, (-lam.float() * dy.float()).to(dy.dtype), dlam


def blend_norm_fwd(x, x0, lam_r, lam_0, eps=RMS_EPS):
    """xr = lam_r*x + lam_0*x0 ; h = rmsnorm(xr). lam_* are 0-d fp32 tensors."""
    xr = (lam_r.float() * x.float() + lam_0.float() * x0.float()).to(x.dtype)
    h, rstd = rmsnorm_fwd(xr, eps)
    return xr, h, rstd


def blend_bwd(dxr, x, x0, lam_r, lam_0, dx0_acc=None):
    """Backward of the blend. Returns (dx, dx0, dlam_r, dlam_0); with `dx0_acc` the x0 term is
    accumulated into that tensor (in place) and it is what is returned as dx0."""
    acc = _acc(x)
    dlr = (dxr.to(acc) * x.to(acc)).sum().float()
    dl0 = (dxr.to(acc) * x0.to(acc)).sum().float()
    dx = (lam_r.float() * dxr.float()).to(x.dtype)
    if dx0_acc is None:
        dx0 = (lam_0.float() * dxr.float()).to(x.dtype)
    else:
        dx0_acc.copy_((dx0_acc.float() + lam_0.float() * dxr.float()).to(x.dtype))
        dx0 = dx0_acc
    return dx, dx0, dlr, dl0


def norm_blend_bwd(xr, dh, rstd, residual, x, x0, lam_r, lam_0, g_lam_r, g_lam_0, dx0_acc=None, extra=None):
    """Backward of h = rmsnorm(xr) with xr = lam_r * x + lam_0 * x0, as one operator: the definition is the chain
    add_cols -> rmsnorm_bwd -> blend_bwd, except that dxr is not rounded to the compute dtype in between. The scalar
    gradients are added into `g_lam_r` / `g_lam_0` (one-element views of the gradient buffer). Returns (dx, dx0)."""
    if extra is not None:
        dh = add_cols(dh.clone(), extra)
    dim = xr.shape[-1]
    acc = _acc(xr)
    dot = (xr.to(acc) * dh.to(acc)).sum(-1, keepdim=True).float()
    r = rstd.unsqueeze(-1)
    dxr = r * dh.float() - (r * r * r * dot * (1.0 / dim)) * xr.float() + residual.float()
    g_lam_r += (dxr.to(acc) * x.to(acc).view_as(dxr)).sum().float()
    g_lam_0 += (dxr.to(acc) * x0.to(acc).view_as(dxr)).sum().float()
    dx = (lam_r.float() * dxr).to(x.dtype).view_as(x)
    if dx0_acc is None:
        dx0 = (lam_0.float() * dxr).to(x.dtype).view_as(x)
    else:
        dx0_acc.copy_((dx0_acc.float().view_as(dxr) + lam_0.float() * dxr).to(x.dtype).view_as(dx0_acc))
        dx0 = dx0_acc
    return dx, dx0


# --------------------------------------------------------------------------
# Rotary tables and QK preparation: per-head RMSNorm -> RoPE (half split) -> scale
# --------------------------------------------------------------------------
def build_rope(seq, head_dim, base, device="cpu", offset=0):
    half = head_dim // 2
    d = torch.arange(half, dtype=torch.float32, device=device)
    inv_freq = 1.0 / torch.pow(torch.tensor(float(base), dtype=torch.float32, device=device),
                               (2.0 * d) / float(head_dim))
    t = torch.arange(offset, offset + seq, dtype=torch.float32, device=device)
    ang = t[:, None] * inv_freq[None, :]
    return torch.cos(ang).contiguous(), torch.sin(ang).contiguous()


def _qk_prep_one(x, cos, sin, eps, scale):
    # x: [B, T, H, D]; cos/sin: [T, D/2] or [B, T, D/2]
    half = x.shape[-1] // 2
    y, _ = rmsnorm_fwd(x, eps)
    c = cos.unsqueeze(-2) if cos.dim() == 3 else cos[None, :, None, :]
    s = sin.unsqueeze(-2) if sin.dim() == 3 else sin[None, :, None, :]
    x1 = y[..., :half].float()
    x2 = y[..., half:].float()
    o1 = (x1 * c + x2 * s) * scale
    o2 = (-x1 * s + x2 * c) * scale
    return torch.cat([o1, o2], -1).to(x.dtype)


def qk_prep_fwd(q_pre, k_pre, cos, sin, eps=RMS_EPS, scale=QK_SCALE):
    return _qk_prep_one(q_pre, cos, sin, eps, scale), _qk_prep_one(k_pre, cos, sin, eps, scale)


def _qk_prep_bwd_one(pre, grad, cos, sin, eps, scale):
    dim = pre.shape[-1]
    half = dim // 2
    c = cos.unsqueeze(-2) if cos.dim() == 3 else cos[None, :, None, :]
    s = sin.unsqueeze(-2) if sin.dim() == 3 else sin[None, :, None, :]
    g1 = grad[..., :half].float()
    g2 = grad[..., half:].float()
    g = torch.cat([scale * (g1 * c - g2 * s), scale * (g1 * s + g2 * c)], -1)
    acc = _acc(pre)
    xf = pre.to(acc)
    ss = xf.square().sum(-1, keepdim=True).float()
    dot = (xf * g.to(acc)).sum(-1, keepdim=True).float()
    r = 1.0 / torch.sqrt(ss * (1.0 / dim) + eps)
    coeff = r * r * r * dot * (1.0 / dim)
    return (r * g - coeff * pre.float()).to(pre.dtype)


def qk_prep_bwd(q_pre, k_pre, dq, dk, cos, sin, eps=RMS_EPS, scale=QK_SCALE, out_q=None, out_k=None):
    gq = _qk_prep_bwd_one(q_pre, dq, cos, sin, eps, scale)
    gk = _qk_prep_bwd_one(k_pre, dk, cos, sin, eps, scale)
    if out_q is not None:
        out_q.copy_(gq)
        gq = out_q
    if out_k is not None:
        out_k.copy_(gk)
        gk = out_k
    return gq, gk


# --------------------------------------------------------------------------
# Attention: causal, optional left window, GQA with contiguous grouping
# q [B,T,H,D], k/v [B,S,KV,D]; query t sits at absolute position q_offset + t
# --------------------------------------------------------------------------
def attention_mask(t_q, t_k, window_left, q_offset, device):
    qpos = torch.arange(t_q, device=device)[:, None] + q_offset
    j = torch.arange(t_k, device=device)[None, :]
    ok = j <= qpos
    if window_left is not None and window_left >= 0:
        ok = ok & ((qpos - j) <= window_left)
    return ok


def attention_fwd(q, k, v, window_left=-1, scale=None, q_offset=None):
    """Returns (out [B,T,H,D], lse [B,H,T]) with lse = max + log(sumexp) in natural log."""
    B, T, H, D = q.shape
    S, KV = k.shape[1], k.shape[2]
    group = H // KV
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if q_offset is None:
        q_offset = S - T
    acc = torch.float32
    qf = q.to(acc).permute(0, 2, 1, 3)  # B,H,T,D
    kf = k.to(acc).permute(0, 2, 1, 3).repeat_interleave(group, dim=1)
    vf = v.to(acc).permute(0, 2, 1, 3).repeat_interleave(group, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    ok = attention_mask(T, S, window_left, q_offset, q.device)
    s = s.masked_fill(~ok, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    o = torch.matmul(p, vf)
    return o.permute(0, 2, 1, 3).to(q.dtype).contiguous(), lse


def attention_bwd(q, k, v, o, lse, do, window_left=-1, scale=None, q_offset=None, out=None):
    B, T, H, D = q.shape
    S, KV = k.shape[1], k.shape[2]
    group = H // KV
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if q_offset is None:
        q_offset = S - T
    acc = torch.float32
    qf = q.to(acc).permute(0, 2, 1, 3)
    kf = k.to(acc).permute(0, 2, 1, 3).repeat_interleave(group, dim=1)
    vf = v.to(acc).permute(0, 2, 1, 3).repeat_interleave(group, dim=1)
    dof = do.to(acc).permute(0, 2, 1, 3)
    of = o.to(acc).permute(0, 2, 1, 3)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    ok = attention_mask(T, S, window_left, q_offset, q.device)
    s = s.masked_fill(~ok, float("-inf"))
    p = torch.exp(s - lse.to(acc).unsqueeze(-1))
    dv = torch.matmul(p.transpose(-1, -2), dof)
    dp = torch.matmul(dof, vf.transpose(-1, -2))
    delta = (dof * of).sum(-1, keepdim=True)
    ds = p * (dp - delta) * scale
    dq = torch.matmul(ds, kf)
    dk = torch.matmul(ds.transpose(-1, -2), qf)
    dk = dk.view(B, KV, group, S, D).sum(2)
    dv = dv.view(B, KV, group, S, D).sum(2)
    res = [dq.permute(0, 2, 1, 3).to(q.dtype).contiguous(),
           dk.permute(0, 2, 1, 3).to(k.dtype).contiguous(),
           dv.permute(0, 2, 1, 3).to(v.dtype).contiguous()]
    if out is not None:
        for i in range(3):
            if out[i] is not None:
                out[i].copy_(res[i])
                res[i] = out[i]
    return tuple(res)


# --------------------------------------------------------------------------
# Value gate: v += 3*sigmoid(h[:, :12] @ Wg^T) * ve   (per kv head)
# --------------------------------------------------------------------------
def value_gate_fwd(h, ve, gate_w, v, head_dim):
    """h [M,C], ve [M,kv_dim], gate_w [KV,12], v [M,kv_dim] -> (v_out, gate [M,KV])."""
    M = h.shape[0]
    KV = gate_w.shape[0]
    pre = torch.matmul(h[:, :VE_GATE_CHANNELS].float(), gate_w.float().t())
    gate = (3.0 / (1.0 + torch.exp(-pre)))
    gate_r = gate.to(h.dtype)
    out = (v.float().view(M, KV, head_dim) + gate.unsqueeze(-1) * ve.float().view(M, KV, head_dim))
    return out.view(M, KV * head_dim).to(v.dtype), gate_r


def value_gate_bwd(h, ve, gate_w, gate, dv, head_dim):
    """Returns (dve [M,kv_dim], dh12 [M,12] fp32, dgate_w [KV,12] fp32)."""
    M = h.shape[0]
    KV = gate_w.shape[0]
    acc = _acc(h)
    g = gate.float()
    dvf = dv.view(M, KV, head_dim)
    dgate = (dvf.to(acc) * ve.view(M, KV, head_dim).to(acc)).sum(-1).float()
    dve = (g.unsqueeze(-1) * dvf.float()).to(dv.dtype).view(M, KV * head_dim)
    dpre = dgate * g * (1.0 - g / 3.0)
    dgw = torch.matmul(dpre.to(acc).t(), h[:, :VE_GATE_CHANNELS].to(acc)).float()
    dh12 = torch.matmul(dpre, gate_w.float())
    return dve, dh12, dgw


# --------------------------------------------------------------------------
# Smear: x[t] = e[t] + lambda*sigmoid(e[t,:24].w)*e[t-1], x[0] = e[0] per row
# --------------------------------------------------------------------------
def smear_fwd(emb, gate_w, lam, seq, prev=None):
    """emb [M,C] (M = B*seq). `prev` ([B,C]) supplies e[-1] for decode; None = none.
    Returns (x0, sig [M] fp32)."""
    M, C = emb.shape
    B = M // seq
    e = emb.view(B, seq, C)
    pre = torch.matmul(e[..., :SMEAR_CHANNELS].float(), gate_w.float().view(-1))
    sig = 1.0 / (1.0 + torch.exp(-pre))
    shifted = torch.zeros_like(e)
    shifted[:, 1:] = e[:, :-1]
    if prev is not None:
        shifted[:, 0] = prev
    else:
        sig = sig.clone()
        sig[:, 0] = 0.0
    x0 = (e.float() + (lam.float() * sig).unsqueeze(-1) * shifted.float()).to(emb.dtype)
    return x0.view(M, C), sig.reshape(M)


def smear_bwd(emb, gate_w, lam, sig, dx0, seq):
    """Returns (de [M,C], dgate_w [24] fp32, dlam 0-d fp32)."""
    M, C = emb.shape
    B = M // seq
    acc = _acc(emb)
    e = emb.view(B, seq, C)
    d = dx0.view(B, seq, C)
    s = sig.view(B, seq).float()
    shifted = torch.zeros_like(e)
    shifted[:, 1:] = e[:, :-1]
    dgate = (d.to(acc) * shifted.to(acc)).sum(-1).float()  # zero at t=0 because shifted is zero
    dlam = (dgate.to(acc) * s.to(acc)).sum().float()
    dpre = dgate * lam.float() * s * (1.0 - s)
    dgw = torch.matmul(dpre.reshape(-1).to(acc), e[..., :SMEAR_CHANNELS].reshape(M, -1).to(acc)).float()
    de = d.float().clone()
    de[..., :SMEAR_CHANNELS] += dpre.unsqueeze(-1) * gate_w.float().view(-1)
    gate_next = lam.float() * s[:, 1:]
    de[:, :-1] += gate_next.unsqueeze(-1) * d[:, 1:].float()
    return de.to(emb.dtype).view(M, C), dgw, dlam


# --------------------------------------------------------------------------
# Embedding gather / scatter-add
# --------------------------------------------------------------------------
def embedding_fwd(ids, table):
    return table.index_select(0, ids.reshape(-1).long())


def embedding_order(ids):
    s, perm = torch.sort(ids.reshape(-1), stable=True)
    return s.to(torch.int32), perm.to(torch.int32)


def embedding_bwd(ids, dout, dtable, order=None):
    dtable.index_add_(0, ids.reshape(-1).long(), dout.to(dtable.dtype))
    return dtable


# --------------------------------------------------------------------------
# Classifier: softcap 15*tanh(z/15) + cross entropy over the real vocabulary
# --------------------------------------------------------------------------
def classifier_fwd_bwd(logits, targets, vocab, *, dlogit_scale, row_scale=None,
                       softcap=LOGIT_SOFTCAP, ignore_index=-1, want_grad=True):
    """logits [R, padded] -> (losses [R] fp32, dlogits [R, padded] or None).

    dlogits = (softmax - onehot) * (1 - tanh^2) * row_scale * dlogit_scale, zero on
    ignored rows and on the padded tail.
    """
    R, padded = logits.shape
    z_raw = logits[:, :vocab].float()
    t = torch.tanh(z_raw / softcap)
    z = softcap * t
    row_max = z.max(dim=-1, keepdim=True).values
    acc = _acc(logits)
    sum_exp = torch.exp((z - row_max).to(acc)).sum(-1, keepdim=True)
    valid = targets != ignore_index
    tgt = targets.clamp(min=0, max=vocab - 1).long()
    in_range = (targets >= 0) & (targets < vocab)
    tz = torch.where(in_range, z.gather(1, tgt[:, None]).squeeze(1), torch.zeros_like(z[:, 0]))
    losses = torch.log(sum_exp).float().squeeze(1) + row_max.squeeze(1) - tz
    losses = torch.where(valid, losses, torch.zeros_like(losses))
    if not want_grad:
        return losses, None
    p = torch.exp(z - row_max) * (1.0 / sum_exp).float()
    onehot = torch.zeros_like(p)
    onehot.scatter_(1, tgt[:, None], in_range[:, None].float())
    g = (p - onehot) * (1.0 - t * t)
    if row_scale is not None:
        g = g * row_scale.float()[:, None]
    g = g.to(logits.dtype).float() * dlogit_scale
    g = torch.where(valid[:, None], g, torch.zeros_like(g))
    dl = torch.zeros_like(logits)
    dl[:, :vocab] = g.to(logits.dtype)
    return losses, dl


# --------------------------------------------------------------------------
# Optimizer updates (fp32 state)
# --------------------------------------------------------------------------
def adamw_update(master, value, grad, m, v, *, lr, beta1, beta2, eps, weight_decay, step,
                 grad_scale=1.0):
    bias1 = 1.0 - beta1 ** step
    bias2 = 1.0 - beta2 ** step
    step_size = lr / bias1
    g = grad.float() * grad_scale
    p = master * (1.0 - lr * weight_decay)
    m.add_((1.0 - beta1) * (g - m))
    v.add_((1.0 - beta2) * (g * g - v))
    denom = torch.sqrt(v / bias2) + eps
    p = p - step_size * (m / denom)
    master.copy_(p)
    if value is not None:
        value.copy_(p.to(value.dtype))


def polar_express(x, ns_steps, matmul=torch.matmul):
    """x: [P, rows, cols] fp32 (already normalised). Returns the orthogonalised stack."""
    rows, cols = x.shape[-2], x.shape[-1]
    tall = rows > cols
    for it in range(min(max(ns_steps, 0), 5)):
        ca, cb, cc = POLAR_COEFFS[it]
        if tall:
            a = matmul(x.transpose(-1, -2), x)
            b = cb * a + cc * matmul(a, a)
            x = ca * x + matmul(x, b)
        else:
            a = matmul(x, x.transpose(-1, -2))
            b = cb * a + cc * matmul(a, a)
            x = ca * x + matmul(b, x)
    return x


def muon_update(grads, master, values, buf1, buf2, *, lr, momentum, beta2, weight_decay,
                ns_steps=5, grad_scale=1.0, nesterov=True, matmul=torch.matmul):
    """One Muon step on a stacked group.

    grads/master/buf1: [P, rows, cols] fp32; values: same shape in the compute dtype (or
    None); buf2: [P, lines] with lines = rows if rows >= cols else cols.
    """
    P, rows, cols = master.shape
    acc = torch.float64
    reduce_cols = rows >= cols
    g = grads.float() * grad_scale
    buf1.add_((1.0 - momentum) * (g - buf1))
    x = (1.0 - momentum) * g + momentum * buf1 if nesterov else buf1.clone()
    # MuonEq: rescale every row to the mean row norm
    frob = torch.sqrt(x.to(acc).square().sum((-1, -2), keepdim=True)).float()
    target = frob / math.sqrt(float(rows))
    row_norm = torch.sqrt(x.to(acc).square().sum(-1, keepdim=True)).float().clamp_min(1e-6)
    x = x * (target / row_norm)
    frob = torch.sqrt(x.to(acc).square().sum((-1, -2), keepdim=True)).float()
    x = x / (frob * 1.01 + 1e-6)
    x = polar_express(x, ns_steps, matmul)
    # Muon+: snap the norm to sqrt(min(rows, cols))
    frob = torch.sqrt(x.to(acc).square().sum((-1, -2), keepdim=True)).float()
    x = x * (math.sqrt(float(min(rows, cols))) / frob.clamp_min(1e-6))
    # NorMuon
    red = -1 if reduce_cols else -2
    line_len = cols if reduce_cols else rows
    v_mean = (x.to(acc).square().sum(red) / line_len).float()  # [P, lines]
    v_norm = torch.sqrt(v_mean.to(acc).sum(-1, keepdim=True).float() * float(line_len))
    buf2.add_((1.0 - beta2) * (v_mean - buf2))
    step_size = 1.0 / torch.sqrt(buf2.clamp_min(1e-10))
    sum_scaled = ((v_mean * float(line_len)).to(acc) * step_size.to(acc) * step_size.to(acc)).sum(-1, keepdim=True)
    denom = torch.sqrt(sum_scaled).float().clamp_min(1e-10)
    step_size = step_size * (v_norm / denom)
    x = x * step_size.unsqueeze(red)
    # cautious weight decay + update
    decay = torch.where(x * master >= 0, lr * weight_decay * master, torch.zeros_like(master))
    p = master - lr * x - decay
    master.copy_(p)
    if values is not None:
        values.copy_(p.to(values.dtype))


def grad_norm_and_clip(grads, clip):
    """Returns (norm, clip_scale) as 0-d fp32 tensors; grads is a list of fp32 tensors."""
    total = None
    for g in grads:
        s = g.to(torch.float64).square().sum()
        total = s if total is None else total + s
    norm = torch.sqrt(total).float()
    if clip is not None and clip > 0:
        scale = torch.where(norm > clip, clip / norm.clamp_min(1e-30), torch.ones_like(norm))
    else:
        scale = torch.ones_like(norm)
    return norm, scale


# --------------------------------------------------------------------------
# Paged KV cache (inference). Pools are [num_pages, page_size, KV, D]; page_table [B, max_pages] int32
# --------------------------------------------------------------------------
def kv_append(k_pool, v_pool, page_table, positions, k_new, v_new):
    """Write rows k_new/v_new [B, T, KV, D] at absolute positions `positions` [B, T] (int32; < 0 = skip)."""
    page_size = k_pool.shape[1]
    B, T = positions.shape
    pos = positions.long()
    valid = pos >= 0
    pos_c = pos.clamp_min(0)
    page = torch.gather(page_table.long(), 1, pos_c // page_size)
    slot = pos_c % page_size
    kp = k_pool.view(-1, *k_pool.shape[2:])
    vp = v_pool.view(-1, *v_pool.shape[2:])
    flat = (page * page_size + slot)[valid]
    kp[flat] = k_new[valid].to(kp.dtype)
    vp[flat] = v_new[valid].to(vp.dtype)


def paged_gather(pool, page_table, length):
    """Contiguous [B, length, KV, D] view of the first `length` positions of every sequence."""
    page_size = pool.shape[1]
    n_pages = (length + page_size - 1) // page_size
    idx = page_table[:, :n_pages].long().clamp_min(0)   # unmapped (released) pages: any page, masked by the caller
    out = pool[idx]  # [B, n_pages, page, KV, D]
    B = idx.shape[0]
    return out.reshape(B, n_pages * page_size, *pool.shape[2:])[:, :length]


def paged_decode_attention(q, k_pool, v_pool, page_table, seq_lens, window_left=-1, scale=None):
    """One new query per sequence. q [B, H, D]; the query of sequence b sits at position seq_lens[b] - 1 and
    sees keys j <= that position with position - j <= window_left. Returns [B, H, D]."""
    B, H, D = q.shape
    KV = k_pool.shape[2]
    group = H // KV
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    max_len = int(seq_lens.max().item())
    k = paged_gather(k_pool, page_table, max_len).float()  # [B, S, KV, D]
    v = paged_gather(v_pool, page_table, max_len).float()
    k = k.repeat_interleave(group, dim=2)
    v = v.repeat_interleave(group, dim=2)
    s = torch.einsum("bhd,bshd->bhs", q.float(), k) * scale
    j = torch.arange(max_len, device=q.device)[None, :]
    qpos = (seq_lens.long() - 1)[:, None]
    ok = j <= qpos
    if window_left is not None and window_left >= 0:
        ok = ok & ((qpos - j) <= window_left)
    s = s.masked_fill(~ok[:, None, :], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("bhs,bshd->bhd", p, v).to(q.dtype)
