"""CUDA implementations of the operators: wrappers over the compiled extension `_C`.

Importing this module loads `nanochat_cpp_b200/_C.so`; it raises if the file is missing so that a
GPU run can never continue on a silent PyTorch fallback.
"""
from __future__ import annotations

import importlib.util
import os

import torch

from . import ref

_HERE = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_SO = os.path.join(_HERE, "_C.so")


def _load():
    if not os.path.exists(_SO):
        raise RuntimeError(f"{_SO} is not built: run `python -m nanochat_cpp_b200.build` "
                           "(the CUDA operators have no PyTorch fallback on a GPU)")
    spec = importlib.util.spec_from_file_location("nanochat_cpp_b200._C", _SO)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class _Counting:
    """Proxy over the extension module that counts kernel launches made through it."""

    # launches per call for entry points that enqueue more than one kernel
    _MULTI = {"attention_bwd": 3, "grad_norm_clip": 2}
    _NOT_KERNELS = {"read_status", "reset_status", "status_tensor"}

    def __init__(self, mod):
        self._mod = mod
        self.launches = 0
        self._cache = {}

    def __getattr__(self, name):
        fn = self._cache.get(name)
        if fn is None:
            raw = getattr(self._mod, name)
            if name in self._NOT_KERNELS:
                fn = raw
            else:
                n = self._MULTI.get(name, 1)

                def fn(*a, _raw=raw, _n=n, **k):
                    self.launches += _n
                    return _raw(*a, **k)
            self._cache[name] = fn
        return fn


_C = _Counting(_load())


def launch_count() -> int:
    """Number of this package's kernels launched so far in this process."""
    return _C.launches


def add_launches(n: int) -> None:
    """Account for kernels that a CUDA-graph replay launched (the wrappers only see them at capture time)."""
    _C.launches += int(n)

EPI_BF16, EPI_BF16_RES, EPI_RELU2, EPI_DRELU2, EPI_F32 = 0, 1, 2, 3, 4


def check_status(device=None) -> None:
    """Raise if any kernel recorded a failure in the device's status word: a bounded wait that ran out (codes 1-6)
    or an index outside its table whose access was skipped (code 7). Synchronizes the device."""
    dev = None if device is None else torch.device(device).index
    if dev is None:
        dev = torch.cuda.current_device()
    code = _C.read_status(dev)
    if code != 0:
        _C.reset_status(dev)
        what = "skipped an index outside its table" if code == 7 else "gave up waiting"
        raise RuntimeError(f"a kernel {what} (status code {code}); see csrc/cuda/ptx.cuh")


# ---------------------------------------------------------------------------
# GEMMs
# ---------------------------------------------------------------------------
# Data-parallel hook: (flag tensor, value) that the next forward GEMM must wait for inside the kernel before
# its TMA producer touches the weight operand (owners publish the flags after pushing updated weights).
_pending_weight_wait = None


def set_weight_wait(flags, value) -> None:
    global _pending_weight_wait
    _pending_weight_wait = (flags, int(value))


def clear_weight_wait() -> None:
    """Drop the pending in-GEMM wait (the caller has enqueued an explicit wait kernel instead)."""
    global _pending_weight_wait
    _pending_weight_wait = None


def gemm(a, b, *, a_mn=False, b_mn=False, epi=EPI_BF16, out=None, r=None, out2=None, alpha=1.0, beta=0.0,
         split_k=True, wait_flags=None, wait_value=0, gather_src=0, gather_counter=None, gather_base=0):
    """out = epilogue(A x B^T). See csrc/cuda/bindings.cpp for operand orders."""
    m = a.shape[-1] if a_mn else a.shape[-2]
    n = b.shape[-1] if b_mn else b.shape[-2]
    if out is None:
        shape = (*a.shape[:-2], m, n)
        out = torch.empty(shape, dtype=torch.float32 if epi == EPI_F32 else torch.bfloat16, device=a.device)
    _C.gemm(a, b, out, a_mn, b_mn, epi, r, out2, alpha, beta, split_k, wait_flags, wait_value, gather_src,
            gather_counter, gather_base)
    return out


def linear_fwd(x, w, *, out=None, residual=None):
    global _pending_weight_wait
    kw = {}
    if _pending_weight_wait is not None:
        kw = dict(wait_flags=_pending_weight_wait[0], wait_value=_pending_weight_wait[1])
        _pending_weight_wait = None
    if residual is not None:
        return gemm(x, w, epi=EPI_BF16_RES, r=residual, out=out, alpha=1.0, beta=1.0, **kw)
    return gemm(x, w, out=out, **kw)


def linear_relu2_fwd(x, w):
    pre = torch.empty((x.shape[0], w.shape[0]), dtype=torch.bfloat16, device=x.device)
    act = torch.empty_like(pre)
    gemm(x, w, epi=EPI_RELU2, out=pre, out2=act)
    return pre, act


def quantize_fp8(x):
    """MXFP8 quantizer kernel; returns the same pair as the definition (the kernel's scale atoms are unpacked)."""
    from . import fp8 as F8
    q, sf = F8.mx_quantize(x, 128)
    return q.view(torch.float8_e4m3fn), F8.mx_scales_from_atoms(sf, x.shape[0], x.shape[1], 128)


def gemm_scaled_fp8(x, w, relu2: bool = False):
    """Quantize both operands to MXFP8 and multiply with tcgen05.mma block scaling (`csrc/cuda/fp8_mx.cu`)."""
    from . import fp8 as F8
    xq, sx = F8.mx_quantize(x, 128)
    wq, sw = F8.mx_quantize(w, F8.mx_tile_n(w.shape[0]))
    if relu2:
        y = torch.empty((x.shape[0], w.shape[0]), dtype=torch.bfloat16, device=x.device)
        act = torch.empty_like(y)
        F8.mx_gemm(xq, sx, wq, sw, y, act)
        return y, act
    return F8.mx_gemm(xq, sx, wq, sw)


def linear_relu2_act_fwd(x, w):
    """act = relu(x @ w^T)^2 only: the pre-activation is never written (its backward uses sqrt(act))."""
    act = torch.empty((x.shape[0], w.shape[0]), dtype=torch.bfloat16, device=x.device)
    gemm(x, w, epi=EPI_RELU2, out=act, out2=act)
    return act


def linear_dgrad_relu2_act(dy, w, act):
    """d(pre) = (dy @ w) * 2 sqrt(act), the backward of act = relu(pre)^2 written in terms of act."""
    return gemm(dy, w, b_mn=True, epi=EPI_DRELU2, r=act, beta=1.0)


def linear_dgrad(dy, w, *, residual=None):
    # dx[M,K] = dy[M,N] @ w[N,K]: B operand is w read MN-major (its K index is contiguous)
    if residual is not None:
        return gemm(dy, w, b_mn=True, epi=EPI_BF16_RES, r=residual, alpha=1.0, beta=1.0)
    return gemm(dy, w, b_mn=True)


def linear_dgrad_relu2(dy, w, pre):
    return gemm(dy, w, b_mn=True, epi=EPI_DRELU2, r=pre)


def linear_wgrad(dy, x, grad, *, accumulate=True):
    # grad[N,K] (+)= dy[M,N]^T @ x[M,K]: both operands are read MN-major
    gemm(dy, x, a_mn=True, b_mn=True, epi=EPI_F32, out=grad, beta=1.0 if accumulate else 0.0)
    return grad


# ---------------------------------------------------------------------------
# Row kernels
# ---------------------------------------------------------------------------
from ..config import LOGIT_SOFTCAP, QK_SCALE, RMS_EPS  # noqa: E402


def _status(t):
    return _C.status_tensor(t.device.index)


def rmsnorm_fwd(x, eps=RMS_EPS):
    y, rstd = _C.rmsnorm_fwd(x, eps)
    return y, rstd


def rmsnorm_fwd_mx(x, eps=RMS_EPS):
    """rmsnorm that also writes its output as MXFP8: (y, rstd, y_e4m3 uint8 [M, K], scale atoms for 128-row tiles).
    The codes and scales equal `fp8.mx_quantize(y, 128)`; the separate pass over y is saved."""
    y, rstd, yq, sf = _C.rmsnorm_fwd_mx(x, eps)
    return y, rstd, yq, sf


def blend_norm_fwd_mx(x, x0, lam_r, lam_0, eps=RMS_EPS):
    """blend + rmsnorm that also writes h as MXFP8: (xr, h, rstd, h_e4m3, scale atoms)."""
    xr, h, rstd, hq, sf = _C.blend_norm_fwd_mx(x, x0, lam_r, lam_0, eps)
    return xr, h, rstd, hq, sf


def rmsnorm_apply(x, rstd):
    return _C.rmsnorm_apply(x, rstd)


def rmsnorm_bwd(x, dy, rstd, residual=None):
    return _C.rmsnorm_bwd(x, dy, rstd, residual)


def add(a, b):
    return _C.add(a, b)


def add_cols(dh, extra):
    _C.add_cols(dh, extra.contiguous())
    return dh


def concat_qkv(dq, dk, dv):
    return torch.cat([dq, dk, dv], dim=1)


def backout_fwd(x, x_backout, lam):
    return _C.backout_fwd(x, x_backout, lam)


def backout_bwd(dy, x_backout, lam):
    dxb, dlam = _C.backout_bwd(dy, x_backout, lam)
    return dy, dxb, dlam[0]


def blend_norm_fwd(x, x0, lam_r, lam_0, eps=RMS_EPS):
    xr, h, rstd = _C.blend_norm_fwd(x, x0, lam_r, lam_0, eps)
    return xr, h, rstd


def blend_bwd(dxr, x, x0, lam_r, lam_0, dx0_acc=None):
    """Returns (dx, dx0, dlam_r, dlam_0). With `dx0_acc` the x0 contribution is accumulated in place
    and returned as the same tensor (one pass instead of blend + add)."""
    if dx0_acc is None:
        dx0 = torch.empty_like(x)
        dx, dlam = _C.blend_bwd(dxr, x, x0, lam_r, lam_0, dx0, False)
    else:
        dx0 = dx0_acc
        dx, dlam = _C.blend_bwd(dxr, x, x0, lam_r, lam_0, dx0, True)
    return dx, dx0, dlam[0], dlam[1]


def norm_blend_bwd(xr, dh, rstd, residual, x, x0, lam_r, lam_0, g_lam_r, g_lam_0, dx0_acc=None, extra=None):
    """One launch for add_cols + rmsnorm_bwd + blend_bwd + the two scalar-gradient adds (see ops.ref)."""
    accumulate = dx0_acc is not None
    dx0 = dx0_acc if accumulate else torch.empty_like(x)
    dx = _C.norm_blend_bwd(xr, dh, rstd, residual, extra, x, x0, lam_r, lam_0, dx0, accumulate, g_lam_r, g_lam_0)
    return dx.view_as(x), dx0


def _fused_heads(a, b):
    """If `b` ([B,T,Hb,D]) starts right after the heads of `a` ([B,T,Ha,D]) in the same token rows, return
    the [B,T,Ha+Hb,D] view covering both, else None."""
    if a.stride() != b.stride() or a.shape[:2] != b.shape[:2] or a.shape[3] != b.shape[3]:
        return None
    if b.data_ptr() != a.data_ptr() + a.shape[2] * a.shape[3] * a.element_size():
        return None
    if a.stride(1) < (a.shape[2] + b.shape[2]) * a.shape[3]:
        return None
    B, T, Ha, D = a.shape
    return a.as_strided((B, T, Ha + b.shape[2], D), a.stride(), a.storage_offset())


def qk_prep_fwd(q_pre, k_pre, cos, sin, eps=RMS_EPS, scale=QK_SCALE, positions=None):
    both = _fused_heads(q_pre, k_pre)
    if both is not None:   # q and k of a fused QKV row: one launch, one output buffer
        out = _C.qk_prep_fwd_one(both, cos, sin, positions, eps, scale)
        H = q_pre.shape[2]
        return out[:, :, :H], out[:, :, H:]
    return (_C.qk_prep_fwd_one(q_pre, cos, sin, positions, eps, scale),
            _C.qk_prep_fwd_one(k_pre, cos, sin, positions, eps, scale))


def qk_prep_bwd(q_pre, k_pre, dq, dk, cos, sin, eps=RMS_EPS, scale=QK_SCALE, out_q=None, out_k=None):
    if out_q is None:
        out_q = torch.empty(dq.shape, dtype=dq.dtype, device=dq.device)
    if out_k is None:
        out_k = torch.empty(dk.shape, dtype=dk.dtype, device=dk.device)
    pre, grad, out = _fused_heads(q_pre, k_pre), _fused_heads(dq, dk), _fused_heads(out_q, out_k)
    if pre is not None and grad is not None and out is not None:
        _C.qk_prep_bwd_one(pre, grad, out, cos, sin, eps, scale)
        return out_q, out_k
    _C.qk_prep_bwd_one(q_pre, dq, out_q, cos, sin, eps, scale)
    _C.qk_prep_bwd_one(k_pre, dk, out_k, cos, sin, eps, scale)
    return out_q, out_k


def value_gate_fwd(h, ve, gate_w, v, head_dim):
    gate = _C.value_gate_fwd(h, ve, gate_w.contiguous(), v, head_dim)   # v updated in place
    return v, gate


def value_gate_fwd_gather(h, ids, table, gate_w, v, head_dim):
    """`value_gate_fwd(h, table[ids], ...)` without materialising the gathered rows (decode)."""
    gate = _C.value_gate_fwd_gather(h, ids, table, gate_w.contiguous(), v, head_dim)   # v updated in place
    return v, gate


def value_gate_bwd(h, ve, gate_w, gate, dv, head_dim):
    dve, dh12, dgw = _C.value_gate_bwd(h, ve, gate_w.contiguous(), gate, dv, head_dim)
    return dve, dh12, dgw


def smear_fwd(emb, gate_w, lam, seq, prev=None):
    x0, sig = _C.smear_fwd(emb, gate_w.contiguous().view(-1), lam, seq, prev)
    return x0, sig


def smear_bwd(emb, gate_w, lam, sig, dx0, seq):
    de, dgw, dlam = _C.smear_bwd(emb, gate_w.contiguous().view(-1), lam, sig, dx0, seq)
    return de, dgw, dlam[0]


def embedding_fwd(ids, table):
    return _C.embedding_fwd(ids.reshape(-1).contiguous(), table)


def embedding_order(ids):
    """(sorted ids, original row of each sorted position) of a stable sort: the fixed summation order of the
    deterministic embedding backward. Computed once per micro-batch and shared by every table of the step."""
    s, perm = torch.sort(ids.reshape(-1), stable=True)
    return s.to(torch.int32).contiguous(), perm.to(torch.int32).contiguous()


def embedding_bwd(ids, dout, dtable, order=None):
    """dtable[ids[m]] += dout[m]. With `order` (from `embedding_order`) the sum runs in a fixed order with one writer
    per table row (bitwise reproducible); without it rows are added with vector atomics in arrival order."""
    if order is not None:
        _C.embedding_bwd_sorted(order[0], order[1], dout, dtable)
    else:
        _C.embedding_bwd(ids.reshape(-1).contiguous(), dout, dtable)
    return dtable


def classifier_fwd_bwd(logits, targets, vocab, *, dlogit_scale, row_scale=None, softcap=LOGIT_SOFTCAP,
                       ignore_index=-1, want_grad=True):
    """In place: when `want_grad` the logits buffer is overwritten with dlogits and returned."""
    ds = None
    if want_grad:
        ds = dlogit_scale if isinstance(dlogit_scale, torch.Tensor) else torch.tensor(
            float(dlogit_scale), dtype=torch.float32, device=logits.device)
        ds = ds.to(torch.float32).reshape(1)
    losses = _C.classifier_fwd_bwd(logits, targets.contiguous(), vocab, ds, row_scale, softcap, ignore_index, want_grad)
    return losses, (logits if want_grad else None)


def linear_wgrad_relu2(dy, pre, grad, *, accumulate=True):
    act = _relu2(pre)
    return linear_wgrad(dy, act, grad, accumulate=accumulate)


def _relu2(pre):
    # recompute act = relu(pre)^2; a GEMM-prologue fusion is not possible with TMA-fed operands,
    # so the activation is rebuilt in one elementwise pass
    return _C.relu2(pre)


def grad_norm_and_clip(grads, clip):
    """`grads` is a list of fp32 tensors; one flat tensor (the whole gradient buffer) is the fast path."""
    if len(grads) == 1:
        out = _C.grad_norm_clip(grads[0].reshape(-1), float(clip if clip else 0.0))
        return out[0], out[1]
    acc = torch.zeros(1, dtype=torch.float64, device=grads[0].device)
    for g in grads:
        _C.sumsq_into(g.reshape(-1), acc)
    norm = acc.sqrt().float()[0]
    if clip and clip > 0:
        scale = torch.where(norm > clip, clip / norm.clamp_min(1e-30), torch.ones_like(norm))
    else:
        scale = torch.ones_like(norm)
    return norm, scale


# ---------------------------------------------------------------------------
# Attention
# ---------------------------------------------------------------------------
def attention_fwd(q, k, v, window_left=-1, scale=None, q_offset=None, variant=2):
    """variant 2 (default): two query tiles per CTA, output accumulated in TMEM; variant 1: one tile per CTA."""
    import math
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    o, lse = _C.attention_fwd(q, k, v, int(window_left), float(scale), -1 if q_offset is None else int(q_offset),
                              _status(q), variant)
    return o, lse


_ds_scratch = {}
_DS_LIMIT_BYTES = int(float(os.environ.get("NANOCHAT_ATTN_DS_GB", "6")) * (1 << 30))


def _ds_workspace(q, k):
    """Scratch for dS^T [B, H, Tk128, Tq128] (bf16), one per device and shape, reused by every layer. None when it
    would exceed NANOCHAT_ATTN_DS_GB (default 6): the backward then recomputes dS for dQ instead of storing it."""
    B, Tq, H, _ = q.shape
    Tk = k.shape[1]
    shape = (B, H, (Tk + 127) // 128 * 128, (Tq + 127) // 128 * 128)
    nbytes = 2 * shape[0] * shape[1] * shape[2] * shape[3]
    if nbytes > _DS_LIMIT_BYTES or _DS_LIMIT_BYTES <= 0:
        return None
    key = (q.device.index, shape)
    ws = _ds_scratch.get(key)
    if ws is None:
        if len(_ds_scratch) > 4:
            _ds_scratch.clear()
        ws = torch.empty(shape, dtype=torch.bfloat16, device=q.device)
        _ds_scratch[key] = ws
    return ws


def attention_bwd(q, k, v, o, lse, do, window_left=-1, scale=None, q_offset=None, out=None):
    """`out` may give (dq, dk, dv) destination views (e.g. column slices of one [M, 3C] buffer)."""
    import math
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    dq, dk, dv = out if out is not None else (None, None, None)
    if dq is None:
        dq = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    if dk is None:
        dk = torch.empty(k.shape, dtype=k.dtype, device=k.device)
    if dv is None:
        dv = torch.empty(v.shape, dtype=v.dtype, device=v.device)
    _C.attention_bwd(q, k, v, o, lse, do, dq, dk, dv, int(window_left), float(scale),
                     -1 if q_offset is None else int(q_offset), _status(q), _ds_workspace(q, k))
    return dq, dk, dv


def adamw_update(master, value, grad, m, v, *, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0):
    gs = grad_scale if isinstance(grad_scale, torch.Tensor) else None
    if gs is None and grad_scale != 1.0:
        gs = torch.tensor(float(grad_scale), dtype=torch.float32, device=master.device)
    _C.adamw_update(master, value, grad, m, v, lr, beta1, beta2, eps, weight_decay, step,
                    None if gs is None else gs.reshape(1))


# small or oddly shaped matrices (the 12-channel value gates) take the PyTorch definition on the device;
# every real matrix goes through optim.muon_cuda.muon_group_step
muon_update = ref.muon_update


# ---------------------------------------------------------------------------
# Paged KV cache
# ---------------------------------------------------------------------------
def kv_append(k_pool, v_pool, page_table, positions, k_new, v_new):
    _C.kv_append(k_pool, v_pool, page_table, positions.contiguous(), k_new, v_new)


def softcap_logits(logits_bf16, vocab, cap):
    """fp32 cap * tanh(logits[:, :vocab] / cap) in one pass over the bf16 logits."""
    return _C.softcap_logits(logits_bf16, int(vocab), float(cap))


def argmax_rows(logits_bf16, vocab):
    """int64 [rows]: argmax over logits[:, :vocab] (lowest index among equal values)."""
    return _C.argmax_rows(logits_bf16, int(vocab))


def decode_prep_append(qk_rows, v_rows, cos, sin, positions, k_pool, v_pool, page_table, num_heads,
                       eps=RMS_EPS, scale=QK_SCALE):
    """Decode prologue in one launch (head_dim 128, one token per sequence): `qk_prep_fwd` of the q and k heads of the
    fused projection rows, k and the value rows appended to the paged cache. Returns q [B, H, D]."""
    return _C.decode_prep_append(qk_rows, v_rows, cos, sin, positions, k_pool, v_pool, page_table, num_heads, eps, scale)


def paged_decode_attention(q, k_pool, v_pool, page_table, seq_lens, window_left=-1, scale=None):
    import math
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    if not (q.stride(2) == 1 and q.stride(1) == q.shape[2] and q.stride(0) % 8 == 0):
        q = q.contiguous()             # the kernel takes any 16-byte aligned stride between sequences
    return _C.paged_decode_attention(q, k_pool, v_pool, page_table, seq_lens, int(window_left), float(scale))


def __getattr__(name):
    # Operators without a kernel are an error on a GPU, not a fallback.
    raise AttributeError(f"ops.cuda has no operator {name!r}")
