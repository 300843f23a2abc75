"""The nanochat training graph with a hand-written forward and backward.

Same graph as the reference (`src/model.cc:894-1180`, `src/ops.cc:1454-1675`):

    e   = rmsnorm(wte[token]);  x = smear(e);  x0 = x
    per layer i:
        xr    = resid[i]*x + x0_lambda[i]*x0          h = rmsnorm(xr)
        q,k,v = h Wq^T, h Wk^T, h Wv^T                (one fused QKV GEMM)
        v    += 3*sigmoid(h[:, :12] Wg^T) * value_embeds[i][token]   (alternating layers)
        q,k   = 1.2 * rope(rmsnorm_head(q)), 1.2 * rope(rmsnorm_head(k))
        a     = attention(q, k, v; causal, left window on S layers, GQA)
        x_mid = xr + a Wo^T                            h2 = rmsnorm(x_mid)
        x     = x_mid + relu(h2 Wfc^T)^2 Wproj^T
        remember x after layer L/2
    x = x - backout_lambda * x_{L/2};  logits = rmsnorm(x) Wlm^T
    loss = mean over valid targets of CE(15*tanh(logits/15))

Nothing here uses autograd: every operator has an explicit backward, the weight
gradients are accumulated by the GEMM epilogue straight into the flat fp32 gradient
buffer, and the LM head is processed in row chunks (GEMM -> softcap/CE forward and
backward in place -> dgrad/wgrad) so full logits never exist. The per-layer hook
`on_layer_grads_ready(layer)` fires as soon as a block's weight gradients are final,
which is what the data-parallel engine overlaps its reduce-scatter with.
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional

import torch

from .. import ops
from ..config import LOGIT_SOFTCAP, QK_SCALE, RMS_EPS, Config
from .params import ParamStore, init_weights


class GPT:
    def __init__(self, cfg: Config, device="cpu", dtype: torch.dtype = torch.bfloat16, seed: int = 0,
                 init: bool = True, head_chunk_rows: int = 11264, allocator=None, fp8=False):
        """`fp8`: run the forward QKV and MLP up-projection products in E4M3 with bf16 outputs; attention, norms,
        the projections with fused residuals, the LM head and the whole backward stay in bf16. "mx" (or True):
        MXFP8, one power-of-two scale per row and 32 K elements applied inside the MMA. "block": fp32 scales per
        1x128 activation block and 128x128 weight block, promoted on the CUDA cores. Call `refresh_fp8()` after
        every optimizer step."""
        cfg.validate()
        self.cfg = cfg
        self.device = torch.device(device)
        self.dtype = dtype
        self.params = ParamStore(cfg, self.device, dtype, allocator=allocator)
        if init:
            init_weights(self.params, seed)
        import os as _os0
        # rows of logits alive at once. 11264 = 44 x 256: with the 1280-wide dgrad output (5 column tiles) a chunk is
        # 220 tile pairs, 2.97 rounds over 74 CTA pairs; 8192 gave 160 = 2.16 rounds, a third of the last one idle.
        self.head_chunk_rows = int(_os0.environ.get("NANOCHAT_HEAD_CHUNK_ROWS", head_chunk_rows))
        self._rope: Dict[int, tuple] = {}
        self._saved: Optional[dict] = None
        self.on_layer_grads_ready: Optional[Callable[[int], None]] = None
        self.on_head_grads_ready: Optional[Callable[[], None]] = None
        self.on_embed_grads_ready: Optional[Callable[[], None]] = None
        import os as _os3
        # False: rebuild the normalised activations in the backward (saves memory)
        self.keep_normed = _os3.environ.get("NANOCHAT_KEEP_NORMED", "1") != "0"
        # True: the MLP keeps act = relu(pre)^2 only; False: keeps pre and rebuilds act for the weight gradient
        self.mlp_keep_act = _os3.environ.get("NANOCHAT_MLP_KEEP_ACT", "1") != "0"
        self.phase_event = None  # a CUDA event recorded between the forward trunk and the head / backward
        # Weight-gradient products are off the critical path of the backward (nothing in the backward reads them),
        # so they run on a second stream: a persistent GEMM CTA per SM leaves most thread slots free, and the
        # memory-bound row kernels of the critical path run beside it instead of after it.
        import os as _os2
        self._wgrad_stream = (torch.cuda.Stream(self.device) if self.device.type == "cuda" and
                              _os2.environ.get("NANOCHAT_WGRAD_STREAM", "1") != "0" else None)
        if fp8 not in (False, None, True, "mx", "block"):
            raise ValueError(f"fp8 must be False, True, 'mx' or 'block', got {fp8!r}")
        self.fp8 = bool(fp8) and self.device.type == "cuda"
        self.fp8_mode = ("block" if fp8 == "block" else "mx") if self.fp8 else None
        # bitwise-reproducible embedding gradients (sorted, single-writer sums instead of atomics)
        import os as _os
        self.deterministic_embedding = _os.environ.get("NANOCHAT_DETERMINISTIC", "0") == "1"
        self._fp8_w: Dict[str, object] = {}
        if self.fp8:
            self.refresh_fp8()

    def _off_path(self, fn, *inputs) -> None:
        """Runs `fn` (a weight-gradient product reading `inputs`) on the side stream, after everything issued so far."""
        side = self._wgrad_stream
        if side is None:
            fn()
            return
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            fn()
        for t in inputs:
            t.record_stream(side)  # the allocator must not hand the block out again before the side stream is done

    def _join_side(self, event=None) -> None:
        """The current stream waits for the side stream (or for `event` recorded on it)."""
        if self._wgrad_stream is not None:
            cur = torch.cuda.current_stream(self.device)
            if event is not None:
                cur.wait_event(event)
            else:
                cur.wait_stream(self._wgrad_stream)

    def refresh_fp8(self) -> None:
        """Re-quantize the fp8 weight copies from the bf16 compute copy (after an optimizer step)."""
        if not self.fp8:
            return
        from ..ops import fp8 as F8
        cfg = self.cfg
        for i in range(cfg.num_layers):
            wqkv = self.params.qkv_view(i)
            fc = self._w(i, "mlp.c_fc")
            for key, w in ((f"qkv{i}", wqkv), (f"fc{i}", fc)):
                if w is None or w.shape[1] % 128 or w.shape[0] % (8 if self.fp8_mode == "mx" else 128):
                    continue
                if key in self._fp8_w:
                    self._fp8_w[key].refresh(w)
                else:
                    self._fp8_w[key] = F8.MxWeight(w) if self.fp8_mode == "mx" else F8.Fp8Weight(w)

    # ------------------------------------------------------------------
    def rope(self, seq: int):
        if seq not in self._rope:
            self._rope[seq] = ops.build_rope(seq, self.cfg.head_dim, self.cfg.rope_base, self.device)
        return self._rope[seq]

    def _w(self, layer: int, name: str):
        return self.params.v(f"transformer.h.{layer}.{name}.weight")

    def _g(self, layer: int, name: str):
        return self.params.g(f"transformer.h.{layer}.{name}.weight")

    def _lam(self, name: str, i: Optional[int] = None):
        t = self.params.m(name)
        return t[i] if i is not None else t[0]

    # ------------------------------------------------------------------
    # forward pieces
    # ------------------------------------------------------------------
    def _embed(self, tokens: torch.Tensor, B: int, T: int, save: Optional[dict], prev=None):
        P = self.params
        emb_raw = ops.embedding_fwd(tokens, P.v("transformer.wte.weight"))
        emb, rstd_e = ops.rmsnorm_fwd(emb_raw)
        x0, sig = ops.smear_fwd(emb, P.v("smear_gate.weight"), self._lam("smear_lambda"), T, prev=prev)
        if save is not None:
            save.update(emb_raw=emb_raw, emb=emb, rstd_e=rstd_e, sig=sig)
        return x0, emb

    def _block_fwd(self, i: int, x, x0, tokens, B: int, T: int, cos, sin, save: Optional[dict]):
        cfg, P = self.cfg, self.params
        H, KV, D = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        M = B * T
        wqkv = P.qkv_view(i)
        hq = None
        fuse_q = self.fp8_mode == "mx" and cfg.hidden_dim % 128 == 0 and ops.get_mode() == "kernels"
        if fuse_q and (f"qkv{i}" in self._fp8_w):
            from ..ops import fp8 as F8
            # the norm kernel writes h a second time as MXFP8: no separate quantizer pass
            xr, h, rstd1, hq0, hq1 = ops.cuda_module().blend_norm_fwd_mx(x, x0, self._lam("resid_lambdas", i),
                                                                        self._lam("x0_lambdas", i))
            hq = (hq0, hq1)
        else:
            xr, h, rstd1 = ops.blend_norm_fwd(x, x0, self._lam("resid_lambdas", i), self._lam("x0_lambdas", i))
        if hq is None and self.fp8 and (f"qkv{i}" in self._fp8_w):
            from ..ops import fp8 as F8
            hq = F8.mx_quantize(h, 128) if self.fp8_mode == "mx" else F8.quantize_rows(h)
        if hq is not None:
            w8 = self._fp8_w[f"qkv{i}"]
            qkv = (F8.mx_gemm if self.fp8_mode == "mx" else F8.fp8_gemm)(hq[0], hq[1], w8.q, w8.s)
            q_pre = qkv[:, : cfg.query_dim]
            k_pre = qkv[:, cfg.query_dim: cfg.query_dim + cfg.kv_dim]
            v = qkv[:, cfg.query_dim + cfg.kv_dim:]
        elif wqkv is not None:
            qkv = ops.linear_fwd(h, wqkv)
            q_pre = qkv[:, : cfg.query_dim]
            k_pre = qkv[:, cfg.query_dim: cfg.query_dim + cfg.kv_dim]
            v = qkv[:, cfg.query_dim + cfg.kv_dim:]
        else:
            q_pre = ops.linear_fwd(h, self._w(i, "attn.c_q"))
            k_pre = ops.linear_fwd(h, self._w(i, "attn.c_k"))
            v = ops.linear_fwd(h, self._w(i, "attn.c_v"))
        ve = gate = None
        if cfg.has_value_embedding(i):
            ve = ops.embedding_fwd(tokens, P.v(f"value_embeds.{i}.weight"))
            v, gate = ops.value_gate_fwd(h, ve, self._w(i, "attn.ve_gate"), v, D)
        q, k = ops.qk_prep_fwd(_heads(q_pre, B, T, H, D), _heads(k_pre, B, T, KV, D), cos, sin)
        v4 = _heads(v, B, T, KV, D)
        attn, lse = ops.attention_fwd(q, k, v4, cfg.window_left(i))
        x_mid = ops.linear_fwd(attn.view(M, H * D), self._w(i, "attn.c_proj"), residual=xr)
        h2q = None
        if fuse_q and (f"fc{i}" in self._fp8_w):
            h2, rstd2, q0, q1 = ops.cuda_module().rmsnorm_fwd_mx(x_mid)
            h2q = (q0, q1)
        else:
            h2, rstd2 = ops.rmsnorm_fwd(x_mid)
        if self.fp8 and (f"fc{i}" in self._fp8_w):
            from ..ops import fp8 as F8
            w8 = self._fp8_w[f"fc{i}"]
            if self.fp8_mode == "mx" and self.mlp_keep_act:
                h2q = h2q if h2q is not None else F8.mx_quantize(h2, 128)
                act = torch.empty((M, w8.q.shape[0]), dtype=torch.bfloat16, device=h2.device)
                F8.mx_gemm(h2q[0], h2q[1], w8.q, w8.s, act, act)      # only relu(pre)^2 is stored
                pre = None
            elif self.fp8_mode == "mx":
                h2q = h2q if h2q is not None else F8.mx_quantize(h2, 128)
                pre = torch.empty((M, w8.q.shape[0]), dtype=torch.bfloat16, device=h2.device)
                act = torch.empty_like(pre)
                F8.mx_gemm(h2q[0], h2q[1], w8.q, w8.s, pre, act)
            else:
                pre, act = F8.linear_fwd_fp8(h2, w8, relu2=True)
        else:
            if self.mlp_keep_act:
                pre, act = None, ops.linear_relu2_act_fwd(h2, self._w(i, "mlp.c_fc"))
            else:
                pre, act = ops.linear_relu2_fwd(h2, self._w(i, "mlp.c_fc"))
        x_out = ops.linear_fwd(act, self._w(i, "mlp.c_proj"), residual=x_mid)
        if save is not None:
            save["layers"].append(dict(x=x, xr=xr, rstd1=rstd1, q_pre=q_pre, k_pre=k_pre, q=q, k=k, v=v4,
                                       ve=ve, gate=gate, attn=attn, lse=lse, x_mid=x_mid, rstd2=rstd2,
                                       pre=pre, act=act if pre is None else None,
                                       # the normalised inputs of the QKV and MLP products are kept for their weight
                                       # gradients (2 x M x hidden per layer) instead of being rebuilt from x and rstd
                                       h=h if self.keep_normed else None, h2=h2 if self.keep_normed else None))
        return x_out

    def _trunk(self, tokens, B, T, save):
        cfg = self.cfg
        cos, sin = self.rope(T)
        x0, _ = self._embed(tokens, B, T, save)
        x = x0
        x_backout = None
        for i in range(cfg.num_layers):
            x = self._block_fwd(i, x, x0, tokens, B, T, cos, sin, save)
            if i == cfg.backout_layer:
                x_backout = x
        x_pre = ops.backout_fwd(x, x_backout, self._lam("backout_lambda"))
        xn, rstd_f = ops.rmsnorm_fwd(x_pre)
        if save is not None:
            save.update(x0=x0, x_last=x, x_backout=x_backout, x_pre=x_pre, rstd_f=rstd_f, cos=cos, sin=sin)
        return xn

    # ------------------------------------------------------------------
    # LM head: chunked GEMM + softcap/CE (+ backward in the same sweep)
    # ------------------------------------------------------------------
    def _head(self, xn, targets, *, dlogit_scale: Optional[torch.Tensor], row_scale=None,
              want_losses: bool = False):
        """Returns (loss_sum 0-d fp32, dxn or None, losses or None). When `dlogit_scale` is
        given the head also accumulates the lm_head gradient and returns d(xn)."""
        cfg, P = self.cfg, self.params
        W = P.v("lm_head.weight")
        M = xn.shape[0]
        chunk = min(self.head_chunk_rows, M)
        want_grad = dlogit_scale is not None
        dxn = torch.empty_like(xn) if want_grad else None
        loss_sum = torch.zeros((), dtype=torch.float32, device=xn.device)
        all_losses = torch.empty(M, dtype=torch.float32, device=xn.device) if want_losses else None
        for a in range(0, M, chunk):
            b = min(a + chunk, M)
            logits = ops.linear_fwd(xn[a:b], W)
            losses, dlogits = ops.classifier_fwd_bwd(
                logits, targets[a:b], cfg.vocab_size, dlogit_scale=dlogit_scale,
                row_scale=None if row_scale is None else row_scale[a:b], want_grad=want_grad)
            loss_sum += losses.sum()
            if want_losses:
                all_losses[a:b] = losses
            if want_grad:
                dxn[a:b] = ops.linear_dgrad(dlogits, W)
                ops.linear_wgrad(dlogits, xn[a:b], P.g("lm_head.weight"), accumulate=True)
        return loss_sum, dxn, all_losses

    # ------------------------------------------------------------------
    # public: evaluation forward
    # ------------------------------------------------------------------
    @torch.no_grad()
    def forward_loss(self, tokens: torch.Tensor, targets: torch.Tensor, return_rows: bool = False):
        """Mean CE over valid targets (reference `ForwardLoss`, src/model.cc:828-844)."""
        B, T = tokens.shape
        tok = tokens.reshape(-1).to(torch.int32)
        tgt = targets.reshape(-1).to(torch.int32)
        xn = self._trunk(tok, B, T, None)
        loss_sum, _, rows = self._head(xn, tgt, dlogit_scale=None, want_losses=return_rows)
        valid = (tgt != -1).sum().clamp_min(1)
        loss = loss_sum / valid.float()
        return (loss, rows) if return_rows else loss

    @torch.no_grad()
    def logits(self, tokens: torch.Tensor) -> torch.Tensor:
        """Raw (un-capped) logits [B, T, vocab] in fp32; for tests and small inputs."""
        B, T = tokens.shape
        xn = self._trunk(tokens.reshape(-1).to(torch.int32), B, T, None)
        lg = ops.linear_fwd(xn, self.params.v("lm_head.weight"))
        return lg[:, : self.cfg.vocab_size].float().view(B, T, -1)

    # ------------------------------------------------------------------
    # public: training forward + backward
    # ------------------------------------------------------------------
    @torch.no_grad()
    def forward_backward(self, tokens: torch.Tensor, targets: torch.Tensor, grad_scale: float = 1.0,
                         row_weights: Optional[torch.Tensor] = None,
                         divisor: Optional[float] = None) -> torch.Tensor:
        """Accumulates d(loss*grad_scale)/d(param) into the flat gradient and returns the
        micro-batch mean loss (0-d fp32 tensor, still on the device).

        `row_weights` ([B*T] fp32) and `divisor` give the weighted backward of the RL step
        (reference `BackwardWeighted`): dlogits are scaled per row and normalised by
        `divisor` instead of the valid-target count.
        """
        cfg, P = self.cfg, self.params
        B, T = tokens.shape
        M = B * T
        tok = tokens.reshape(-1).to(torch.int32)
        tgt = targets.reshape(-1).to(torch.int32)
        order = ops.embedding_order(tok) if self.deterministic_embedding else None
        save: dict = {"layers": []}
        xn = self._trunk(tok, B, T, save)
        if self.phase_event is not None:  # end of the forward trunk (the head runs forward and backward fused)
            self.phase_event.record()
        valid = (tgt != -1).sum().clamp_min(1).float()
        denom = valid if divisor is None else torch.full_like(valid, float(divisor))
        dscale = (grad_scale / denom)
        loss_sum, dxn, _ = self._head(xn, tgt, dlogit_scale=dscale, row_scale=row_weights)
        if self.on_head_grads_ready is not None:
            self.on_head_grads_ready()
        loss = loss_sum / valid

        # ---- backward through the tail --------------------------------
        dx_pre = ops.rmsnorm_bwd(save["x_pre"], dxn, save["rstd_f"])
        del dxn
        lam_b = self._lam("backout_lambda")
        dx, dxb, dlam_b = ops.backout_bwd(dx_pre, save["x_backout"], lam_b)
        P.g("backout_lambda").add_(dlam_b)
        del dx_pre
        x0 = save["x0"]
        dx0 = None
        cos, sin = save["cos"], save["sin"]
        H, KV, D = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        pending = None
        for i in reversed(range(cfg.num_layers)):
            s = save["layers"][i]
            if i == cfg.backout_layer:
                dx = ops.add(dx, dxb)
                dxb = None
            # MLP
            if s["act"] is not None:  # the activation was saved instead of the pre-activation: nothing to recompute
                self._off_path(lambda: ops.linear_wgrad(dx, s["act"], self._g(i, "mlp.c_proj")), dx, s["act"])
                dpre = ops.linear_dgrad_relu2_act(dx, self._w(i, "mlp.c_proj"), s["act"])
            else:
                self._off_path(lambda: ops.linear_wgrad_relu2(dx, s["pre"], self._g(i, "mlp.c_proj")), dx, s["pre"])
                dpre = ops.linear_dgrad_relu2(dx, self._w(i, "mlp.c_proj"), s["pre"])
            h2 = s["h2"] if s["h2"] is not None else ops.rmsnorm_apply(s["x_mid"], s["rstd2"])
            self._off_path(lambda: ops.linear_wgrad(dpre, h2, self._g(i, "mlp.c_fc")), dpre, h2)
            dh2 = ops.linear_dgrad(dpre, self._w(i, "mlp.c_fc"))
            del dpre, h2
            dx_mid = ops.rmsnorm_bwd(s["x_mid"], dh2, s["rstd2"], residual=dx)
            del dh2
            # attention output projection
            attn2 = s["attn"].view(M, H * D)
            self._off_path(lambda: ops.linear_wgrad(dx_mid, attn2, self._g(i, "attn.c_proj")), dx_mid, attn2)
            dattn = ops.linear_dgrad(dx_mid, self._w(i, "attn.c_proj"))
            qd, kd = cfg.query_dim, cfg.kv_dim
            dqkv = torch.empty(M, qd + 2 * kd, dtype=dx_mid.dtype, device=dx_mid.device)
            dv4 = _heads(dqkv[:, qd + kd:], B, T, KV, D)
            dqk = torch.empty(M, qd + kd, dtype=dx_mid.dtype, device=dx_mid.device)
            dq, dk, _ = ops.attention_bwd(s["q"], s["k"], s["v"], s["attn"], s["lse"], dattn.view(B, T, H, D),
                                          cfg.window_left(i),
                                          out=(_heads(dqk[:, :qd], B, T, H, D), _heads(dqk[:, qd:], B, T, KV, D), dv4))
            del dattn
            ops.qk_prep_bwd(_heads(s["q_pre"], B, T, H, D), _heads(s["k_pre"], B, T, KV, D), dq, dk, cos, sin,
                            out_q=_heads(dqkv[:, :qd], B, T, H, D), out_k=_heads(dqkv[:, qd:qd + kd], B, T, KV, D))
            del dq, dk, dqk
            h = s["h"] if s["h"] is not None else ops.rmsnorm_apply(s["xr"], s["rstd1"])
            dv2 = dqkv[:, qd + kd:]
            dh12 = None
            if cfg.has_value_embedding(i):
                dve, dh12, dgw = ops.value_gate_bwd(h, s["ve"], self._w(i, "attn.ve_gate"), s["gate"], dv2, D)
                self._g(i, "attn.ve_gate").add_(dgw)
                ops.embedding_bwd(tok, dve, P.g(f"value_embeds.{i}.weight"), order=order)
                del dve
            gqkv = P.qkv_view(i, "g")
            wqkv = P.qkv_view(i)
            if gqkv is not None:
                self._off_path(lambda: ops.linear_wgrad(dqkv, h, gqkv), dqkv, h)
                dh = ops.linear_dgrad(dqkv, wqkv)
            else:
                def _three():
                    ops.linear_wgrad(dqkv[:, :qd], h, self._g(i, "attn.c_q"))
                    ops.linear_wgrad(dqkv[:, qd:qd + kd], h, self._g(i, "attn.c_k"))
                    ops.linear_wgrad(dqkv[:, qd + kd:], h, self._g(i, "attn.c_v"))
                self._off_path(_three, dqkv, h)
                dh = ops.linear_dgrad(dqkv[:, :qd], self._w(i, "attn.c_q"))
                dh = ops.linear_dgrad(dqkv[:, qd:qd + kd], self._w(i, "attn.c_k"), residual=dh)
                dh = ops.linear_dgrad(dqkv[:, qd + kd:], self._w(i, "attn.c_v"), residual=dh)
            del dqkv, dv2, dv4
            # norm backward, blend backward, the gate's 12 columns and both scalar gradients in one launch
            dx, dx0 = ops.norm_blend_bwd(s["xr"], dh, s["rstd1"], dx_mid, s["x"], x0, self._lam("resid_lambdas", i),
                                         self._lam("x0_lambdas", i), P.g("resid_lambdas")[i:i + 1],
                                         P.g("x0_lambdas")[i:i + 1], dx0_acc=dx0, extra=dh12)
            del dh, dx_mid, h
            save["layers"][i] = None
            if self.on_layer_grads_ready is not None:
                # a layer is announced one layer late, once its side-stream products are known to be complete,
                # so the wait never stalls the critical path
                if pending is not None:
                    self._join_side(pending[1])
                    self.on_layer_grads_ready(pending[0])
                done = self._wgrad_stream.record_event() if self._wgrad_stream is not None else None
                pending = (i, done)
        if pending is not None:
            self._join_side(pending[1])
            self.on_layer_grads_ready(pending[0])
        # ---- embedding side --------------------------------------------
        dx0 = ops.add(dx0, dx)
        de, dgw, dlam = ops.smear_bwd(save["emb"], P.v("smear_gate.weight"), self._lam("smear_lambda"),
                                      save["sig"], dx0, T)
        P.g("smear_gate.weight").view(-1).add_(dgw)
        P.g("smear_lambda").add_(dlam)
        de_raw = ops.rmsnorm_bwd(save["emb_raw"], de, save["rstd_e"])
        ops.embedding_bwd(tok, de_raw, P.g("transformer.wte.weight"), order=order)
        self._join_side()
        if self.on_embed_grads_ready is not None:
            self.on_embed_grads_ready()
        self._saved = None
        return loss

    # ------------------------------------------------------------------
    def zero_grad(self):
        self.params.zero_grad()

    def num_params(self) -> int:
        return self.params.num_params()

    def state_dict(self) -> Dict[str, torch.Tensor]:
        return {s.name: self.params.m(s.name) for s in self.params.specs}

    def load_state_dict(self, sd: Dict[str, torch.Tensor]) -> None:
        for s in self.params.specs:
            self.params.m(s.name).copy_(sd[s.name].to(torch.float32).view(s.shape))
        self.params.sync_compute()


def _heads(x2d: torch.Tensor, B: int, T: int, H: int, D: int) -> torch.Tensor:
    """[M, >=H*D] (possibly a column slice of a wider row) -> [B, T, H, D] strided view."""
    return x2d.as_strided((B, T, H, D), (T * x2d.stride(0), x2d.stride(0), D, 1), x2d.storage_offset())
