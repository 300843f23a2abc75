"""Batched inference over a paged KV cache.

Semantics are those of the reference inference graph (`src/generate.cc:266-412`): the cache holds PREPARED
keys (after QK-norm, RoPE at the absolute position, x1.2) and values AFTER the value-embedding gate, per layer;
every sequence also keeps the normalised embedding of its previous token (the smear needs it at decode time);
RoPE tables follow absolute positions and grow on demand; the backout activation is taken after layer L/2;
the soft-cap is applied to the rows that are sampled from. Differences from the reference are structural only:
the cache is paged (16-token pages from one pool, a page table per sequence), prefill and decode are batched
over sequences, the embedding mix and greedy selection stay on the device (sampling with a temperature draws from
the reference's per-row streams in the host runtime), and on a GPU the decode step can be replayed from a CUDA graph.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from .. import ops
from ..config import LOGIT_SOFTCAP, Config
from ..models.gpt import GPT, _heads

PAGE_SIZE = 16


class PagedKVCache:
    """K/V pools per layer, one page table shared by all layers."""

    def __init__(self, cfg: Config, batch: int, max_seq: int, device, dtype, page_size: int = PAGE_SIZE):
        self.cfg, self.batch, self.max_seq, self.page_size = cfg, batch, max_seq, page_size
        self.pages_per_seq = (max_seq + page_size - 1) // page_size
        n_pages = batch * self.pages_per_seq
        shape = (n_pages, page_size, cfg.num_kv_heads, cfg.head_dim)
        self.k = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(cfg.num_layers)]
        self.v = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(cfg.num_layers)]
        # sequence b owns pages [b*pages_per_seq, (b+1)*pages_per_seq): a static assignment through the table, so
        # the kernels only ever see the indirection
        self.page_table = torch.arange(n_pages, dtype=torch.int32, device=device).view(batch, self.pages_per_seq)
        self.seq_lens = torch.zeros(batch, dtype=torch.int32, device=device)
        self.prev_emb = torch.zeros(batch, cfg.hidden_dim, dtype=dtype, device=device)
        self.has_prev = False

    def reset(self) -> None:
        self.seq_lens.zero_()
        self.has_prev = False

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.k + self.v)


class InferenceEngine:
    def __init__(self, model: GPT, use_cuda_graph: bool = True):
        self.model = model
        self.cfg = model.cfg
        self.device = model.device
        self.dtype = model.dtype
        self._rope_len = 0
        self._cos = self._sin = None
        self.use_cuda_graph = use_cuda_graph and self.device.type == "cuda"
        self._graph = None
        self._graph_key = None
        self._graph_cache = None   # strong reference: the captured graph addresses this cache's tensors

    # ------------------------------------------------------------------ helpers
    def new_cache(self, batch: int, max_seq: int) -> PagedKVCache:
        return PagedKVCache(self.cfg, batch, max_seq, self.device, self.dtype)

    def _rope(self, upto: int):
        if upto > self._rope_len:
            n = max(upto, 2 * self._rope_len, self.cfg.seq_len)
            self._cos, self._sin = ops.build_rope(n, self.cfg.head_dim, self.cfg.rope_base, self.device)
            self._rope_len = n
        return self._cos, self._sin

    # ------------------------------------------------------------------ forward over T new tokens per sequence
    @torch.no_grad()
    def _forward(self, cache: PagedKVCache, tokens: torch.Tensor, decode: bool) -> torch.Tensor:
        """tokens [B, T] appended at positions seq_lens[b] + t. Returns the final normalised hidden states
        [B*T, C]. Prefill requires every sequence of the batch to sit at the same position."""
        cfg, m, P = self.cfg, self.model, self.model.params
        B, T = tokens.shape
        H, KV, D = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        M = B * T
        tok = tokens.reshape(-1).to(torch.int32)
        emb_raw = ops.embedding_fwd(tok, P.v("transformer.wte.weight"))
        emb, _ = ops.rmsnorm_fwd(emb_raw)
        x0, _ = ops.smear_fwd(emb, P.v("smear_gate.weight"), m._lam("smear_lambda"), T,
                              prev=cache.prev_emb if cache.has_prev else None)
        cache.prev_emb.copy_(emb.view(B, T, -1)[:, -1])
        # absolute positions of the new tokens
        pos = cache.seq_lens[:, None] + torch.arange(T, device=self.device, dtype=torch.int32)[None, :]
        kernel_decode = decode and self.device.type == "cuda" and ops.get_mode() == "kernels"
        if decode:
            cos_all, sin_all = self._rope(cache.max_seq)
            cos = sin = None
            if not kernel_decode:      # the kernels index the tables by position themselves
                cos, sin = cos_all[pos.long()], sin_all[pos.long()]       # [B, 1, D/2] gathered per sequence
            t0 = None
        else:
            t0 = int(cache.seq_lens[0].item())
            cos_all, sin_all = self._rope(t0 + T)
            cos, sin = cos_all[t0:t0 + T], sin_all[t0:t0 + T]
        new_lens = cache.seq_lens + T
        fused_prologue = kernel_decode and D == 128 and cache.page_table.shape[0] == B
        pos_flat = pos.reshape(-1).contiguous()
        x = x0
        x_backout = None
        for i in range(cfg.num_layers):
            xr, h, _ = ops.blend_norm_fwd(x, x0, m._lam("resid_lambdas", i), m._lam("x0_lambdas", i))
            wqkv = P.qkv_view(i)
            if wqkv is not None:
                qkv = ops.linear_fwd(h, wqkv)
                q_pre, k_pre = qkv[:, : cfg.query_dim], qkv[:, cfg.query_dim: cfg.query_dim + cfg.kv_dim]
                v = qkv[:, cfg.query_dim + cfg.kv_dim:]
            else:
                q_pre = ops.linear_fwd(h, m._w(i, "attn.c_q"))
                k_pre = ops.linear_fwd(h, m._w(i, "attn.c_k"))
                v = ops.linear_fwd(h, m._w(i, "attn.c_v"))
            if cfg.has_value_embedding(i):
                if fused_prologue:      # the gate kernel reads the embedding rows straight from the table
                    v, _ = ops.cuda_module().value_gate_fwd_gather(h, tok, P.v(f"value_embeds.{i}.weight"),
                                                                   m._w(i, "attn.ve_gate"), v, D)
                else:
                    ve = ops.embedding_fwd(tok, P.v(f"value_embeds.{i}.weight"))
                    v, _ = ops.value_gate_fwd(h, ve, m._w(i, "attn.ve_gate"), v, D)
            wl = cfg.window_left(i)
            if fused_prologue and wqkv is not None:
                # one launch: q / k preparation, k and v appended to their pages; q comes back dense
                q3 = ops.cuda_module().decode_prep_append(qkv, v, cos_all, sin_all, pos_flat, cache.k[i], cache.v[i],
                                                          cache.page_table, H)
                attn = ops.paged_decode_attention(q3, cache.k[i], cache.v[i], cache.page_table, new_lens,
                                                  wl).view(B, 1, H, D)
                x_mid = ops.linear_fwd(attn.reshape(M, H * D), m._w(i, "attn.c_proj"), residual=xr)
                h2, _ = ops.rmsnorm_fwd(x_mid)
                act = ops.linear_relu2_act_fwd(h2, m._w(i, "mlp.c_fc"))
                x = ops.linear_fwd(act, m._w(i, "mlp.c_proj"), residual=x_mid)
                if i == cfg.backout_layer:
                    x_backout = x
                continue
            q4, k4 = _heads(q_pre, B, T, H, D), _heads(k_pre, B, T, KV, D)
            if kernel_decode:
                q, k = ops.cuda_module().qk_prep_fwd(q4, k4, cos_all, sin_all, positions=pos.reshape(-1).contiguous())
            else:
                q, k = ops.qk_prep_fwd(q4, k4, cos, sin)
            v4 = _heads(v, B, T, KV, D)
            ops.kv_append(cache.k[i], cache.v[i], cache.page_table, pos, k, v4)
            if decode:
                attn = ops.paged_decode_attention(q[:, 0], cache.k[i], cache.v[i], cache.page_table,
                                                  new_lens, wl).view(B, 1, H, D)
            elif t0 == 0:
                attn, _ = ops.attention_fwd(q, k, v4, wl)
            else:
                kk = ops.paged_gather(cache.k[i], cache.page_table, t0 + T)
                vv = ops.paged_gather(cache.v[i], cache.page_table, t0 + T)
                attn, _ = ops.attention_fwd(q, kk.contiguous(), vv.contiguous(), wl, q_offset=t0)
            x_mid = ops.linear_fwd(attn.reshape(M, H * D), m._w(i, "attn.c_proj"), residual=xr)
            h2, _ = ops.rmsnorm_fwd(x_mid)
            act = ops.linear_relu2_act_fwd(h2, m._w(i, "mlp.c_fc"))
            x = ops.linear_fwd(act, m._w(i, "mlp.c_proj"), residual=x_mid)
            if i == cfg.backout_layer:
                x_backout = x
        cache.seq_lens.add_(T)
        cache.has_prev = True
        x_pre = ops.backout_fwd(x, x_backout, m._lam("backout_lambda"))
        xn, _ = ops.rmsnorm_fwd(x_pre)
        return xn

    def _greedy(self, xn_rows: torch.Tensor) -> torch.Tensor:
        """Token ids of the largest logit per row (int64). The soft cap is monotonic, so on the kernel path the
        arg-max is taken over the bf16 logits directly and the fp32 capped copy is never made."""
        lg = ops.linear_fwd(xn_rows.contiguous(), self.model.params.v("lm_head.weight"))
        if lg.is_cuda and ops.get_mode() == "kernels":
            return ops.cuda_module().argmax_rows(lg, self.cfg.vocab_size)
        return lg[:, : self.cfg.vocab_size].float().argmax(dim=-1)

    def _logits(self, xn_rows: torch.Tensor) -> torch.Tensor:
        """Soft-capped logits over the real vocabulary, fp32."""
        lg = ops.linear_fwd(xn_rows.contiguous(), self.model.params.v("lm_head.weight"))
        if lg.is_cuda and ops.get_mode() == "kernels" and self.cfg.vocab_size % 2 == 0:
            return ops.cuda_module().softcap_logits(lg, self.cfg.vocab_size, LOGIT_SOFTCAP)
        z = lg[:, : self.cfg.vocab_size].float()
        return LOGIT_SOFTCAP * torch.tanh(z / LOGIT_SOFTCAP)

    # ------------------------------------------------------------------ public steps
    @torch.no_grad()
    def prefill(self, cache: PagedKVCache, tokens: torch.Tensor) -> torch.Tensor:
        """tokens [B, T] (same length for every sequence). Returns logits of the last position [B, vocab]."""
        B, T = tokens.shape
        if int(cache.seq_lens.max().item()) + T > cache.max_seq:
            raise ValueError("prompt does not fit the KV cache")
        xn = self._forward(cache, tokens, decode=False)
        return self._logits(xn.view(B, T, -1)[:, -1])

    @torch.no_grad()
    def decode(self, cache: PagedKVCache, tokens: torch.Tensor, greedy: bool = False) -> torch.Tensor:
        """tokens [B]: one new token per sequence. Returns logits [B, vocab], or with `greedy` the next token ids
        [B] (int64) without materialising the logits in fp32."""
        pdl = self.device.type == "cuda" and ops.get_mode() == "kernels"
        if pdl:     # the step's small kernels are launched so that each is resident before the one before it ends
            ops.cuda_module()._C.set_pdl_enabled(True)
        try:
            xn = self._forward(cache, tokens.view(-1, 1), decode=True)
            return self._greedy(xn) if greedy else self._logits(xn)
        finally:
            if pdl:
                ops.cuda_module()._C.set_pdl_enabled(False)

    # ------------------------------------------------------------------ CUDA-graph decode
    @torch.no_grad()
    def decode_graphed(self, cache: PagedKVCache, tokens: torch.Tensor, greedy: bool = False) -> torch.Tensor:
        """Same as `decode`; the step is captured once per (cache, batch) and replayed. Falls back to the eager
        step when capture is not possible."""
        if not self.use_cuda_graph:
            return self.decode(cache, tokens, greedy)
        # The graph bakes in the addresses of this cache's pools, page table, lengths and previous-embedding slot,
        # so it is valid for this cache object only. The engine keeps the cache alive while the graph exists and
        # compares by identity: an `id()` can be reused by a new cache once the old one is freed.
        key = (tokens.shape[0], cache.max_seq, bool(greedy))
        if self._graph_cache is not cache or self._graph_key != key:
            self._graph = None
            self._graph_key = key
            self._graph_cache = cache
            try:
                self._static_tok = tokens.clone()
                # warm up on a side stream (allocations, tensor-map cache), restoring the cache state afterwards
                lens, prev, had = cache.seq_lens.clone(), cache.prev_emb.clone(), cache.has_prev
                s = torch.cuda.Stream()
                s.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(s):
                    self.decode(cache, self._static_tok, greedy)
                torch.cuda.current_stream().wait_stream(s)
                cache.seq_lens.copy_(lens)
                cache.prev_emb.copy_(prev)
                cache.has_prev = had
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self._static_out = self.decode(cache, self._static_tok, greedy)
                cache.seq_lens.copy_(lens)
                cache.prev_emb.copy_(prev)
                cache.has_prev = had
                self._graph = g
            except Exception:
                self._graph = None
                self._graph_cache = None
                self.use_cuda_graph = False
                torch.cuda.synchronize()
                return self.decode(cache, tokens, greedy)
        self._static_tok.copy_(tokens)
        self._graph.replay()
        cache.has_prev = True
        return self._static_out


# ---------------------------------------------------------------------------------------------------------
# Sampling on the device
# ---------------------------------------------------------------------------------------------------------
def sample(logits: torch.Tensor, temperature: float, top_k: int, seed: int, rows: torch.Tensor, step: int):
    """Greedy for temperature <= 0. Otherwise temperature / top-k sampling with the streams of the reference
    (src/generate.cc:54, 614-669) as the native engine consumes them: row r owns xoshiro256**(MixSeed(seed, r)) and
    its `step`-th draw picks the `step`-th sampled token by walking the cumulative distribution. The draw itself
    runs in the host runtime (`ncb_sample_rows`) on a copy of the logits, so a seed gives the same rollout on this
    engine and on the native ones wherever their logits agree."""
    if not temperature > 0.0:
        return logits.argmax(dim=-1)
    import ctypes
    import numpy as np
    from ..data import native
    L = native.lib()
    L.ncb_sample_rows.restype = None
    L.ncb_sample_rows.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_int,
                                  ctypes.c_uint64, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]
    host = np.ascontiguousarray(logits.detach().float().cpu().numpy())
    ids = np.ascontiguousarray(rows.detach().cpu().numpy().astype(np.int64))
    out = np.empty(host.shape[0], dtype=np.int32)
    L.ncb_sample_rows(host.ctypes.data, host.shape[0], host.shape[1], float(temperature), int(top_k),
                      ctypes.c_uint64(int(seed) & 0xFFFFFFFFFFFFFFFF), ids.ctypes.data, int(step), out.ctypes.data)
    return torch.from_numpy(out.astype(np.int64)).to(logits.device)


@dataclass
class GenerateParams:
    """Mirror of the reference's `GenerateParams` (include/nanochat/model.h:244-299)."""
    num_samples: int = 1
    max_tokens: int = 64
    temperature: float = 0.0
    top_k: int = 0
    seed: int = 0
    stop_id: int = -1
    bos_id: int = -1
    stop_ids: Sequence[int] = ()


@dataclass
class GeneratedSequence:
    tokens: List[int]   # prompt followed by the generated tokens (the terminal token is not included)
    mask: List[int]     # 1 = sampled, 0 = prompt or forced


@torch.no_grad()
def generate_multi(engine: InferenceEngine, prompts: torch.Tensor, params: GenerateParams,
                   forced: Optional[callable] = None) -> List[GeneratedSequence]:
    """prompts [N, L] (equal lengths). Every prompt is decoded `num_samples` times: row r = prompt r // S. A row
    stops at `stop_id`, `bos_id`, any of `stop_ids`, or `max_tokens` (reference src/generate.cc:458-576).
    `forced(row, tokens_so_far)` may return a token to force at the next position (tool output injection)."""
    N, Lp = prompts.shape
    S = max(1, params.num_samples)
    rows = N * S
    dev = engine.device
    cache = engine.new_cache(rows, Lp + params.max_tokens + 1)
    tok = prompts.to(dev).repeat_interleave(S, dim=0)
    logits = engine.prefill(cache, tok)
    out = [GeneratedSequence(tok[r].tolist(), [0] * Lp) for r in range(rows)]
    live = torch.ones(rows, dtype=torch.bool, device=dev)
    row_ids = torch.arange(rows, device=dev)
    stops = {s for s in (params.stop_id, params.bos_id, *params.stop_ids) if s is not None and s >= 0}
    stop_t = torch.tensor(sorted(stops), device=dev, dtype=torch.int64) if stops else None
    # greedy decoding without forced tokens never needs the logits after the prefill: the step returns token ids
    greedy_ids = (not params.temperature > 0.0) and forced is None
    pred = None
    for step in range(params.max_tokens):
        nxt = pred if pred is not None else sample(logits, params.temperature, params.top_k, params.seed, row_ids, step)
        was_forced = [False] * rows
        if forced is not None:
            host = nxt.tolist()
            for r in range(rows):
                if bool(live[r]):
                    f = forced(r, out[r].tokens)
                    if f is not None:
                        host[r], was_forced[r] = int(f), True
            nxt = torch.tensor(host, device=dev)
        if stop_t is not None:
            hit = (nxt[:, None] == stop_t[None, :]).any(dim=1)
            live = live & ~hit
        if not bool(live.any()):
            break
        host_nxt, host_live = nxt.tolist(), live.tolist()
        for r in range(rows):
            if host_live[r]:
                out[r].tokens.append(host_nxt[r])
                out[r].mask.append(0 if was_forced[r] else 1)
        if step + 1 == params.max_tokens:
            break
        if greedy_ids:
            pred = engine.decode_graphed(cache, nxt, greedy=True)
        else:
            logits = engine.decode_graphed(cache, nxt) if forced is None else engine.decode(cache, nxt)
    return out


def generate(engine: InferenceEngine, prompt: Sequence[int], params: GenerateParams, forced=None):
    """One prompt, `num_samples` continuations (reference `GenerateBatch`)."""
    p = torch.tensor([list(prompt)], dtype=torch.int64)
    return generate_multi(engine, p, params, forced)
