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


class PageAllocator:
    """Free list over the pages of one pool. Pages are handed out on demand and come back when a sequence is reset
    or, on windowed layers, when every key of the page has left the attention window."""

    def __init__(self, num_pages: int):
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, -1, -1))   # stack: page 0 first

    @property
    def available(self) -> int:
        return len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise MemoryError("KV page pool exhausted")
        return self._free.pop()

    def release(self, page: int) -> None:
        self._free.append(page)


class _PageMap:
    """Logical page -> physical page of every sequence for one family of layers (all-history or windowed), with the
    host copy that the allocator edits and the device copy that the kernels read."""

    def __init__(self, batch: int, pages_per_seq: int, pool_pages: int, device):
        self.alloc = PageAllocator(pool_pages)
        self.host = torch.full((batch, pages_per_seq), -1, dtype=torch.int32)
        self.device = torch.full((batch, pages_per_seq), -1, dtype=torch.int32, device=device)
        self.dirty = False
        self.low = [0] * batch      # every logical page below low[row] is unmapped

    def ensure(self, row: int, first_page: int, last_page: int) -> None:
        t = self.host[row]
        for p in range(first_page, last_page + 1):
            if int(t[p]) < 0:
                t[p] = self.alloc.alloc()
                self.dirty = True

    def release_below(self, row: int, page_end: int) -> None:
        """Unmap logical pages [0, page_end) of `row`."""
        t = self.host[row]
        page_end = min(page_end, t.shape[0])
        for p in range(self.low[row], page_end):
            if int(t[p]) >= 0:
                self.alloc.release(int(t[p]))
                t[p] = -1
                self.dirty = True
        self.low[row] = max(self.low[row], page_end)

    def release_all(self, row: int) -> None:
        self.release_below(row, self.host.shape[1])
        self.low[row] = 0

    def push(self) -> None:
        """A blocking copy (once per page boundary, not per token): the host table is edited again before the device
        has run the steps that were queued behind an asynchronous copy, so the copy must have read it by then."""
        if self.dirty:
            self.device.copy_(self.host)
            self.dirty = False


class PagedKVCache:
    """K/V pools per layer in 16-token pages, handed out by a free-list allocator.

    Two page maps: layers that attend to the whole history ("L") keep every page of a sequence; windowed layers ("S")
    only keep the pages that still hold a key inside the window, so their pools are sized by the window, not by the
    sequence, and a page whose last key has left the window goes back to the free list. The kernels see only the
    indirection (`page_table[b, position // page_size]`; an unmapped entry is -1 and is never inside the range a
    query reads). `pool_pages` below the worst case over-subscribes the all-history pool: pages are mapped when a
    sequence reaches them and `MemoryError` is raised when none is left.

    The reference's cache is one contiguous [max_seq] buffer per layer and sequence (src/generate.cc:266-300)."""

    def __init__(self, cfg: Config, batch: int, max_seq: int, device, dtype, page_size: int = PAGE_SIZE,
                 pool_pages: Optional[int] = None, windowed: bool = True):
        self.cfg, self.batch, self.max_seq, self.page_size = cfg, batch, max_seq, page_size
        device = torch.device(device)
        self.pages_per_seq = (max_seq + page_size - 1) // page_size
        windows = [cfg.window_left(i) for i in range(cfg.num_layers)]
        short = [w for w in windows if w is not None and 0 <= w < max_seq]
        self.window = min(short) if (windowed and short) else -1
        self.is_windowed = [self.window >= 0 and w is not None and 0 <= w < max_seq for w in windows]
        n_full = batch * self.pages_per_seq if pool_pages is None else int(pool_pages)
        # a window of w keys back plus the query touches at most (w + page) // page + 1 pages. A chunk of a long
        # prompt needs the window before its first token and stores the window before its last: twice that.
        s_pages = min(self.pages_per_seq, 2 * ((max(self.window, 0) + page_size) // page_size + 1))
        n_win = batch * s_pages
        self.full = _PageMap(batch, self.pages_per_seq, n_full, device)
        self.win = _PageMap(batch, self.pages_per_seq, n_win, device) if any(self.is_windowed) else None
        self.k, self.v = [], []
        for i in range(cfg.num_layers):
            n = n_win if self.is_windowed[i] else n_full
            shape = (n, page_size, cfg.num_kv_heads, cfg.head_dim)
            self.k.append(torch.zeros(shape, dtype=dtype, device=device))
            self.v.append(torch.zeros(shape, dtype=dtype, device=device))
        self.seq_lens = torch.zeros(batch, dtype=torch.int32, device=device)
        self.lens_host = [0] * batch          # the host's copy of seq_lens (every step advances it without a sync)
        self.prev_emb = torch.zeros(batch, cfg.hidden_dim, dtype=dtype, device=device)
        self.has_prev = False

    # -- what the kernels read
    @property
    def page_table(self) -> torch.Tensor:
        return self.full.device

    def table(self, layer: int) -> torch.Tensor:
        return self.win.device if self.is_windowed[layer] else self.full.device

    def append_floor(self, new_len: int) -> int:
        """Windowed layers keep positions >= this (a page boundary) when `new_len` tokens are in the cache."""
        if self.window < 0:
            return 0
        return max(0, (new_len - 1 - self.window)) // self.page_size * self.page_size

    # -- allocation (host side, before the step's kernels are launched)
    def prepare(self, count: int, rows: Optional[Sequence[int]] = None) -> None:
        """Map the pages that the next `count` tokens of `rows` (default: all) will be written to, release the
        windowed pages that fall out of every later query's window, and publish the tables to the device."""
        ps = self.page_size
        for r in (range(self.batch) if rows is None else rows):
            n0 = self.lens_host[r]
            n1 = n0 + count
            if n1 > self.max_seq:
                raise ValueError("sequence does not fit the KV cache")
            if count == 1 and n0 % ps:
                continue          # decode inside a page: mapped when the page was entered, nothing to release yet
            if count > 0:
                self.full.ensure(r, n0 // ps, (n1 - 1) // ps)
            if self.win is not None and count > 0:
                # the first new query (position n0) still reads keys >= n0 - window; what lies below is released
                self.win.release_below(r, self.append_floor(n0 + 1) // ps)
                self.win.ensure(r, max(n0, self.append_floor(n1)) // ps, (n1 - 1) // ps)
        self.full.push()
        if self.win is not None:
            self.win.push()

    def advance_host(self, count: int, rows: Optional[Sequence[int]] = None) -> None:
        for r in (range(self.batch) if rows is None else rows):
            self.lens_host[r] += count

    def reset(self, rows: Optional[Sequence[int]] = None) -> None:
        """Forget `rows` (default: all): their pages return to the free lists."""
        for r in (range(self.batch) if rows is None else rows):
            self.full.release_all(r)
            if self.win is not None:
                self.win.release_all(r)
            self.lens_host[r] = 0
        if rows is None:
            self.seq_lens.zero_()
            self.has_prev = False
        else:
            self.seq_lens[torch.as_tensor(list(rows), device=self.seq_lens.device)] = 0
        self.full.push()
        if self.win is not None:
            self.win.push()

    def pages_in_use(self) -> dict:
        out = {"full": self.full.alloc.num_pages - self.full.alloc.available}
        if self.win is not None:
            out["windowed"] = self.win.alloc.num_pages - self.win.alloc.available
        return out

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.k + self.v)

    def rows(self, index: Sequence[int]) -> "_CacheRows":
        return _CacheRows(self, list(index))


class _CacheRows:
    """A subset of a cache's sequences with the attributes the forward pass reads: the pools are shared, the table
    rows / lengths / previous embeddings are copies that `commit` writes back. Lets sequences of different lengths be
    prefilled group by group."""

    def __init__(self, parent: PagedKVCache, index: List[int]):
        self.parent, self.index = parent, index
        dev = parent.seq_lens.device
        self._idx = torch.as_tensor(index, dtype=torch.long, device=dev)
        self.cfg, self.max_seq, self.page_size, self.batch = parent.cfg, parent.max_seq, parent.page_size, len(index)
        self.k, self.v = parent.k, parent.v
        self.is_windowed, self.window = parent.is_windowed, parent.window
        self.seq_lens = parent.seq_lens[self._idx].clone()
        self.lens_host = [parent.lens_host[r] for r in index]
        self.prev_emb = parent.prev_emb[self._idx].clone()
        self.has_prev = parent.has_prev
        self._tables = None

    def prepare(self, count: int, rows=None) -> None:
        self.parent.prepare(count, self.index)
        self._tables = (self.parent.full.device[self._idx].contiguous(),
                        None if self.parent.win is None else self.parent.win.device[self._idx].contiguous())

    @property
    def page_table(self):
        return self._tables[0]

    def table(self, layer: int):
        return self._tables[1] if self.is_windowed[layer] else self._tables[0]

    def append_floor(self, new_len: int) -> int:
        return self.parent.append_floor(new_len)

    def advance_host(self, count: int, rows=None) -> None:
        self.parent.advance_host(count, self.index)
        self.lens_host = [n + count for n in self.lens_host]

    def commit(self) -> None:
        self.parent.seq_lens[self._idx] = self.seq_lens
        self.parent.prev_emb[self._idx] = self.prev_emb


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
        if not (self.device.type == "cuda" and torch.cuda.is_current_stream_capturing()):
            cache.prepare(T)     # under graph capture / replay the caller has mapped the pages already
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
            t0 = cache.lens_host[0]
            if any(n != t0 for n in cache.lens_host):
                raise ValueError("prefill needs every sequence at the same position; use prefill_ragged")
            cos_all, sin_all = self._rope(t0 + T)
            cos, sin = cos_all[t0:t0 + T], sin_all[t0:t0 + T]
        new_lens = cache.seq_lens + T
        fused_prologue = kernel_decode and D == 128 and cache.page_table.shape[0] == B
        pos_flat = pos.reshape(-1).contiguous()
        # windowed layers keep only what a later query can still see: earlier positions of a long prompt are not stored
        pos_win = pos
        if not decode and cache.window >= 0:
            floor = cache.append_floor(t0 + T)
            if floor > t0:
                pos_win = torch.where(pos >= floor, pos, torch.full_like(pos, -1))
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
                table = cache.table(i)
                q3 = ops.cuda_module().decode_prep_append(qkv, v, cos_all, sin_all, pos_flat, cache.k[i], cache.v[i],
                                                          table, H)
                attn = ops.paged_decode_attention(q3, cache.k[i], cache.v[i], table, new_lens, wl).view(B, 1, H, D)
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
            table = cache.table(i)
            ops.kv_append(cache.k[i], cache.v[i], table, pos_win if cache.is_windowed[i] else pos, k, v4)
            if decode:
                attn = ops.paged_decode_attention(q[:, 0], cache.k[i], cache.v[i], table,
                                                  new_lens, wl).view(B, 1, H, D)
            elif t0 == 0:
                attn, _ = ops.attention_fwd(q, k, v4, wl)
            else:
                # a continued prompt: earlier keys come from the pages, this chunk's own keys are written over them
                # (on a windowed layer the chunk's early positions were not stored)
                kk = ops.paged_gather(cache.k[i], table, t0 + T).contiguous()
                vv = ops.paged_gather(cache.v[i], table, t0 + T).contiguous()
                kk[:, t0:], vv[:, t0:] = k, v4
                attn, _ = ops.attention_fwd(q, kk, vv, wl, q_offset=t0)
            x_mid = ops.linear_fwd(attn.reshape(M, H * D), m._w(i, "attn.c_proj"), residual=xr)
            h2, _ = ops.rmsnorm_fwd(x_mid)
            act = ops.linear_relu2_act_fwd(h2, m._w(i, "mlp.c_fc"))
            x = ops.linear_fwd(act, m._w(i, "mlp.c_proj"), residual=x_mid)
            if i == cfg.backout_layer:
                x_backout = x
        cache.seq_lens.add_(T)
        cache.advance_host(T)
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
        if max(cache.lens_host) + T > cache.max_seq:
            raise ValueError("prompt does not fit the KV cache")
        xn = self._forward(cache, tokens, decode=False)
        return self._logits(xn.view(B, T, -1)[:, -1])

    @torch.no_grad()
    def prefill_ragged(self, cache: PagedKVCache, prompts: Sequence[Sequence[int]]) -> torch.Tensor:
        """Prompts of different lengths, one per sequence of the cache. Sequences of equal length are prefilled
        together (one pass per distinct length). Returns the logits of every prompt's last position [B, vocab]."""
        if len(prompts) != cache.batch:
            raise ValueError("one prompt per sequence of the cache")
        groups = {}
        for r, p in enumerate(prompts):
            if len(p) == 0:
                raise ValueError("empty prompt")
            groups.setdefault(len(p), []).append(r)
        out = None
        for length, rows in sorted(groups.items()):
            view = cache.rows(rows)
            tok = torch.tensor([list(prompts[r]) for r in rows], dtype=torch.long, device=self.device)
            xn = self._forward(view, tok, decode=False)
            view.commit()
            lg = self._logits(xn.view(len(rows), length, -1)[:, -1])
            if out is None:
                out = torch.empty(cache.batch, lg.shape[1], dtype=lg.dtype, device=lg.device)
            out[torch.as_tensor(rows, device=lg.device)] = lg
        cache.has_prev = True
        return out

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
            lens_host = list(cache.lens_host)
            try:
                self._static_tok = tokens.clone()
                # warm up on a side stream (allocations, tensor-map cache), restoring the cache state afterwards
                lens, prev, had = cache.seq_lens.clone(), cache.prev_emb.clone(), cache.has_prev
                lens_host = list(cache.lens_host)
                cache.prepare(1)
                s = torch.cuda.Stream()
                s.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(s):
                    self.decode(cache, self._static_tok, greedy)
                torch.cuda.current_stream().wait_stream(s)
                cache.seq_lens.copy_(lens)
                cache.prev_emb.copy_(prev)
                cache.has_prev = had
                cache.lens_host[:] = lens_host
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self._static_out = self.decode(cache, self._static_tok, greedy)
                cache.seq_lens.copy_(lens)
                cache.prev_emb.copy_(prev)
                cache.has_prev = had
                cache.lens_host[:] = lens_host
                self._graph = g
            except Exception:
                cache.lens_host[:] = lens_host
                self._graph = None
                self._graph_cache = None
                self.use_cuda_graph = False
                torch.cuda.synchronize()
                return self.decode(cache, tokens, greedy)
        cache.prepare(1)            # page mapping is host work: before the replay, never inside the graph
        self._static_tok.copy_(tokens)
        self._graph.replay()
        cache.advance_host(1)
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
def generate_multi(engine: InferenceEngine, prompts, params: GenerateParams,
                   forced: Optional[callable] = None) -> List[GeneratedSequence]:
    """prompts: a tensor [N, L], or a list of token lists of any lengths (the reference's multi-prompt call takes
    prompts of different lengths too, src/generate.cc:458-576). Every prompt is decoded `num_samples` times: row r =
    prompt r // S. A row stops at `stop_id`, `bos_id`, any of `stop_ids`, or `max_tokens`.
    `forced(row, tokens_so_far)` may return a token to force at the next position (tool output injection)."""
    S = max(1, params.num_samples)
    dev = engine.device
    if isinstance(prompts, torch.Tensor):
        lists = None
        N, longest = prompts.shape
    else:
        lists = [list(p) for p in prompts]
        N, longest = len(lists), max(len(p) for p in lists)
        if all(len(p) == longest for p in lists):
            prompts, lists = torch.tensor(lists, dtype=torch.int64), None
    rows = N * S
    cache = engine.new_cache(rows, longest + params.max_tokens + 1)
    if lists is None:
        tok = prompts.to(dev).repeat_interleave(S, dim=0)
        logits = engine.prefill(cache, tok)
        out = [GeneratedSequence(tok[r].tolist(), [0] * longest) for r in range(rows)]
    else:
        per_row = [lists[r // S] for r in range(rows)]
        logits = engine.prefill_ragged(cache, per_row)
        out = [GeneratedSequence(list(p), [0] * len(p)) for p in per_row]
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
