"""Fused data-parallel transport: bf16 reduce-scatter by peer stores + owner update that pushes parameters.

One step, per rank (see csrc/cuda/comm.cu for the kernels):

  backward ──► layer i done ──► grad_push(bucket i)        (push stream: every element another rank owns is
                                                            rounded to bf16 and stored into that owner's
                                                            receive slot over NVLink), then signal(slot i)
                              └► grad_reduce_local(i)      (comm stream: waits for slot i of ALL ranks, then
                                                            sums its own fp32 values and the N-1 received bf16
                                                            values in rank order, stores locally, adds to sumsq)
  (`NANOCHAT_DP_REDUCE=pull` selects the first design instead: signal, then the owner loads its fp32 segments
   from every peer's gradient buffer - twice the bytes, by loads.)
  all buckets reduced ──► all-reduce of one double (grad norm) ──► clip scale
  AdamW slices: update + push bf16 to every rank ──► signal(slot A)
  Muon matrices: Newton-Schulz, update + push bf16 to every rank ──► signal(slot M)
  next forward: embeddings wait for slot A (tiny kernel); the first QKV GEMM's TMA producer waits for slot M
  inside the GEMM kernel (no all-gather collective, no barrier).

The buffers that peers touch (flat fp32 gradient, flat bf16 parameters, flag words) live in symmetric
memory obtained from `torch.distributed._symmetric_memory` (plumbing only: allocation + address exchange).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist


class SymmetricBuffer:
    """A tensor that exists at the same size on every rank, with the peer addresses of all copies."""

    def __init__(self, numel: int, dtype: torch.dtype, device, group):
        import torch.distributed._symmetric_memory as symm
        self.tensor = symm.empty(numel, dtype=dtype, device=device)
        self.tensor.zero_()
        self.handle = symm.rendezvous(self.tensor, group)
        self.ptrs: List[int] = [int(p) for p in self.handle.buffer_ptrs]


def push_rows(placed, rank: int, world: int, bucket: int):
    """The push table of one rank for one bucket: rows (first_vec, src_off, dst_pos, dst_rank, count) over the elements
    other ranks own, and the number of 16-byte vectors in all. Destinations come in rotated order (rank + 1,
    rank + 2, ...): the kernel walks the table front to back, so with every rank starting at rank 0 all senders would
    store into the same receiver at the same time and share its one inbound link."""
    rows, first = [], 0
    for k in range(1, world):
        r = (rank + k) % world
        for off, cnt, pos in placed[r][bucket]:
            rows.append([first, off, pos, r, cnt])
            first += (cnt + 7) // 8
    return rows, first


def plan_reduce_scatter(specs, owners: Dict[str, int], world: int, L: int):
    """Layout of the bf16 reduce-scatter, a pure function of the parameter list (every rank computes the same).

    Returns `(placed, cap)`: `placed[rank][bucket]` lists `(offset, count, position)` for every contiguous run of
    elements that `rank` owns in `bucket` (offset in the flat gradient buffer, position in the owner's receive
    space, padded to 8 elements); `cap` is the largest receive space over the ranks. Buckets: b < L is layer b
    (its matrices and its value embedding), L is the LM head, L + 1 the token embedding and the scalars."""
    from .dp import adamw_slice

    def bucket_of(s) -> int:
        return L if s.kind == "lm_head" else s.layer if s.kind in ("matrix", "value_embed") else L + 1

    owned = [[[] for _ in range(L + 2)] for _ in range(world)]
    for s in specs:
        o = owners[s.name]
        for r in range(world):
            if o == r:
                owned[r][bucket_of(s)].append((s.offset, s.count))
            elif o == -1:
                a, e = adamw_slice(s, r, world)
                if e > a:
                    owned[r][bucket_of(s)].append((s.offset + a, e - a))
    placed = [[[] for _ in range(L + 2)] for _ in range(world)]
    cap = 0
    for r in range(world):
        pos = 0
        for b in range(L + 2):
            for off, cnt in sorted(owned[r][b]):
                placed[r][b].append((off, cnt, pos))
                pos += (cnt + 7) // 8 * 8
        cap = max(cap, pos)
    return placed, cap


class FusedTransport:
    def __init__(self, rank: int, world: int, device, group=None):
        self.rank, self.world = rank, world
        self.device = torch.device(device)
        self.group = group if group is not None else dist.group.WORLD
        self.buffers: List[SymmetricBuffer] = []
        self.grad: Optional[SymmetricBuffer] = None
        self.value: Optional[SymmetricBuffer] = None
        self.flags: Optional[SymmetricBuffer] = None
        self.comm_stream = torch.cuda.Stream(device=self.device)
        self.push_stream = torch.cuda.Stream(device=self.device)
        import os
        self.reduce_mode = os.environ.get("NANOCHAT_DP_REDUCE", "push")     # push (bf16, stores) | pull (fp32, loads)
        # how an owner's new parameters reach the other ranks: "peer" = one 16-byte store per rank through its peer
        # pointer; "multimem" = one multimem.st to the buffer's NVLink multicast address, replicated by the switch
        # (this GPU's outbound bytes drop from (world - 1) x to 1 x). Opt-in; falls back where the buffer has no
        # multicast mapping.
        self.push_mode = os.environ.get("NANOCHAT_DP_PUSH", "peer")
        self._push_targets = None
        self.recv: Optional[SymmetricBuffer] = None
        self.recv_stride = 0
        self.sumsq = torch.zeros(1, dtype=torch.float64, device=self.device)
        self.buckets: List[dict] = []
        self.num_slots = 0
        self.reduce_ctas = int(os.environ.get("NANOCHAT_DP_REDUCE_CTAS", 148 * 2))
        self.push_ctas = int(os.environ.get("NANOCHAT_DP_PUSH_CTAS", 148 * 2))
        self.adamw_ctas = int(os.environ.get("NANOCHAT_DP_ADAMW_CTAS", 148 * 2))

    # ------------------------------------------------------------------ allocation
    def allocator(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        buf = SymmetricBuffer(numel, dtype, self.device, self.group)
        self.buffers.append(buf)
        if dtype == torch.float32 and self.grad is None:
            self.grad = buf
        elif dtype == torch.bfloat16 and self.value is None:
            self.value = buf
        return buf.tensor

    # ------------------------------------------------------------------ buckets
    def build_buckets(self, store, owners: Dict[str, int], slices: Dict[str, Tuple[int, int]]) -> None:
        """Bucket b < L: everything whose gradient is final when layer b's backward is done (its matrices and
        its value embedding); bucket L: LM head; bucket L+1: token embedding and the scalars."""
        cfg = store.cfg
        L = cfg.num_layers
        per: List[List[Tuple[int, int]]] = [[] for _ in range(L + 2)]
        for s in store.specs:
            if s.kind == "lm_head":
                b = L
            elif s.kind in ("matrix", "value_embed"):
                b = s.layer
            else:
                b = L + 1
            o = owners[s.name]
            if o == self.rank:
                seg = (s.offset, (s.count + 3) // 4 * 4)
            elif o == -1:
                a, e = slices[s.name]
                if e <= a:
                    continue
                seg = (s.offset + a, (e - a + 3) // 4 * 4)
            else:
                continue
            per[b].append(seg)
        self.buckets = []
        for b, segs in enumerate(per):
            segs.sort()
            total = sum(c for _, c in segs)
            t = torch.tensor(segs if segs else [[0, 0]], dtype=torch.int64, device=self.device).reshape(-1, 2)
            self.buckets.append(dict(segs=t, total=total, n=len(segs)))
        if max(bk["n"] for bk in self.buckets) > 64:
            raise ValueError("a reduction bucket has more than 64 segments (the kernel's segment table)")
        if self.reduce_mode == "push":
            self._build_push_tables(store, owners, L)
        self._events = [torch.cuda.Event() for _ in self.buckets]
        self.slot_adamw = L + 2
        self.slot_muon = L + 3
        self.num_slots = L + 4
        self.flags = SymmetricBuffer(self.num_slots * self.world, torch.int32, self.device, self.group)

    def _build_push_tables(self, store, owners: Dict[str, int], L: int) -> None:
        """Tables of the bf16 reduce-scatter. Every rank computes the ownership of ALL ranks (it is a pure function
        of the parameter list), lays each owner's elements out bucket by bucket in a receive space (positions
        padded to 8 elements = one 16-byte bf16 store) and derives: for every bucket, what it must push where, and
        where its own elements sit. The receive buffer holds one such space per source rank."""
        placed, cap = plan_reduce_scatter(store.specs, owners, self.world, L)
        self.recv_stride = cap
        self.recv = SymmetricBuffer(max(cap, 8) * self.world, torch.bfloat16, self.device, self.group)
        for b, bk in enumerate(self.buckets):
            rows, first = push_rows(placed, self.rank, self.world, b)
            if len(rows) > 128:
                raise ValueError("a bucket pushes more than 128 segments (the kernel's segment table)")
            bk["push_rows"] = torch.tensor(rows if rows else [[0, 0, 0, 0, 0]], dtype=torch.int64,
                                           device=self.device).reshape(-1, 5)
            bk["push_n"], bk["push_vec"] = len(rows), first
            rows, first = [], 0
            for off, cnt, pos in placed[self.rank][b]:
                rows.append([first, off, pos, cnt])
                first += (cnt + 7) // 8
            if len(rows) > 64:
                raise ValueError("a rank owns more than 64 runs in one bucket (the reduction kernel's segment table)")
            bk["own_rows"] = torch.tensor(rows if rows else [[0, 0, 0, 0]], dtype=torch.int64,
                                          device=self.device).reshape(-1, 4)
            bk["own_n"], bk["own_vec"] = len(rows), first
        self._events2 = [torch.cuda.Event() for _ in self.buckets]

    # ------------------------------------------------------------------ step pieces
    def signal(self, slot: int, value: int) -> None:
        from ..ops import cuda as K
        K._C.comm_signal(self.flags.ptrs, self.rank, slot, value)

    def reduce_bucket(self, b: int, step: int, scale: float = 1.0) -> None:
        """Publish "bucket b is final on this rank" on the current stream and enqueue this rank's share of the
        reduction on the communication stream."""
        from ..ops import cuda as K
        bk = self.buckets[b]
        status = K._C.status_tensor(self.device.index)
        if self.reduce_mode == "push":
            # The push never waits for anybody, so it may run as soon as this rank's bucket is final; the local
            # reduction is ordered after this rank's own push + signal (second event), for the reason given below.
            ev = self._events[b]
            ev.record(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.push_stream):
                self.push_stream.wait_event(ev)
                if bk["push_n"]:
                    K._C.comm_grad_push(self.grad.tensor, self.recv.ptrs, self.recv_stride, self.rank, bk["push_rows"],
                                        bk["push_vec"], scale, self.push_ctas)
                self.signal(b, step)
                self._events2[b].record(self.push_stream)
            if bk["own_n"] == 0:
                return
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(self._events2[b])
                K._C.comm_grad_reduce_local(self.grad.tensor, self.recv.tensor, self.recv_stride, self.world, self.rank,
                                            bk["own_rows"], bk["own_vec"], scale, self.flags.tensor, b, step,
                                            self.sumsq, status, self.reduce_ctas)
            return
        self.signal(b, step)
        if bk["total"] == 0:
            return
        # The reduction must not become resident before this rank's own backward has reached the bucket: its
        # CTAs spin on the peers' flags, and a spinning grid that starts early can keep the backward kernels of
        # BOTH ranks off the SMs (each waits for a signal that sits behind the other's blocked backward).
        # Ordered after the local signal, a waiting reduction only ever waits for a peer that is behind and
        # whose own reductions can all complete, so some rank always makes progress.
        ev = self._events[b]
        ev.record(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.comm_stream):
            self.comm_stream.wait_event(ev)
            K._C.comm_reduce_pull(self.grad.ptrs, self.rank, bk["segs"], bk["total"], scale, self.flags.tensor, b,
                                  step, self.sumsq, status, self.reduce_ctas)

    def begin_reduction(self) -> None:
        with torch.cuda.stream(self.comm_stream):
            self.sumsq.zero_()
        # the reduction kernels must not start before this step's zero_() of sumsq, nor before earlier work on
        # the compute stream that they are ordered after by flags only
        self.comm_stream.wait_stream(torch.cuda.current_stream(self.device))
        self.push_stream.wait_stream(torch.cuda.current_stream(self.device))

    def global_grad_norm(self, clip: float):
        """Joins the communication stream, all-reduces the squared norm and returns (norm, clip_scale)."""
        torch.cuda.current_stream(self.device).wait_stream(self.comm_stream)
        torch.cuda.current_stream(self.device).wait_stream(self.push_stream)
        total = self.sumsq.clone()
        if self.world > 1:
            dist.all_reduce(total, op=dist.ReduceOp.SUM, group=self.group)
        norm = total.sqrt().float()[0]
        if clip and clip > 0:
            scale = torch.where(norm > clip, clip / norm.clamp_min(1e-30), torch.ones_like(norm))
        else:
            scale = torch.ones_like(norm)
        return norm, scale

    def wait(self, slot: int, value: int) -> None:
        from ..ops import cuda as K
        K._C.comm_wait(self.flags.tensor, self.world, slot, value, K._C.status_tensor(self.device.index))

    def flag_view(self, slot: int) -> torch.Tensor:
        return self.flags.tensor[slot * self.world:(slot + 1) * self.world]

    # ------------------------------------------------------------------ pushing updates
    def push_targets(self):
        """(peer pointers of the parameter buffer, its multicast address or 0)."""
        if self._push_targets is None:
            self._push_targets = (self.value.ptrs, 0)
            if self.push_mode == "multimem":
                h = self.value.handle
                mc = int(getattr(h, "multicast_ptr", 0) or 0)
                if mc != 0:
                    self._push_targets = (self.value.ptrs, mc + int(getattr(h, "offset", 0) or 0))
                elif self.rank == 0:
                    print("[dp] NANOCHAT_DP_PUSH=multimem: the parameter buffer has no multicast mapping; "
                          "using peer stores", flush=True)
        return self._push_targets

    def adamw_push(self, master, offset: int, grad, m, v, *, lr, beta1, beta2, eps, weight_decay, step, grad_scale):
        from ..ops import cuda as K
        gs = grad_scale.reshape(1) if isinstance(grad_scale, torch.Tensor) else None
        ptrs, mc = self.push_targets()
        # two CTAs per SM: the slices run on a side stream beside the Newton-Schulz products, whose CTAs (one per SM,
        # most of its shared memory) must still find room to become resident
        K._C.comm_adamw_push(master, ptrs, offset, grad, m, v, lr, beta1, beta2, eps, weight_decay, step, gs, mc,
                             self.adamw_ctas)

    def muon_apply_push(self, master, offset: int, xb, scale0, line_scale, lines_are_rows: bool, lr: float, wd: float):
        from ..ops import cuda as K
        ptrs, mc = self.push_targets()
        K._C.comm_muon_apply_push(master, ptrs, offset, xb, scale0, line_scale, lines_are_rows, lr, wd, mc)

    def push_span(self, offset: int, count: int) -> None:
        """Copy a (small) span of this rank's parameter buffer to every peer with ordinary peer copies."""
        local = self.value.tensor[offset:offset + count]
        for r in range(self.world):
            if r == self.rank:
                continue
            peer = self.value.handle.get_buffer(r, (self.value.tensor.numel(),), self.value.tensor.dtype)
            peer[offset:offset + count].copy_(local)


class Pusher:
    """Adapter handed to the Optimizer: owner updates write straight into every rank's parameters."""

    def __init__(self, transport: FusedTransport):
        self.t = transport

    def adamw_push(self, master, offset, grad, m, v, **kw):
        self.t.adamw_push(master, offset, grad, m, v, **kw)

    def after_adamw(self, step: int) -> None:
        self.t.signal(self.t.slot_adamw, step)

    def make_muon_apply(self, specs):
        t = self.t

        def apply(p, master, xb, scale0, line_scale, lines_are_rows, lr, wd):
            t.muon_apply_push(master, specs[p].offset, xb, scale0, line_scale, lines_are_rows, lr, wd)

        def batched(scratch, masters, X, scale, line_scale, lines_are_rows, lr, wd):
            from ..ops import cuda as K
            offs = scratch.table("voff", None, values=tuple(s.offset for s in specs))
            ptrs, mc = t.push_targets()
            K._C.comm_muon_apply_push_batched(scratch.table("m", masters), offs, ptrs, X, scale, line_scale,
                                              lines_are_rows, lr, wd, mc)
        if all(s.offset % 8 == 0 for s in specs):
            apply.batched = batched
        return apply

    def side_stream(self):
        """Stream on which the optimizer may run the AdamW slices while Newton-Schulz runs on the compute stream."""
        return self.t.comm_stream

    def push_span(self, offset: int, count: int) -> None:
        self.t.push_span(offset, count)

    def after_muon(self, step: int) -> None:
        self.t.signal(self.t.slot_muon, step)
