"""Data parallelism with an owner-sharded optimizer.

Every parameter has one owner rank that holds its optimizer state and computes its update; the
result equals "one rank on the global batch" (the reference's contract, `src/train_parallel_test.cc`)
because gradients are summed over ranks after each rank scaled its backward by `1/(accum * world)`
(`src/train.h:117-122`).

* Muon matrices are owned whole (Newton-Schulz needs the full matrix), dealt round-robin inside each
  shape group so every rank gets the same mix of shapes.
* AdamW tensors (embeddings, LM head, scalars) are elementwise, so each is split into `world` equal
  contiguous slices.

Two transports implement the same step:
  `nccl`   - baseline: the owners' gradient shards are packed into a [world, shard] staging buffer,
             `reduce_scatter_tensor` (fp32) leaves every owner its reduced shard, the owner updates, the
             owned bf16 parameters are packed and `all_gather_into_tensor` distributes them (on CPU ranks,
             where gloo has no reduce-scatter, an all-reduce of the flat gradient and of a masked parameter
             buffer stands in).
  `fused`  - the sm_100a kernels of `parallel.fused` over NVLink peer memory (reduce-scatter fused with
             the owner's update, all-gather fused into the first consuming GEMM).
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..models.params import ParamSpec, ParamStore
from ..optim.optimizer import build_groups, OptimizerConfig


def assign_owners(store: ParamStore, world: int) -> Dict[str, int]:
    """Owner rank of every Muon matrix (AdamW tensors are sliced, not owned whole: owner -1)."""
    _, muon = build_groups(store, OptimizerConfig())
    owners: Dict[str, int] = {}
    k = 0
    for g in muon:
        for s in g.params:
            owners[s.name] = k % world
            k += 1
    for s in store.specs:
        owners.setdefault(s.name, -1)
    return owners


def adamw_slice(spec: ParamSpec, rank: int, world: int) -> Tuple[int, int]:
    """[begin, end) of `rank`'s slice inside the flattened parameter (multiples of 64 elements)."""
    n = spec.count
    per = ((n + world - 1) // world + 63) // 64 * 64
    a = min(n, rank * per)
    b = min(n, a + per)
    return a, b


class DataParallel:
    def __init__(self, rank: int, world_size: int, transport: str = "nccl", group=None, device=None):
        self.rank, self.world_size = rank, world_size
        self.transport = transport
        self.group = group
        self.fused = None
        if transport == "fused":
            from .fused import FusedTransport
            self.fused = FusedTransport(rank, world_size, device, group)
        elif transport != "nccl":
            raise ValueError(f"unknown data-parallel transport {transport!r}")
        self.model = None
        self.optimizer = None
        self.owners: Dict[str, int] = {}
        self._last_micro = True

    # ------------------------------------------------------------------------------------------
    def prepare(self, store: ParamStore) -> None:
        """Fix the ownership map; must run before the optimizer allocates its state."""
        self.owners = assign_owners(store, self.world_size)
        self.slices: Dict[str, Tuple[int, int]] = {}
        for s in store.specs:
            if self.owners[s.name] == -1:
                self.slices[s.name] = adamw_slice(s, self.rank, self.world_size)

    def owned(self, spec: ParamSpec) -> bool:
        """True for parameters this rank updates (its Muon matrices, and its slice of every AdamW tensor)."""
        return self.owners[spec.name] in (-1, self.rank)

    def allocator(self):
        """Allocator for the parameter store (symmetric memory for the fused transport, else None)."""
        return None if self.fused is None else self.fused.allocator

    def attach(self, model, optimizer) -> None:
        self.model, self.optimizer = model, optimizer
        store = model.params
        if self.world_size > 1:  # every rank must start from identical weights
            dist.broadcast(store.master, src=0, group=self.group)
            store.sync_compute()
        if self.fused is not None:
            from .fused import Pusher
            f = self.fused
            f.build_buckets(store, self.owners, self.slices)
            optimizer.pusher = Pusher(f)
            L = store.cfg.num_layers
            model.on_layer_grads_ready = lambda i: self._bucket_ready(i)
            model.on_head_grads_ready = lambda: self._bucket_ready(L)
            model.on_embed_grads_ready = lambda: self._bucket_ready(L + 1)
            self._step = 0
            torch.cuda.synchronize()
            if self.world_size > 1:
                dist.barrier(group=self.group)

    def _bucket_ready(self, b: int) -> None:
        if self._last_micro:
            self.fused.reduce_bucket(b, self._step)

    def begin_step(self, step: int = 0) -> None:
        if self.fused is None:
            return
        self._step = step
        f = self.fused
        if step > 1:
            # parameters updated by the previous step: embeddings and scalars are needed first (tiny wait kernel);
            # the matrices are waited for inside the first GEMM that reads a weight
            f.wait(f.slot_adamw, step - 1)
            from ..ops import cuda as K
            K.set_weight_wait(f.flag_view(f.slot_muon), step - 1)
        f.begin_reduction()

    def set_last_micro(self, last: bool) -> None:
        self._last_micro = last

    @torch.no_grad()
    def finish_step(self, step: int) -> None:
        store = self.model.params
        opt = self.optimizer
        if self.fused is not None:
            norm, clip = self.fused.global_grad_norm(opt.config.clip)
            opt.last_grad_norm = norm
            opt.step(step, clip_scale=clip)
            return
        use_rs = self.world_size > 1 and store.grad.is_cuda
        if use_rs:
            self._nccl_reduce_scatter()
        elif self.world_size > 1:
            dist.all_reduce(store.grad, op=dist.ReduceOp.SUM, group=self.group)
        from .. import ops
        if use_rs:
            # every rank holds the reduced gradient of what it owns only: the norm is the sum of the owners' parts
            total = self._nccl["g_shard"].square().sum(dtype=torch.float64).reshape(1)  # gaps in the shard are zero
            dist.all_reduce(total, op=dist.ReduceOp.SUM, group=self.group)
            norm = total.sqrt().float()[0]
            clip_v = opt.config.clip
            clip = torch.where(norm > clip_v, clip_v / norm.clamp_min(1e-30), torch.ones_like(norm)) \
                if clip_v and clip_v > 0 else torch.ones_like(norm)
        else:
            norm, clip = ops.grad_norm_and_clip([store.grad], opt.config.clip)
        opt.last_grad_norm = norm
        opt.step(step, clip_scale=clip)
        if use_rs:
            self._nccl_all_gather()
        elif self.world_size > 1:
            self._gather_params()

    # ---- NCCL baseline: reduce-scatter / all-gather over packed owner shards ---------------------------------
    def _nccl_layout(self):
        """Views for packing: per owner rank, the (flat offset, count, position) runs of `plan_reduce_scatter`."""
        if getattr(self, "_nccl", None) is not None:
            return self._nccl
        from .fused import plan_reduce_scatter
        store = self.model.params
        L = store.cfg.num_layers
        placed, cap = plan_reduce_scatter(store.specs, self.owners, self.world_size, L)
        dev = store.grad.device
        g_stage = torch.zeros(self.world_size, cap, dtype=torch.float32, device=dev)
        g_shard = torch.zeros(cap, dtype=torch.float32, device=dev)
        p_stage = torch.zeros(self.world_size, cap, dtype=store.value.dtype, device=dev)
        p_shard = torch.zeros(cap, dtype=store.value.dtype, device=dev)
        runs = [[run for b in range(L + 2) for run in placed[r][b]] for r in range(self.world_size)]
        pack_src = [store.grad[o:o + c] for r in range(self.world_size) for (o, c, _) in runs[r]]
        pack_dst = [g_stage[r, p:p + c] for r in range(self.world_size) for (o, c, p) in runs[r]]
        mine = runs[self.rank]
        own_grad = [store.grad[o:o + c] for (o, c, _) in mine]
        own_from_shard = [g_shard[p:p + c] for (o, c, p) in mine]
        own_val = [store.value[o:o + c] for (o, c, _) in mine]
        own_to_shard = [p_shard[p:p + c] for (o, c, p) in mine]
        all_val = [store.value[o:o + c] for r in range(self.world_size) for (o, c, _) in runs[r]]
        all_from_stage = [p_stage[r, p:p + c] for r in range(self.world_size) for (o, c, p) in runs[r]]
        self._nccl = dict(g_stage=g_stage, g_shard=g_shard, p_stage=p_stage, p_shard=p_shard, pack_src=pack_src,
                          pack_dst=pack_dst, own_grad=own_grad, own_from_shard=own_from_shard, own_val=own_val,
                          own_to_shard=own_to_shard, all_val=all_val, all_from_stage=all_from_stage)
        return self._nccl

    @torch.no_grad()
    def _nccl_reduce_scatter(self) -> None:
        n = self._nccl_layout()
        torch._foreach_copy_(n["pack_dst"], n["pack_src"])
        dist.reduce_scatter_tensor(n["g_shard"], n["g_stage"].view(-1), op=dist.ReduceOp.SUM, group=self.group)
        torch._foreach_copy_(n["own_grad"], n["own_from_shard"])

    @torch.no_grad()
    def _nccl_all_gather(self) -> None:
        n = self._nccl_layout()
        torch._foreach_copy_(n["own_to_shard"], n["own_val"])
        dist.all_gather_into_tensor(n["p_stage"].view(-1), n["p_shard"], group=self.group)
        torch._foreach_copy_(n["all_val"], n["all_from_stage"])

    @torch.no_grad()
    def _gather_params(self) -> None:
        """CPU ranks: every rank zeroes what it does not own in the compute copy; a sum all-reduce rebuilds it."""
        store = self.model.params
        val = store.value
        keep = torch.zeros_like(val)
        for s in store.specs:
            o = self.owners[s.name]
            if o == self.rank:
                keep[s.offset:s.offset + s.count] = val[s.offset:s.offset + s.count]
            elif o == -1:
                a, b = self.slices[s.name]
                keep[s.offset + a:s.offset + b] = val[s.offset + a:s.offset + b]
        dist.all_reduce(keep, op=dist.ReduceOp.SUM, group=self.group)
        val.copy_(keep)
