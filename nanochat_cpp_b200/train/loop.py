"""Training step and loop.

The step is the reference's (`src/train.cc:792-945`): zero the gradients, run `grad_accum`
forward/backward micro-batches scaled by `1/(grad_accum * world)`, synchronise gradients across ranks,
take one optimizer step, and log `step | loss | lr | grad_norm | tok/s | mfu | ...` on logging steps.
Nothing in the step reads the device: the loss stays on the device and is fetched only when a caller
asks for it, so non-logging steps are fully asynchronous.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Iterable, List, Optional, Sequence, Tuple

import torch

from ..config import Config
from ..models import GPT
from ..optim import Optimizer, OptimizerConfig, SchedulerConfig
from . import mfu as perf


@dataclass
class TrainConfig:
    batch: int = 8
    grad_accum: int = 1
    num_iterations: int = 100
    log_every: int = 10
    eval_every: int = 0
    save_every: int = 0
    eval_steps: int = 10
    seed: int = 42
    checkpoint: str = ""
    resume: str = ""
    log: str = ""
    dtype: str = "bf16"
    head_chunk_rows: int = 11264
    fp8: object = False          # False, True / "mx", or "block" (see models.GPT)
    # "auto": replay a micro-batch's forward + backward from a CUDA graph when the step is bound by launch rate
    # (several small micro-batches); "on" / "off" force it. Never the headline path of a large single micro-batch.
    cuda_graph: str = "auto"
    optim: OptimizerConfig = field(default_factory=OptimizerConfig)
    sched: SchedulerConfig = field(default_factory=SchedulerConfig)


class Trainer:
    """One rank of a (possibly data-parallel) training job."""

    def __init__(self, cfg: Config, tc: TrainConfig, device="cuda", dp=None, model: Optional[GPT] = None):
        self.cfg, self.tc = cfg, tc
        self.device = torch.device(device)
        dtype = torch.bfloat16 if tc.dtype == "bf16" else torch.float32
        self.model = model or GPT(cfg, self.device, dtype, seed=tc.seed, head_chunk_rows=tc.head_chunk_rows,
                                  allocator=None if dp is None else dp.allocator(), fp8=tc.fp8)
        if tc.sched.num_iterations == 0:
            tc.sched.num_iterations = tc.num_iterations
        self.dp = dp
        self.world = 1 if dp is None else dp.world_size
        if dp is not None:
            dp.prepare(self.model.params)
        self.optimizer = Optimizer(self.model.params, tc.optim, tc.sched,
                                   owned=None if dp is None else dp.owned,
                                   adamw_slices=None if dp is None else dp.slices)
        if dp is not None:
            dp.attach(self.model, self.optimizer)
        self.step_count = 0
        self._graphs = {}
        self.graph_replays = 0
        self.last_loss: Optional[torch.Tensor] = None
        self.time_phases = False      # set for one step by the loop on logging steps
        self._phase_events = None

    @torch.no_grad()
    def train_step(self, micro_batches: Sequence[Tuple[torch.Tensor, torch.Tensor]]) -> torch.Tensor:
        """`micro_batches`: `grad_accum` pairs of (tokens [B,T], targets [B,T]) already on the device.
        Returns the mean micro-batch loss as a 0-d device tensor."""
        m = self.model
        accum = len(micro_batches)
        scale = 1.0 / (accum * self.world)
        timed = self.time_phases and self.device.type == "cuda"
        ev = None
        if timed:  # phase timers of a logging step: events only, nothing is synchronised here
            ev = {k: torch.cuda.Event(enable_timing=True) for k in ("start", "bwd_end", "end")}
            ev["fwd_end"] = [torch.cuda.Event(enable_timing=True) for _ in range(accum)]
            ev["micro"] = [torch.cuda.Event(enable_timing=True) for _ in range(accum)]
            ev["start"].record()
        if self.dp is not None:
            self.dp.begin_step(self.step_count + 1)
        m.zero_grad()
        total = None
        for k, (tokens, targets) in enumerate(micro_batches):
            if self.dp is not None:
                self.dp.set_last_micro(k == accum - 1)
            if timed:
                ev["micro"][k].record()
                m.phase_event = ev["fwd_end"][k]
            loss = None
            if self._graphable(k, accum, timed, tokens):
                loss = self._micro_graphed(tokens, targets, scale)
            if loss is None:
                loss = m.forward_backward(tokens, targets, grad_scale=scale)
            total = loss if total is None else total + loss
        m.phase_event = None
        if timed:
            ev["bwd_end"].record()
        self.step_count += 1
        if self.dp is not None:
            self.dp.finish_step(self.step_count)
        else:
            self.optimizer.step(self.step_count)
        if timed:
            ev["end"].record()
            self._phase_events = ev
        if m.fp8:
            self.wait_for_weights()
            m.refresh_fp8()
        self.last_loss = total / accum
        return self.last_loss

    # ------------------------------------------------------------------ CUDA-graph micro-batches
    def _graphable(self, k: int, accum: int, timed: bool, tokens: torch.Tensor) -> bool:
        """A micro-batch can be replayed from a graph when nothing in it changes from step to step: no phase timers,
        no fp8 re-quantisation, and under data parallelism not the last micro-batch (its backward launches the
        bucket reductions, whose flag values count steps)."""
        mode = self.tc.cuda_graph
        if mode == "off" or self.device.type != "cuda" or timed or self.model.fp8:
            return False
        if self.dp is not None and k == accum - 1:
            return False
        if mode == "auto":
            # launch-bound shapes only: a few thousand kernels of a few microseconds each per micro-batch
            return accum >= 2 and tokens.numel() * self.cfg.hidden_dim <= (1 << 24)
        return True

    def _micro_graphed(self, tokens: torch.Tensor, targets: torch.Tensor, scale: float):
        """Forward + backward of one micro-batch replayed from a CUDA graph (captured on the second step, after an
        eager step has warmed every cache). Gradients accumulate into the flat buffer exactly as in the eager call.
        Returns None when this call has to run eagerly."""
        from ..ops import cuda as K
        if self.step_count < 1:
            return None
        f = getattr(self.dp, "fused", None) if self.dp is not None else None
        if f is not None and self.step_count > 0:
            # the wait for the pushed matrices normally rides in the first GEMM; a replayed graph cannot carry this
            # step's flag value, so it is enqueued as its own (bounded) wait kernel
            f.wait(f.slot_muon, self.step_count)
            K.clear_weight_wait()
        key = (tuple(tokens.shape), tokens.dtype, targets.dtype, float(scale))
        entry = self._graphs.get(key)
        if entry is None:
            if len(self._graphs) >= 2:
                return None
            tok_s, tgt_s = tokens.clone(), targets.clone()
            torch.cuda.synchronize(self.device)
            g = torch.cuda.CUDAGraph()
            n0 = K.launch_count()
            try:
                with torch.cuda.graph(g, capture_error_mode="thread_local"):
                    loss_s = self.model.forward_backward(tok_s, tgt_s, grad_scale=scale)
            except Exception as e:   # capture is an optimisation: fall back to eager launches for good
                self.tc.cuda_graph = "off"
                self._graphs.clear()
                torch.cuda.synchronize(self.device)
                if self._rank0():
                    print(f"[train] CUDA-graph capture of the micro-batch failed ({type(e).__name__}: {e}); "
                          "continuing with eager launches", flush=True)
                return None
            entry = (g, tok_s, tgt_s, loss_s, K.launch_count() - n0)
            K.add_launches(-entry[4])       # capture enqueued nothing; replays are counted below
            self._graphs[key] = entry
        g, tok_s, tgt_s, loss_s, kernels = entry
        tok_s.copy_(tokens)
        tgt_s.copy_(targets)
        g.replay()
        K.add_launches(kernels)
        self.graph_replays += 1
        return loss_s.clone()

    def wait_for_weights(self) -> None:
        """Under the fused transport the owners push the new bf16 weights into every rank's buffer asynchronously
        and the next training forward waits for them inside its first GEMM. Anything else that reads the weights
        right after a step (evaluation, generation, the fp8 re-quantisation, a checkpoint) calls this first: it
        enqueues, on the compute stream, the bounded waits for this step's pushes."""
        f = getattr(self.dp, "fused", None) if self.dp is not None else None
        if f is not None and self.step_count > 0:
            f.wait(f.slot_adamw, self.step_count)
            f.wait(f.slot_muon, self.step_count)

    def phase_times(self) -> dict:
        """fwd / bwd / opt milliseconds of the last step run with `time_phases` (after a device synchronise). `opt`
        is the optimizer step including, under data parallelism, whatever gradient synchronisation is still
        outstanding after the last backward kernel (`sync` is reported inside it: the fused transport has no
        separate phase)."""
        ev = self._phase_events
        if ev is None:
            return {"fwd_ms": 0.0, "bwd_ms": 0.0, "sync_ms": 0.0, "opt_ms": 0.0}
        accum = len(ev["micro"])
        fwd = sum(ev["micro"][k].elapsed_time(ev["fwd_end"][k]) for k in range(accum))
        whole = ev["start"].elapsed_time(ev["bwd_end"])
        return {"fwd_ms": fwd, "bwd_ms": max(0.0, whole - fwd), "sync_ms": 0.0,
                "opt_ms": ev["bwd_end"].elapsed_time(ev["end"])}

    def tokens_per_step(self) -> int:
        return self.tc.batch * self.cfg.seq_len * self.tc.grad_accum * self.world

    # ------------------------------------------------------------------ the loop
    def _rank0(self) -> bool:
        return self.dp is None or self.dp.rank == 0

    def _stage(self, loader):
        """`grad_accum` micro-batches from the loader through pinned host buffers to the device.

        The copies are asynchronous and the host may run several steps ahead of the GPU, so the pinned buffers
        rotate over two sets and each set carries an event recorded after its copies: a set is refilled only once
        that event has fired, i.e. once the device has read the previous contents."""
        B, T = self.tc.batch, self.cfg.seq_len
        cuda = self.device.type == "cuda"
        if not hasattr(self, "_pinned"):
            self._pinned = [dict(bufs=[(torch.empty((B, T), dtype=torch.int32, pin_memory=cuda),
                                        torch.empty((B, T), dtype=torch.int32, pin_memory=cuda))
                                       for _ in range(self.tc.grad_accum)], event=None)
                            for _ in range(2 if cuda else 1)]
            self._pinned_next = 0
        cur = self._pinned[self._pinned_next]
        self._pinned_next = (self._pinned_next + 1) % len(self._pinned)
        if cur["event"] is not None:
            cur["event"].synchronize()
        out = []
        for tok_h, tgt_h in cur["bufs"]:
            loader.next_into(tok_h.numpy(), tgt_h.numpy())
            out.append((tok_h.to(self.device, non_blocking=True).long(),
                        tgt_h.to(self.device, non_blocking=True).long()))
        if cuda:
            cur["event"] = torch.cuda.Event()
            cur["event"].record()
        return out

    def check_device_status(self) -> None:
        """Reads the per-device status word that every bounded wait reports through (a kernel that gave up waiting
        returns early and leaves wrong output behind). Under data parallelism the codes are max-reduced so that every
        rank raises on the same step; the caller must have synchronised the device. Raising here, before the next
        checkpoint is written, lets the launcher restart the group from the last good file."""
        if self.device.type != "cuda":
            return
        from .. import ops
        if ops.get_mode() != "kernels":
            return
        K = ops.cuda_module()
        code = int(K._C.read_status(self.device.index if self.device.index is not None else torch.cuda.current_device()))
        if self.dp is not None and self.world > 1:
            import torch.distributed as dist
            t = torch.tensor([code], dtype=torch.int32, device=self.device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            code = int(t.item())
        if code != 0:
            K._C.reset_status(self.device.index if self.device.index is not None else torch.cuda.current_device())
            raise RuntimeError(f"step {self.step_count}: a kernel gave up waiting on some rank (status code {code}); "
                               "the step's results are not trustworthy, restart from the last checkpoint")

    def _heartbeat(self):
        """A `parallel.health.Heartbeat` over the process group's store (data-parallel runs only)."""
        if self.dp is None or self.world <= 1:
            return None
        try:
            import torch.distributed as dist
            from torch.distributed.distributed_c10d import _get_default_store
            from ..parallel.health import Heartbeat
            if not dist.is_initialized():
                return None
            return Heartbeat(_get_default_store(), self.dp.rank, self.world, timeout_s=600.0, prefix="train_hb")
        except Exception:
            return None

    def resume(self, path: str, loader=None) -> int:
        """Restores weights, optimizer state and step (and the loader position from `<path>.cursor`)."""
        import os
        from .checkpointer import load_checkpoint
        _, meta = load_checkpoint(path, self.model, self.optimizer)
        self.step_count = int(meta.get("step", 0))
        self.optimizer.step_count = self.step_count
        if loader is not None and os.path.exists(path + ".cursor"):
            loader.load_cursor(path + ".cursor")
        return self.step_count      # every rank reads the same canonical file, so no broadcast is needed

    def save(self, path: str, loader=None, stage: str = "base") -> None:
        from .checkpointer import save_checkpoint
        save_checkpoint(path, self.model, self.optimizer, step=self.step_count, stage=stage, dp=self.dp,
                        loader=loader if self._rank0() else None)

    def run(self, train_loader, val_loader=None, token_bytes=None, metrics_dir: str = "", out=None) -> dict:
        """The training loop of the reference (`src/train.cc:726-945`): steps `step_count+1 .. num_iterations`, a log
        line every `log_every` steps (and on the last), validation bits per byte every `eval_every`, a checkpoint
        every `save_every` and at the end. Returns the summary that is also written to `summary.json`."""
        import json
        import os
        import sys
        from ..eval import eval_bpb
        tc = self.tc
        out = out or sys.stdout
        log_f = open(tc.log, "a") if tc.log and self._rank0() else None
        met_f = None
        if metrics_dir and self._rank0():
            os.makedirs(metrics_dir, exist_ok=True)
            met_f = open(os.path.join(metrics_dir, "metrics.jsonl"), "a")

        def emit(line: str) -> None:
            if self._rank0():
                print(line, file=out, flush=True)
                if log_f:
                    log_f.write(line + "\n")
                    log_f.flush()

        peaks = perf.measured_peaks()
        fpt = perf.flops_per_token(self.cfg)
        muon_flops = perf.muon_flops_per_step(self.cfg, tc.optim.muon_ns_steps)
        tokens_step = self.tokens_per_step()
        cuda = self.device.type == "cuda"
        t_log = time.perf_counter()
        steps_since = 0
        data_ms = 0.0
        last = {}
        losses = []
        first = self.step_count + 1
        hb = self._heartbeat()
        for step in range(first, tc.num_iterations + 1):
            t0 = time.perf_counter()
            micro = self._stage(train_loader)
            data_ms += (time.perf_counter() - t0) * 1e3
            final = step == tc.num_iterations
            self.time_phases = (tc.log_every > 0 and step % tc.log_every == 0) or final
            if hb is not None:
                hb.check(step)      # a peer that left or went silent is found before this rank launches the step
            loss = self.train_step(micro)
            if hb is not None:
                hb.beat(step)
            steps_since += 1
            eval_ms = 0.0
            bpb = None
            if val_loader is not None and tc.eval_every > 0 and (step % tc.eval_every == 0 or final):
                te = time.perf_counter()
                self.wait_for_weights()
                bpb = eval_bpb(self.model, val_loader, tc.eval_steps, token_bytes)
                eval_ms = (time.perf_counter() - te) * 1e3
                emit(f"[nanochat] step {step} val_bpb {bpb:.6f}")
            if (tc.log_every > 0 and step % tc.log_every == 0) or final:
                if cuda:
                    torch.cuda.synchronize(self.device)
                    self.check_device_status()
                now = time.perf_counter()
                step_ms = ((now - t_log) * 1e3 - eval_ms) / max(steps_since, 1)
                tok_s = tokens_step / (step_ms / 1e3)
                lv = float(loss)
                gn = self.optimizer.grad_norm()
                lr = self.optimizer.scheduler.lr_multiplier(step)
                mfu_v = perf.mfu(tok_s / self.world, self.cfg, peaks["bf16_tflops_sustained"])
                phases = self.phase_times() if cuda else {"fwd_ms": 0.0, "bwd_ms": 0.0, "sync_ms": 0.0, "opt_ms": 0.0}
                last = dict(step=step, loss=lv, lr=lr, grad_norm=gn, tok_s=tok_s, mfu=mfu_v,
                            model_tflops=tok_s * fpt / 1e12, optim_tflops=muon_flops / (step_ms / 1e3) / 1e12,
                            step_ms=step_ms, data_ms=data_ms / max(steps_since, 1), eval_ms=eval_ms, **phases)
                if bpb is not None:
                    last["val_bpb"] = bpb
                losses.append(lv)
                emit(format_log_line(step, lv, lr, gn, tok_s, mfu_v, last["model_tflops"], last["optim_tflops"],
                                     step_ms, last["data_ms"], fwd_ms=phases["fwd_ms"], bwd_ms=phases["bwd_ms"],
                                     sync_ms=phases["sync_ms"], opt_ms=phases["opt_ms"], eval_ms=eval_ms))
                if met_f:
                    met_f.write(json.dumps(last) + "\n")
                    met_f.flush()
                t_log, steps_since, data_ms = time.perf_counter(), 0, 0.0
            if tc.checkpoint and ((tc.save_every > 0 and step % tc.save_every == 0) or final):
                if cuda:
                    torch.cuda.synchronize(self.device)
                    self.check_device_status()      # never overwrite a good checkpoint with a failed step's weights
                self.save(tc.checkpoint, train_loader)
                emit(f"[nanochat] saved {tc.checkpoint} at step {step}")
        summary = dict(final_step=self.step_count, final_loss=losses[-1] if losses else None, world_size=self.world,
                       tokens_per_step=tokens_step, last=last)
        if metrics_dir and self._rank0():
            with open(os.path.join(metrics_dir, "summary.json"), "w") as f:
                json.dump(summary, f, indent=1)
        for f in (log_f, met_f):
            if f:
                f.close()
        return summary


def format_log_line(step: int, loss: float, lr: float, grad_norm: float, tok_s: float, mfu_v: float,
                    model_tflops: float, optim_tflops: float, step_ms: float, data_ms: float = 0.0,
                    fwd_ms: float = 0.0, bwd_ms: float = 0.0, sync_ms: float = 0.0, opt_ms: float = 0.0,
                    eval_ms: float = 0.0) -> str:
    """One text line per logged step, fields in the reference's order (`src/train.cc:74-101`)."""
    return (f"step {step:6d} | loss {loss:.6f} | lr {lr:.6g} | grad_norm {grad_norm:.4f} | tok/s {tok_s:.0f} | "
            f"mfu {mfu_v:.4f} | model_tflops {model_tflops:.1f} | optim_tflops {optim_tflops:.2f} | "
            f"step_ms {step_ms:.2f} | data_ms {data_ms:.2f} | fwd_ms {fwd_ms:.2f} | bwd_ms {bwd_ms:.2f} | "
            f"sync_ms {sync_ms:.2f} | opt_ms {opt_ms:.2f} | eval_ms {eval_ms:.2f}")
