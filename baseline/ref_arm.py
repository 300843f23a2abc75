"""Reference arm of the benchmark: runs the hand-built, unmodified reference (`baseline/_ref/`, made by
`baseline/ref_build/build_ref.py`) on the benchmark's metric and configuration and returns the JSON line.

One process per rank, as the reference's own launcher does it: `CUDA_VISIBLE_DEVICES` selects the rank's GPU
and `NANOCHAT_RANK / NANOCHAT_WORLD_SIZE / NANOCHAT_MASTER_ADDR / NANOCHAT_MASTER_PORT` form its group
(reference src/train_command.cc:71-74), so its own gradient ring (host-staged, TCP on 127.0.0.1) carries the
gradients. Nothing of this repository's package is imported on this path.

Timing comes from the reference itself: with `--log-every 1` its loop drains the device at every phase boundary
and prints `step_ms` (data + forward + backward + sync + optimizer, reference src/train.cc:726-945); the
device-timed value is the sum of `step_ms` over the K timed steps, and the end-to-end value is the wall-clock
time between the arrival of the log line of step W and that of step W+K (every reference step copies its token
and target ids host->device and, when it logs, reads the loss back). Both are the maximum over ranks.
"""
from __future__ import annotations

import json
import os
import re
import subprocess
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)

PRESETS = {
    # name: layers, hidden, heads, kv_heads, vocab, seq
    "d20": (20, 1280, 10, 10, 65536, 2048),
    "d12": (12, 768, 6, 6, 32768, 2048),
    "d26": (26, 1664, 13, 13, 65536, 2048),
    "tiny": (4, 256, 4, 4, 4096, 256),
}

STEP_RE = re.compile(r"^step (\d+) \| loss ([-\d.naninf]+) \|.*?tok/s ([\d.]+) \|.*?step_ms ([\d.]+) \| data_ms ([\d.]+) \| "
                     r"fwd_ms ([\d.]+) \| bwd_ms ([\d.]+) \| sync_ms ([\d.]+) \| opt_ms ([\d.]+)")


def ref_dir() -> str:
    return os.environ.get("NANOCHAT_REF_DIR", os.path.join(HERE, "_ref"))


def ensure_built() -> str | None:
    """Returns None when `ref_train` is ready, else the reason it is not."""
    d = ref_dir()
    exe = os.path.join(d, "ref_train")
    if os.path.exists(exe) and os.path.exists(os.path.join(d, "libnanochat_ref.so")):
        return None
    src = os.environ.get("NANOCHAT_REF_SRC", "/root/reference")
    if not os.path.isdir(src):
        return f"baseline/_ref is not built and the reference sources are not at {src}"
    p = subprocess.run([sys.executable, os.path.join(HERE, "ref_build", "build_ref.py"), "--ref", src],
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0 or not os.path.exists(exe):
        return "hand build of the reference failed: " + p.stdout.strip().splitlines()[-1][:200]
    return None


def _free_port_base() -> int:
    base = int(os.environ.get("MASTER_PORT", "29500"))
    port = base + 1733
    return port if port < 65000 else base - 1733


def run_train(args, sampler_cls):
    """Runs this rank's reference process; returns (record, error)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    d = ref_dir()
    exe = os.path.join(d, "ref_train")
    layers, hidden, heads, kv, vocab, seq = PRESETS[args.preset]
    micro = args.micro_batch or args.batch
    accum = max(1, args.batch // micro)

    tok = f"/tmp/ref_tok_{vocab}_{os.getpid()}.bin"
    p = subprocess.run([exe, "make-tokenizer", "--out", tok, "--vocab", str(vocab)], cwd=d,
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        return None, "make-tokenizer failed: " + p.stdout.strip()[-200:]

    env = dict(os.environ)
    visible = os.environ.get("CUDA_VISIBLE_DEVICES")
    gpu = visible.split(",")[local_rank] if visible else str(local_rank)
    env.update({"CUDA_VISIBLE_DEVICES": gpu, "NANOCHAT_RANK": str(rank), "NANOCHAT_WORLD_SIZE": str(world),
                "NANOCHAT_MASTER_ADDR": "127.0.0.1", "NANOCHAT_MASTER_PORT": str(_free_port_base()),
                "NANOCHAT_SANDBOX": "bench", "OMP_NUM_THREADS": env.get("NANOCHAT_REF_OMP", "8")})
    total = args.warmup + args.steps
    cmd = [exe, "train", "--tokenizer", tok, "--layers", str(layers), "--hidden", str(hidden), "--heads", str(heads),
           "--kv-heads", str(kv), "--vocab", str(vocab), "--padded-vocab", str(vocab), "--seq", str(seq),
           "--batch", str(micro), "--grad-accum", str(accum), "--num-iterations", str(total),
           "--log-every", "1", "--device", args.ref_device, "--hw-check", args.ref_hw_check, "--seed", str(1234 + rank)]
    if args.preset == "tiny":
        cmd += ["--rope-base", "10000"]
    proc = subprocess.Popen(cmd, cwd=d, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, bufsize=1)
    steps = []            # (step, t_arrival, step_ms, tok_s, loss, phases)
    tail = []
    sampler = None
    clocks = {}
    t_start = time.perf_counter()
    deadline = t_start + float(os.environ.get("NANOCHAT_REF_TIMEOUT", "780"))
    error = None
    for line in proc.stdout:
        now = time.perf_counter()
        line = line.rstrip("\n")
        tail.append(line)
        del tail[:-40]
        m = STEP_RE.match(line)
        if m:
            steps.append((int(m.group(1)), now, float(m.group(4)), float(m.group(3)), m.group(2),
                          [float(m.group(i)) for i in range(5, 10)]))
            if len(steps) == args.warmup and rank == 0 and sampler_cls is not None:
                sampler = sampler_cls(int(gpu))
                sampler.start()
            if len(steps) == total and sampler is not None:
                clocks = sampler.stop()
                sampler = None
        if now > deadline:
            error = f"reference run passed its time limit after {len(steps)} of {total} steps"
            break
    if sampler is not None:
        clocks = sampler.stop()
    if error is not None:
        # past the limit: stop this rank's process (only the PID started here)
        proc.terminate()
    try:
        proc.wait(timeout=60)
    except Exception:
        proc.kill()
    try:
        os.remove(tok)
    except OSError:
        pass
    if error is None and len(steps) < total:
        error = "reference process ended early: " + " | ".join(tail[-4:])[-400:]
    log_dir = os.environ.get("NANOCHAT_REF_LOG_DIR")
    if log_dir and (error is not None or os.environ.get("NANOCHAT_REF_LOG_ALWAYS") == "1"):
        try:       # the last lines of this rank's reference process, for the record of a failed run
            os.makedirs(log_dir, exist_ok=True)
            with open(os.path.join(log_dir, f"reference_rank{rank}.log"), "w") as f:
                f.write("\n".join(tail) + "\n")
        except OSError:
            pass
    if error is not None:
        return None, error
    timed = steps[args.warmup:total]
    dev_ms = sum(s[2] for s in timed)
    t_begin = steps[args.warmup - 1][1] if args.warmup > 0 else t_start
    e2e_ms = (timed[-1][1] - t_begin) * 1e3
    phases = [sum(s[5][i] for s in timed) / len(timed) for i in range(5)]
    rec = {"dev_ms": dev_ms, "e2e_ms": e2e_ms, "clocks": clocks, "loss": timed[-1][4],
           "phases_ms": dict(zip(("data", "fwd", "bwd", "sync", "opt"), [round(x, 3) for x in phases])),
           "layers": layers, "hidden": hidden, "heads": heads, "kv": kv, "vocab": vocab, "seq": seq,
           "micro": micro, "accum": accum}
    return rec, None


def main(args, sampler_cls=None) -> int:
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("gloo")
    reason = ensure_built() if rank == 0 else None
    if dist is not None:
        dist.barrier()          # other ranks look at the build only after rank 0 has checked (or made) it
    if reason is None:
        try:
            import ctypes
            # fails here, with a reason, if the build or a CUDA library it links is missing on this machine
            ctypes.CDLL(os.path.join(ref_dir(), "libnanochat_ref.so"))
        except OSError as e:
            reason = f"libnanochat_ref.so does not load: {e}"
    if dist is not None:
        flag = torch.tensor([1 if reason is not None else 0])
        dist.all_reduce(flag, op=dist.ReduceOp.MAX)
        if int(flag) and reason is None:
            reason = "another rank could not load the reference build"
    if reason is not None:
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": reason}))
        if dist is not None:
            dist.destroy_process_group()
        return 0

    rec, err = run_train(args, sampler_cls)
    if dist is not None:
        import torch
        vals = torch.tensor([rec["dev_ms"] if rec else -1.0, rec["e2e_ms"] if rec else -1.0,
                             0.0 if err is None else 1.0], dtype=torch.float64)
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
        failed = float(vals[2]) > 0
        if not failed:
            rec["dev_ms"], rec["e2e_ms"] = float(vals[0]), float(vals[1])
        else:
            # every rank's own account: the first one that is not just "a peer went away" names the cause
            said = [None] * world
            dist.all_gather_object(said, err)
            own = [f"rank {r}: {e}" for r, e in enumerate(said) if e and "timed out waiting for a peer" not in e]
            err = (own[0] if own else next((f"rank {r}: {e}" for r, e in enumerate(said) if e), err))[:600]
    if rank == 0:
        if err is not None:
            print(json.dumps({"impl": "reference", "unavailable": err}))
        else:
            tokens = args.batch * rec["seq"] * world
            value = tokens * args.steps / (rec["dev_ms"] / 1e3)
            e2e = tokens * args.steps / (rec["e2e_ms"] / 1e3)
            window = ((rec["seq"] // 4 + 127) // 128) * 128
            line = {
                "metric": "train_tokens_per_sec", "value": round(value, 1), "unit": "tokens/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(rec["dev_ms"] / args.steps, 3),
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
                "data": "synthetic Zipf(1.1) documents tokenized by the reference's loader, random-init weights",
                "impl": "reference",
                "config": {"model": args.preset, "layers": rec["layers"], "hidden": rec["hidden"], "heads": rec["heads"],
                           "kv_heads": rec["kv"], "vocab": rec["vocab"], "global_batch": args.batch * world,
                           "per_gpu_batch": args.batch, "micro_batch": rec["micro"], "seq_len": rec["seq"],
                           "short_window": window, "window_pattern": "SSSL", "parallelism": f"dp{world}",
                           "optimizer": "Muon(ns=5)+AdamW, replicated; fp32 gradient ring all-reduce staged through host memory",
                           "note": "unmodified reference sources, hand-built for sm_100 (cuBLAS GEMMs, mma.sync flash attention); "
                                   f"its window formula gives {window} at seq {rec['seq']} and has no override",
                           "device_row": args.ref_device,
                           "hw_check": args.ref_hw_check + (" (its start-up gate fails an fp8 cublasLt case on sm_100 that "
                                                            "the bf16 run never uses)" if args.ref_hw_check == "off" else ""),
                           "l2": "per-step working set >> 126 MB L2, no flush needed",
                           "timing": "reference's own step_ms (device drained at phase boundaries), max over ranks"},
                "e2e": {"value": round(e2e, 1), "unit": "tokens/s",
                        "h2d_bytes_per_step": args.batch * rec["seq"] * 4 * 2, "d2h_bytes_per_step": 8,
                        "ms_per_step": round(rec["e2e_ms"] / args.steps, 3)},
                "gpu_launches": None, "final_loss": rec["loss"], "phases_ms": rec["phases_ms"], "clocks": rec["clocks"],
            }
            print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()
    return 0


GEN_RE = re.compile(r"^\[harness\] generate prompts=(\d+) prompt_tokens=(\d+) new_tokens=(\d+) wall_s=([\d.]+)")


def main_decode(args, sampler_cls=None) -> int:
    """Decode benchmark through the reference's own `GenerateMultiPrompt` (src/generate.cc:578-612): one replica per
    GPU, `--prompts` prompts of `--prompt-len` uniform-random ids, greedy decode of `--new-tokens` tokens each. The
    reference prefills each prompt at batch 1 and decodes it token by token, sampling on the host, so only the
    combined time exists: `value` is generated tokens / wall-clock seconds of the whole call (prefill included),
    max over ranks."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("gloo")
    reason = ensure_built() if rank == 0 else None
    if dist is not None:
        dist.barrier()
    d = ref_dir()
    exe = os.path.join(d, "ref_train")
    rec = None
    if reason is None:
        layers, hidden, heads, kv, vocab, seq = PRESETS[args.preset]
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        gpu = visible.split(",")[local_rank] if visible else str(local_rank)
        env = dict(os.environ)
        env.update({"CUDA_VISIBLE_DEVICES": gpu, "NANOCHAT_SANDBOX": "bench"})
        cmd = [exe, "generate", "--layers", str(layers), "--hidden", str(hidden), "--heads", str(heads), "--kv-heads",
               str(kv), "--vocab", str(vocab), "--padded-vocab", str(vocab), "--seq", str(seq), "--prompts",
               str(args.prompts), "--prompt-tokens", str(args.prompt_len), "--max-tokens", str(args.new_tokens),
               "--seed", str(rank)]
        sampler = None
        if rank == 0 and sampler_cls is not None:
            sampler = sampler_cls(int(gpu))
            sampler.start()
        try:
            p = subprocess.run(cmd, cwd=d, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                               timeout=float(os.environ.get("NANOCHAT_REF_TIMEOUT", "780")))
            out = p.stdout
        except subprocess.TimeoutExpired as e:
            out = (e.stdout or b"").decode() if isinstance(e.stdout, bytes) else (e.stdout or "")
            reason = "reference generate passed its time limit"
        clocks = sampler.stop() if sampler is not None else {}
        for line in out.splitlines():
            m = GEN_RE.match(line)
            if m:
                rec = {"new": int(m.group(3)), "wall_s": float(m.group(4)), "clocks": clocks}
        if rec is None and reason is None:
            reason = "reference generate printed no result: " + " | ".join(out.strip().splitlines()[-3:])[-300:]
    wall = rec["wall_s"] if rec else -1.0
    if dist is not None:
        import torch
        t = torch.tensor([wall, 1.0 if reason is not None else 0.0], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        wall = float(t[0])
        if float(t[1]) > 0 and reason is None:
            reason = "another rank's reference process failed"
    if rank == 0:
        if reason is not None:
            print(json.dumps({"impl": "reference", "unavailable": reason}))
        else:
            total_new = rec["new"] * world
            print(json.dumps({
                "metric": "decode_tokens_per_sec", "value": round(total_new / wall, 1), "unit": "tokens/s",
                "n_gpus": world, "steps": args.new_tokens, "warmup": 1, "ms_per_step": round(wall * 1e3 / args.new_tokens / args.prompts, 4),
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "impl": "reference",
                "data": "uniform-random prompt ids, random-init weights",
                "e2e": {"value": round(total_new / wall, 1), "unit": "tokens/s", "h2d_bytes_per_step": 4,
                        "d2h_bytes_per_step": PRESETS[args.preset][4] * 4},
                "gpu_launches": None, "clocks": rec["clocks"],
                "config": {"model": args.preset, "prompts_per_gpu": args.prompts, "prompt_len": args.prompt_len,
                           "new_tokens": args.new_tokens, "dtype": "bf16", "sampling": "greedy",
                           "note": "reference GenerateMultiPrompt: contiguous KV cache, batch-1 prefill and decode per "
                                   "prompt, host sampling; wall clock of the whole call (prefill included)",
                           "parallelism": f"{world} replicas"}}))
    if dist is not None:
        dist.destroy_process_group()
    return 0
