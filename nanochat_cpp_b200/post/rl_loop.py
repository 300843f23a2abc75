"""The reinforcement-learning driver: Python renders prompts, scores rollouts and computes advantages; a worker
(in this process, or a child process behind the line protocol of `post.rl`) samples and takes the optimizer steps.

One step (reference python/nanochat_cpp/rl.py `run`): every prompt is sampled `num_samples` times in one rollout
request; a reply's reward comes from the task; the advantage of a reply is its reward minus the mean reward of its
prompt's group; the step's batch holds every reply (prompt positions and padding carry target -1, sampled
positions carry the token and the reply's advantage as weight) and goes to the worker as one `advantage` request.
"""
from __future__ import annotations

import subprocess
import sys
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

from ..chat.render import render_for_completion, special_ids
from .rl import RlWorker, _fields


class InProcessWorker:
    def __init__(self, worker: RlWorker):
        self.worker = worker

    def request(self, line: str) -> Dict[str, str]:
        return _parse(self.worker.handle(line))

    def close(self) -> None:
        pass


class PipeWorker:
    """A child `rl_worker` process; requests and replies are single text lines on its stdin / stdout."""

    def __init__(self, argv: Sequence[str], env: Optional[dict] = None):
        self.proc = subprocess.Popen(list(argv), stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env,
                                     bufsize=1)

    @classmethod
    def spawn(cls, model_flags: Sequence[str], checkpoint: str = "", device: str = "auto", env=None):
        argv = [sys.executable, "-m", "nanochat_cpp_b200.cli", "rl_worker", *model_flags, "--device", device]
        if checkpoint:
            argv += ["--checkpoint", checkpoint]
        return cls(argv, env)

    @classmethod
    def spawn_native(cls, model_flags: Sequence[str], checkpoint: str = "", device: str = "cpu", env=None):
        """The native worker (`nanochat_cli rl_worker`, C++ on the CPU or on a CUDA device): the same line protocol."""
        import os
        exe = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "nanochat_cli")
        argv = [exe, "rl_worker", *model_flags, "--device", device]
        if checkpoint:
            argv += ["--checkpoint", checkpoint]
        return cls(argv, env)

    def request(self, line: str) -> Dict[str, str]:
        self.proc.stdin.write(line + "\n")
        self.proc.stdin.flush()
        reply = self.proc.stdout.readline()
        if not reply:
            raise RuntimeError("the worker closed its pipe")
        return _parse(reply)

    def close(self) -> None:
        try:
            if self.proc.poll() is None:
                self.request("quit")
        finally:
            self.proc.stdin.close()
            self.proc.wait(timeout=30)


def _parse(reply: str) -> Dict[str, str]:
    words = reply.strip().split(" ")
    f = _fields(words[1:])
    f["type"] = words[0]
    if f.get("ok") != "1":
        raise RuntimeError(f"worker refused {words[0]}: {f.get('error', reply.strip())}")
    return f


def advantages(group: Sequence[float]) -> List[float]:
    mean = sum(group) / len(group)
    return [r - mean for r in group]


@dataclass
class RlReport:
    steps: int
    losses: List[float] = field(default_factory=list)
    grad_norms: List[float] = field(default_factory=list)
    mean_rewards: List[float] = field(default_factory=list)
    checkpoint: Optional[str] = None


def _batch(rows: List[List[int]], masks: List[List[int]], adv: Sequence[float], pad: int):
    """Rows right-padded to one length; targets are the next token where it was sampled, else -1."""
    seq = max(len(r) for r in rows)
    tokens, targets, weights = [], [], []
    for r, m, a in zip(rows, masks, adv):
        n = len(r)
        tokens += r + [pad] * (seq - n)
        tgt = [r[i + 1] if i + 1 < n and m[i + 1] else -1 for i in range(seq)]
        targets += tgt
        weights += [a if t >= 0 else 0.0 for t in tgt]
    return tokens, targets, weights, seq


def run(worker, task, conversations: Sequence[dict], tokenizer, *, num_samples: int = 4, steps: int = 1,
        max_tokens: int = 64, temperature: float = 1.0, top_k: int = 0, seed: int = 0, num_passes: int = 1,
        examples_per_rank: Optional[int] = None, checkpoint: Optional[str] = None,
        checkpoint_interval: int = 0, on_step: Optional[Callable] = None) -> RlReport:
    if not conversations:
        raise ValueError("prompts must not be empty")
    if steps < 1 or num_samples < 1:
        raise ValueError("steps and num_samples must be positive")
    sp = special_ids(tokenizer)
    pad, stop = sp["<|bos|>"], sp["<|assistant_end|>"]
    prompts = [render_for_completion(c, tokenizer) for c in conversations]
    plen = max(len(p) for p in prompts)
    flat = [t for p in prompts for t in [pad] * (plen - len(p)) + p]       # left-padded to one length
    per_rank = examples_per_rank or len(prompts)
    rep = RlReport(steps=steps, checkpoint=checkpoint)
    for step in range(1, steps + 1):
        r = worker.request(f"rollout prompt_len={plen} num_prompts={len(prompts)} prompts={','.join(map(str, flat))} "
                           f"num_samples={num_samples} max_tokens={max_tokens} temperature={temperature:.9g} "
                           f"top_k={top_k} seed={seed + step - 1} stop_id={stop}")
        lengths = [int(x) for x in r["lengths"].split(",")]
        toks = [int(x) for x in r["tokens"].split(",")]
        msk = [int(x) for x in r["masks"].split(",")]
        rows, masks, at = [], [], 0
        for n in lengths:
            rows.append(toks[at:at + n])
            masks.append(msk[at:at + n])
            at += n
        rewards = []
        for i, conv in enumerate(conversations):
            for s in range(num_samples):
                k = i * num_samples + s
                text = tokenizer.decode([t for t, m in zip(rows[k], masks[k]) if m])
                fn = getattr(task, "reward", None) or (lambda c, t: float(task.evaluate(c, t)))
                rewards.append(float(fn(conv, text)))
        adv = [a for i in range(len(prompts)) for a in advantages(rewards[i * num_samples:(i + 1) * num_samples])]
        tokens, targets, weights, seq = _batch(rows, masks, adv, pad)
        a = worker.request(f"advantage batch={len(rows)} seq={seq} num_passes={num_passes} "
                           f"examples_per_rank={per_rank} tokens={','.join(map(str, tokens))} "
                           f"targets={','.join(map(str, targets))} "
                           f"advantages={','.join('%.9g' % w for w in weights)}")
        rep.losses.append(float(a["loss"]))
        rep.grad_norms.append(float(a["grad_norm"]))
        rep.mean_rewards.append(sum(rewards) / len(rewards))
        if on_step is not None:
            on_step(step, rep.losses[-1], rep.grad_norms[-1], rewards)
        if checkpoint and checkpoint_interval and step % checkpoint_interval == 0:
            worker.request(f"save path={checkpoint}")
    if checkpoint:
        worker.request(f"save path={checkpoint}")
    return rep
