"""Chat evaluation over the five tasks with per-task isolation and the centred "core" means.

Surface of the reference's `ChatEvaluator` (python/nanochat_cpp/chat.py:533-705): `task(name, **options)` evaluates
one task and lets a failure propagate; `run(tasks)` turns a failing task into a skipped `TaskReport`; `chat_core` and
`categorical_core` are means of (accuracy - baseline) / (1 - baseline) and are `None` when a task was skipped.
Datasets arrive through a loader seam (the reference's `seam.register_hub_loader`): a callable
`loader(task_name) -> Task`. Nothing here downloads; `directory_loader(path)` reads `<path>/<task>.jsonl`.
"""
from __future__ import annotations

import dataclasses
import os
from typing import Callable, Dict, Optional, Sequence, Tuple

from .tasks import ARC, GSM8K, MMLU, HumanEval, Task, evaluate_task

ALL_TASKS = ("ARC-Easy", "ARC-Challenge", "MMLU", "GSM8K", "HumanEval")
CATEGORICAL_TASKS = ("ARC-Easy", "ARC-Challenge", "MMLU")
GENERATIVE_TASKS = ("GSM8K", "HumanEval")
BASELINES = {"ARC-Easy": 0.25, "ARC-Challenge": 0.25, "MMLU": 0.25, "GSM8K": 0.0, "HumanEval": 0.0}
_TASK_TYPES = {"ARC-Easy": ARC, "ARC-Challenge": ARC, "MMLU": MMLU, "GSM8K": GSM8K, "HumanEval": HumanEval}

_registered_loader: Optional[Callable[[str], Task]] = None


def register_task_loader(loader: Optional[Callable[[str], Task]]) -> None:
    """Process-wide dataset loader used when a `ChatEvaluator` is built without one."""
    global _registered_loader
    _registered_loader = loader


def directory_loader(path: str) -> Callable[[str], Task]:
    """Loader over local JSON-lines files named after the tasks (`ARC-Easy.jsonl`, `MMLU.jsonl`, ...)."""
    def load(name: str) -> Task:
        file = os.path.join(path, name + ".jsonl")
        if not os.path.exists(file):
            raise FileNotFoundError(f"no dataset file for task {name!r}: {file}")
        return _TASK_TYPES[name].from_jsonl(file)
    return load


def build_task(name: str, loader: Optional[Callable[[str], Task]] = None) -> Task:
    if name not in ALL_TASKS:
        raise ValueError(f"unknown task {name!r}; valid: {list(ALL_TASKS)}")
    loader = loader or _registered_loader
    if loader is None:
        base = os.environ.get("NANOCHAT_BASE_DIR")
        if not base:
            raise RuntimeError("no task loader registered and NANOCHAT_BASE_DIR is not set")
        loader = directory_loader(os.path.join(base, "eval_tasks"))
    return loader(name)


@dataclasses.dataclass(frozen=True)
class TaskReport:
    name: str
    correct: int
    total: int
    accuracy: float
    baseline: float
    skipped: bool = False
    error: Optional[str] = None


@dataclasses.dataclass(frozen=True)
class ChatReport:
    tasks: Tuple[TaskReport, ...]
    chat_core: Optional[float]
    categorical_core: Optional[float]


def centered_mean(reports: Sequence[TaskReport], names: Sequence[str]) -> Optional[float]:
    """Mean of (accuracy - baseline) / (1 - baseline) over `names`; None if one of them is missing or skipped."""
    by_name = {r.name: r for r in reports}
    values = []
    for name in names:
        r = by_name.get(name)
        if r is None or r.skipped:
            return None
        denom = 1.0 - BASELINES[name]
        if denom == 0.0:
            return None
        values.append((r.accuracy - BASELINES[name]) / denom)
    return sum(values) / len(values) if values else None


class ChatEvaluator:
    def __init__(self, model, tokenizer, *, task_loader: Optional[Callable[[str], Task]] = None, score_batch: int = 8):
        self.model, self.tokenizer = model, tokenizer
        self.task_loader = task_loader
        self.score_batch = score_batch      # rows per scoring forward: bounds the logits workspace

    def task(self, name: str, **options) -> TaskReport:
        """Evaluates one task; a failure propagates to the caller."""
        task = build_task(name, self.task_loader)
        r = evaluate_task(task, self.model, self.tokenizer, max_problems=options.get("max_problems"),
                          batch=self.score_batch, num_samples=int(options.get("num_samples", 1)),
                          max_tokens=int(options.get("max_new_tokens", 512)),
                          temperature=float(options.get("temperature", 0.0)), top_k=int(options.get("top_k", 50)),
                          seed=int(options.get("seed", 0)))
        total = int(r["total"])
        return TaskReport(name, int(r["passed"]), total, r["passed"] / total if total else float("nan"),
                          BASELINES[name])

    def run(self, tasks: Optional[Sequence[str]] = None, *, max_problems: Optional[int] = None, seed: int = 0,
            data_dir: Optional[str] = None) -> ChatReport:
        """Evaluates `tasks` (default: all five); a task that raises becomes a skipped report with the error text."""
        if data_dir is not None:
            os.environ["NANOCHAT_BASE_DIR"] = os.path.abspath(data_dir)
        names = list(tasks) if tasks is not None else list(ALL_TASKS)
        reports = []
        for name in names:
            try:
                reports.append(self.task(name, max_problems=max_problems, seed=seed))
            except (KeyboardInterrupt, GeneratorExit):
                raise
            except BaseException as error:  # noqa: BLE001 - one task must not take the others down
                reports.append(TaskReport(name, 0, 0, float("nan"), BASELINES.get(name, 0.0), skipped=True,
                                          error=f"{type(error).__name__}: {error}"))
        return ChatReport(tuple(reports), centered_mean(reports, ALL_TASKS), centered_mean(reports, CATEGORICAL_TASKS))
