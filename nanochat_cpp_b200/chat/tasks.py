"""Evaluation tasks: ARC, MMLU (multiple choice, scored by comparing the logits of the answer letters), GSM8K and
HumanEval (generative, scored on the sampled reply).

Same task definitions as the reference (python/nanochat_cpp/tasks.py, from upstream nanochat's `tasks/`): the
multiple-choice prompt format, the GSM8K `<<expr=result>>` tool-call parts and `#### answer` extraction, the
HumanEval program extraction. Datasets come from local files (JSON lines with the public datasets' field names),
because nothing here downloads; `Task(rows)` also takes rows already in memory.
"""
from __future__ import annotations

import json
import re
import subprocess
import sys
from typing import Dict, List, Optional, Sequence

import numpy as np


class Task:
    eval_type = "generative"     # or "categorical"

    def __init__(self, rows: Sequence[dict], start: int = 0, stop: Optional[int] = None, step: int = 1):
        # a row source that can slice itself without reading every row (a parquet-backed dataset) stays lazy
        self.rows = rows.lazy_slice(start, stop, step) if hasattr(rows, "lazy_slice") else list(rows)[start:stop:step]

    @classmethod
    def from_jsonl(cls, path: str, **kw):
        with open(path, encoding="utf-8") as f:
            return cls([json.loads(line) for line in f if line.strip()], **kw)

    def __len__(self) -> int:
        return len(self.rows)

    def __getitem__(self, i: int) -> dict:
        return self.get_example(i)

    def get_example(self, i: int) -> dict:
        raise NotImplementedError

    def evaluate(self, conversation: dict, reply: str) -> bool:
        raise NotImplementedError


def render_mc(question: str, letters: Sequence[str], choices: Sequence[str]) -> str:
    q = f"Multiple Choice question: {question}\n"
    q += "".join(f"- {c}={l}\n" for l, c in zip(letters, choices))
    return q + "\nRespond only with the letter of the correct answer."


class ARC(Task):
    """Rows: {"question", "choices": {"text": [...], "label": [...]}, "answerKey"}."""
    eval_type = "categorical"

    def get_example(self, i):
        r = self.rows[i]
        letters, texts = r["choices"]["label"], r["choices"]["text"]
        assert r["answerKey"] in letters
        return {"messages": [{"role": "user", "content": render_mc(r["question"], letters, texts)},
                             {"role": "assistant", "content": r["answerKey"]}], "letters": list(letters)}

    def evaluate(self, conversation, reply):
        return reply == conversation["messages"][-1]["content"]


class MMLU(Task):
    """Rows: {"question", "choices": [4 strings], "answer": index, "subject"}."""
    eval_type = "categorical"
    letters = ("A", "B", "C", "D")

    def get_example(self, i):
        r = self.rows[i]
        assert len(r["choices"]) == 4
        return {"messages": [{"role": "user", "content": render_mc(r["question"], self.letters, r["choices"])},
                             {"role": "assistant", "content": self.letters[r["answer"]]}],
                "subject": r.get("subject", ""), "letters": list(self.letters)}

    def evaluate(self, conversation, reply):
        return reply == conversation["messages"][-1]["content"]


_ANSWER = re.compile(r"#### (\-?[0-9\.\,]+)")


def extract_answer(text: str) -> Optional[str]:
    m = _ANSWER.search(text)
    return m.group(1).strip().replace(",", "") if m else None


class GSM8K(Task):
    """Rows: {"question", "answer"}; `<<12*3=36>>` annotations in the answer become calculator tool calls."""

    def get_example(self, i):
        r = self.rows[i]
        parts = []
        for piece in re.split(r"(<<[^>]+>>)", r["answer"]):
            if piece.startswith("<<") and piece.endswith(">>"):
                inner = piece[2:-2]
                expr, result = inner.rsplit("=", 1) if "=" in inner else (inner, "")
                parts += [{"type": "python", "text": expr}, {"type": "python_output", "text": result}]
            elif piece:
                parts.append({"type": "text", "text": piece})
        return {"messages": [{"role": "user", "content": r["question"]}, {"role": "assistant", "content": parts}]}

    def evaluate(self, conversation, reply):
        last = conversation["messages"][-1]["content"]
        ref = extract_answer(last[-1]["text"] if isinstance(last, list) else last)
        return ref is not None and extract_answer(reply) == ref

    def reward(self, conversation, reply) -> float:
        return float(self.evaluate(conversation, reply))


def extract_imports(prompt: str) -> str:
    return "\n".join(l for l in prompt.split("\n") if l.strip().startswith(("import ", "from ")))


def extract_program(completion: str) -> str:
    blocks = re.findall(r"```(?:python)?\s*\n(.*?)\n```", completion, re.DOTALL)
    return blocks[0].strip() if blocks else completion.strip()


class HumanEval(Task):
    """Rows: {"prompt", "canonical_solution", "entry_point", "test"}. Programs run in a child interpreter with a
    time limit; pass `executor=` (a callable `code -> result with .success`, e.g. `bridge.hub_data.code_executor()`)
    to run them under resource limits in a scrubbed environment instead."""

    def __init__(self, rows, *args, executor=None, **kw):
        super().__init__(rows, *args, **kw)
        self.executor = executor

    def get_example(self, i):
        r = self.rows[i]
        return {"messages": [{"role": "user", "content": r["prompt"]},
                             {"role": "assistant", "content": r["prompt"] + r["canonical_solution"]}],
                "entry_point": r["entry_point"], "test": r["test"]}

    def evaluate(self, conversation, reply, timeout: float = 5.0):
        program = "\n\n".join([extract_imports(conversation["messages"][0]["content"]), extract_program(reply),
                               conversation["test"], f"check({conversation['entry_point']})"])
        if self.executor is not None:
            return bool(self.executor(program).success)
        try:
            return subprocess.run([sys.executable, "-I", "-c", program], capture_output=True,
                                  timeout=timeout).returncode == 0
        except subprocess.TimeoutExpired:
            return False


def evaluate_task(task: Task, model, tokenizer, *, max_problems: Optional[int] = None, batch: int = 8,
                  num_samples: int = 1, max_tokens: int = 256, temperature: float = 0.0, top_k: int = 50,
                  seed: int = 0) -> Dict[str, float]:
    """Accuracy of `model` on `task`. Categorical tasks compare the logits of the answer letters at the position
    after `<|assistant_start|>` (one batched forward per `batch` problems, no sampling); generative tasks sample
    `num_samples` replies through the chat engine and count a problem as passed when any of them passes."""
    from ..eval import score_batch
    from .engine import ChatEngine
    from .render import render_for_completion
    gpt = getattr(model, "gpt", model)
    n = len(task) if max_problems is None else min(len(task), max_problems)
    passed = 0
    if task.eval_type == "categorical":
        pad = tokenizer.get_bos_token_id() if hasattr(tokenizer, "get_bos_token_id") else tokenizer.bos_id
        for b0 in range(0, n, batch):
            convs = [task[i] for i in range(b0, min(n, b0 + batch))]
            prompts = [render_for_completion(c, tokenizer) for c in convs]
            width = max(len(p) for p in prompts)
            toks = np.full((len(prompts), width), pad, dtype=np.int64)
            focus = []
            for r, (p, c) in enumerate(zip(prompts, convs)):
                toks[r, :len(p)] = p
                ids = [tokenizer.encode(l)[0] for l in c["letters"]]
                focus.append((len(p) - 1, ids))
            res = score_batch(gpt, toks, [len(p) for p in prompts], focus)
            for c, r in zip(convs, res):
                pick = c["letters"][int(np.argmax(r.focus_logits))]
                passed += bool(task.evaluate(c, pick))
    else:
        eng = ChatEngine(gpt, tokenizer)
        for i in range(n):
            c = task[i]
            prompt = render_for_completion(c, tokenizer)
            rows = eng.generate(prompt, num_samples=num_samples, max_tokens=max_tokens, temperature=temperature,
                                top_k=top_k, seed=seed + i)
            passed += any(task.evaluate(c, tokenizer.decode(t[len(prompt):])) for t, _ in rows)
    return {"accuracy": passed / max(n, 1), "passed": passed, "total": n}
