"""Generation with the calculator tool.

While a row decodes, `<|python_start|> expr <|python_end|>` from the model is a tool call: the expression is
evaluated by `use_calculator` and `<|output_start|> result <|output_end|>` is forced into the row (mask 0: the
model did not sample it). A row ends at `<|assistant_end|>` or `<|bos|>`. Behaviour of the reference's `ChatEngine`
(python/nanochat_cpp/chat.py:402-531), which mirrors upstream nanochat's engine; decoding itself runs on this
package's paged-KV inference engine.
"""
from __future__ import annotations

import ast
import operator
from collections import deque
from typing import Dict, List, Optional, Sequence

import torch

from .render import special_ids

_OPS = {ast.Add: operator.add, ast.Sub: operator.sub, ast.Mult: operator.mul, ast.Div: operator.truediv}
_BANNED = ("__", "import", "exec", "eval", "compile", "open", "file", "input", "raw_input", "globals", "locals",
           "vars", "dir", "getattr", "setattr", "delattr", "hasattr")


def _value(node):
    if isinstance(node, ast.Expression):
        return _value(node.body)
    if isinstance(node, ast.Constant) and not isinstance(node.value, bool) and isinstance(node.value,
                                                                                          (int, float, str)):
        return node.value
    if isinstance(node, ast.UnaryOp) and isinstance(node.op, ast.USub):
        return -_value(node.operand)
    if isinstance(node, ast.BinOp) and type(node.op) in _OPS:
        return _OPS[type(node.op)](_value(node.left), _value(node.right))
    if (isinstance(node, ast.Call) and not node.keywords and len(node.args) == 1
            and isinstance(node.func, ast.Attribute) and node.func.attr == "count"):
        hay, needle = _value(node.func.value), _value(node.args[0])
        if isinstance(hay, str) and isinstance(needle, str):
            return hay.count(needle)
    raise ValueError("unsupported expression")


def use_calculator(expr: str) -> Optional[str]:
    """The text the tool returns for `expr`, or None when the expression is not allowed: plain arithmetic
    (`+ - * /`, parentheses, no `**`; thousands separators are dropped) or a `'text'.count('t')` call."""
    expr = expr.replace(",", "")
    if all(c in "0123456789*+-/.() " for c in expr):
        if "**" in expr:
            return None
    else:
        ok = "abcdefghijklmnopqrstuvwxyzABCDEFGHIJKLMNOPQRSTUVWXYZ0123456789'\"()._ "
        if not all(c in ok for c in expr) or any(b in expr.lower() for b in _BANNED) or ".count(" not in expr:
            return None
    try:
        v = _value(ast.parse(expr, mode="eval"))
    except Exception:
        return None
    if isinstance(v, bool) or not isinstance(v, (int, float, str)):
        return None
    return str(v)


class ChatEngine:
    def __init__(self, model, tokenizer, use_cuda_graph: bool = False):
        from ..inference import InferenceEngine
        self.gpt = getattr(model, "gpt", model)
        self.tokenizer = tokenizer
        self.sp: Dict[str, int] = special_ids(tokenizer)
        self.engine = InferenceEngine(self.gpt, use_cuda_graph=use_cuda_graph)

    def generate(self, prompt: Sequence[int], *, num_samples: int = 1, max_tokens: int = 256,
                 temperature: float = 1.0, top_k: int = 0, seed: int = 0):
        """Returns `num_samples` rows of (tokens, mask); tokens start with the prompt and exclude the end marker."""
        from ..inference import GenerateParams, generate_multi
        sp = self.sp
        rows = max(1, num_samples)
        state = [dict(queue=deque(), in_py=False, expr=[], seen=len(prompt)) for _ in range(rows)]

        def forced(r: int, tokens: List[int]):
            st = state[r]
            for t in tokens[st["seen"]:]:          # advance the tool state machine over what was appended
                if t == sp["<|python_start|>"]:
                    st["in_py"], st["expr"] = True, []
                elif t == sp["<|python_end|>"] and st["in_py"]:
                    st["in_py"] = False
                    result = use_calculator(self.tokenizer.decode(st["expr"])) if st["expr"] else None
                    if result is not None:
                        st["queue"].extend([sp["<|output_start|>"], *self.tokenizer.encode(result),
                                            sp["<|output_end|>"]])
                elif st["in_py"]:
                    st["expr"].append(t)
            st["seen"] = len(tokens)
            return st["queue"].popleft() if st["queue"] else None

        params = GenerateParams(num_samples=rows, max_tokens=max_tokens, temperature=temperature, top_k=top_k,
                                seed=seed, stop_ids=(sp["<|assistant_end|>"], sp["<|bos|>"]))
        out = generate_multi(self.engine, torch.tensor([list(prompt)], dtype=torch.int64), params, forced=forced)
        return [(r.tokens, r.mask) for r in out]

    def reply(self, conversation: dict, **kw) -> str:
        """Text of one sampled assistant reply to `conversation` (whose last message is a placeholder reply)."""
        from .render import render_for_completion
        prompt = render_for_completion(conversation, self.tokenizer)
        tokens, mask = self.generate(prompt, num_samples=1, **kw)[0]
        return self.tokenizer.decode(tokens[len(prompt):])
