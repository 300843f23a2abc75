"""The chat template.

A conversation `{"messages": [{"role", "content"}, ...]}` becomes
`<|bos|> (<|user_start|> text <|user_end|> <|assistant_start|> reply <|assistant_end|>)*`. A leading system message
is folded into the first user message with a blank line between. An assistant reply is a string or a list of parts:
`text`, `python` (a tool call, wrapped in `<|python_start|>`/`<|python_end|>`) and `python_output` (what the tool
returned, wrapped in `<|output_start|>`/`<|output_end|>`). The training mask is 1 on what the assistant must learn
to produce (its text, its tool calls, its end token) and 0 elsewhere (BOS, user text, tool output). Same template
and mask as the reference (python/nanochat_cpp/chat.py:154-235), which takes them from upstream nanochat.
"""
from __future__ import annotations

import copy
from typing import Dict, List, Tuple

CHAT_SPECIALS = ("<|bos|>", "<|user_start|>", "<|user_end|>", "<|assistant_start|>", "<|assistant_end|>",
                 "<|python_start|>", "<|python_end|>", "<|output_start|>", "<|output_end|>")


def special_ids(tokenizer) -> Dict[str, int]:
    """Name -> id for the chat markers; works with this package's tokenizers and the API wrapper."""
    get = getattr(tokenizer, "encode_special", None) or getattr(tokenizer, "special_id")
    out = {}
    for name in CHAT_SPECIALS:
        i = get(name)
        if i is None or i < 0:
            raise ValueError(f"the tokenizer lacks the chat special token {name}")
        out[name] = int(i)
    return out


def _fold_system(messages: List[dict]) -> List[dict]:
    messages = copy.deepcopy(messages)
    if not messages:
        raise ValueError("a conversation must have at least one message")
    if messages[0]["role"] == "system":
        if len(messages) < 2 or messages[1]["role"] != "user":
            raise ValueError("a system message must be followed by a user message")
        messages[1]["content"] = messages[0]["content"] + "\n\n" + messages[1]["content"]
        messages = messages[1:]
    for i, m in enumerate(messages):
        want = "user" if i % 2 == 0 else "assistant"
        if m["role"] != want:
            raise ValueError(f"message {i} has role {m['role']} but should be {want}")
    return messages


def _assistant_tokens(content, tokenizer, sp) -> Tuple[List[int], List[int]]:
    ids: List[int] = []
    mask: List[int] = []

    def add(tokens, keep):
        ids.extend(tokens)
        mask.extend([keep] * len(tokens))

    if isinstance(content, str):
        add(tokenizer.encode(content), 1)
        return ids, mask
    for part in content:
        kind = part["type"]
        if kind == "text":
            add(tokenizer.encode(part["text"]), 1)
        elif kind == "python":
            add([sp["<|python_start|>"]], 1)
            add(tokenizer.encode(part["text"]), 1)
            add([sp["<|python_end|>"]], 1)
        elif kind == "python_output":
            add([sp["<|output_start|>"]], 0)
            add(tokenizer.encode(part["text"]), 0)
            add([sp["<|output_end|>"]], 0)
        else:
            raise ValueError(f"unknown part type: {kind}")
    return ids, mask


def render_conversation(conversation: dict, tokenizer, max_tokens: int = 2048) -> Tuple[List[int], List[int]]:
    """(ids, mask) for supervised training, truncated to `max_tokens`."""
    sp = special_ids(tokenizer)
    ids, mask = [sp["<|bos|>"]], [0]
    for m in _fold_system(conversation["messages"]):
        if m["role"] == "user":
            body = tokenizer.encode(m["content"])
            ids += [sp["<|user_start|>"], *body, sp["<|user_end|>"]]
            mask += [0] * (len(body) + 2)
        else:
            a_ids, a_mask = _assistant_tokens(m["content"], tokenizer, sp)
            ids += [sp["<|assistant_start|>"], *a_ids, sp["<|assistant_end|>"]]
            mask += [0, *a_mask, 1]
    return ids[:max_tokens], mask[:max_tokens]


def render_for_completion(conversation: dict, tokenizer) -> List[int]:
    """Prompt ids for generation: the conversation without its last assistant reply, ending in
    `<|assistant_start|>`."""
    messages = list(conversation["messages"])
    if not messages or messages[-1]["role"] != "assistant":
        raise ValueError("the last message must be from the assistant")
    sp = special_ids(tokenizer)
    ids = [sp["<|bos|>"]]
    for m in _fold_system(messages[:-1]):
        if m["role"] == "user":
            ids += [sp["<|user_start|>"], *tokenizer.encode(m["content"]), sp["<|user_end|>"]]
        else:
            a_ids, _ = _assistant_tokens(m["content"], tokenizer, sp)
            ids += [sp["<|assistant_start|>"], *a_ids, sp["<|assistant_end|>"]]
    ids.append(sp["<|assistant_start|>"])
    return ids
