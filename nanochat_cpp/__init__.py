"""`nanochat_cpp`: the import name of the reference's Python package, served by `nanochat_cpp_b200`.

    import nanochat_cpp as nc
    model = nc.Model(nc.Config(12))

Sub-modules keep the reference's names: `nanochat_cpp.chat`, `.tasks`, `.rl`, `.sft`, `.sft_data`, `.runtime`,
`.pipeline`, `.checkpoint`, `.data`.
"""
import sys as _sys

from nanochat_cpp_b200 import api as _api
from nanochat_cpp_b200.api import (Config, Evaluator, GeneratedRow, Model, Optimizer, ParamView, ScoreReport,  # noqa: F401
                                   TokenData, Tokenizer, Trainer, evaluate, model_flags, no_grad, tokenizer)
from nanochat_cpp_b200 import chat as _chat, native_mesh as mesh, pipeline, runtime  # noqa: F401
from nanochat_cpp_b200.chat import engine as _engine, render as _render, sft_data, tasks  # noqa: F401
from nanochat_cpp_b200.post import rl_loop as rl, sft  # noqa: F401
from nanochat_cpp_b200.train import checkpointer as checkpoint  # noqa: F401
from nanochat_cpp_b200.data import native as data  # noqa: F401

chat = _chat
api = _api
for _name, _mod in (("chat", chat), ("tasks", tasks), ("rl", rl), ("sft", sft), ("sft_data", sft_data),
                    ("runtime", runtime), ("mesh", mesh), ("pipeline", pipeline), ("checkpoint", checkpoint), ("data", data),
                    ("api", api)):
    _sys.modules[__name__ + "." + _name] = _mod

__all__ = ["Config", "Tokenizer", "Model", "Optimizer", "TokenData", "Trainer", "Evaluator", "no_grad", "evaluate",
           "model_flags", "tokenizer", "chat", "tasks", "rl", "sft", "sft_data", "runtime", "mesh", "pipeline", "checkpoint",
           "data"]
