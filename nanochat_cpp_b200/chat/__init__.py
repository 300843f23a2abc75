"""Chat: the conversation template, the tool-using engine, evaluation tasks and the SFT data pipeline."""
from .render import CHAT_SPECIALS, render_conversation, render_for_completion
from .engine import ChatEngine, use_calculator
from .sft_data import PackedRowStream, TaskMixture, pack_rows
from .tasks import ARC, GSM8K, MMLU, HumanEval, Task, evaluate_task
from .evaluator import (ALL_TASKS, BASELINES, CATEGORICAL_TASKS, ChatEvaluator, ChatReport, TaskReport, build_task,
                        centered_mean, directory_loader, register_task_loader)

__all__ = ["CHAT_SPECIALS", "render_conversation", "render_for_completion", "ChatEngine", "use_calculator",
           "PackedRowStream", "TaskMixture", "pack_rows", "Task", "ARC", "MMLU", "GSM8K", "HumanEval", "evaluate_task",
           "ALL_TASKS", "BASELINES", "CATEGORICAL_TASKS", "ChatEvaluator", "ChatReport", "TaskReport", "build_task",
           "centered_mean", "directory_loader", "register_task_loader"]
