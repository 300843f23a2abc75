from .loop import TrainConfig, Trainer, format_log_line  # noqa: F401
