from .optimizer import Optimizer, OptimizerConfig, build_groups  # noqa: F401
from .scheduler import Scheduler, SchedulerConfig  # noqa: F401
