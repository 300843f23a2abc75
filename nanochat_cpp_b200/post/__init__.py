"""Post-training: supervised fine-tuning over packed rows, and the policy-gradient step with its worker."""
from .sft import SftConfig, SftShard, load_sft_shard, run_sft, save_sft_shard, sft_optimizer_config, sft_scheduler_config
from .rl import RlWorker, rl_step

__all__ = ["SftConfig", "SftShard", "load_sft_shard", "save_sft_shard", "run_sft", "sft_optimizer_config",
           "sft_scheduler_config", "RlWorker", "rl_step"]
