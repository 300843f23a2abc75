"""nanochat on B200: PyTorch orchestration over hand-written sm_100a kernels.

Sub-packages: `models` (graph + parameters), `ops` (operators: CUDA kernels and their
PyTorch definitions), `optim` (Muon + AdamW + schedules), `parallel` (data parallel with
owner-sharded optimizer and the fused communication kernels), `train` (loop, logging,
checkpointing, performance model), `data` (loader, tokenizer, formats - native C++),
`inference` (paged KV cache engine), `utils`.
"""
from .config import Config, preset  # noqa: F401

__version__ = "0.1.0"
