"""Data parallelism: owner-sharded optimizer with a fused peer-memory transport and an NCCL baseline."""
from .dp import DataParallel, adamw_slice, assign_owners

__all__ = ["DataParallel", "adamw_slice", "assign_owners"]
