"""Distributed training layer: engine, sharding, owner-directed transfers, EMA, checkpoints."""

from .communication import gather_to_owner, partial_gradient, replicate_tensor, write_from_owner
from .ema import ShardedEMA
from .engine import violaEngine
from .partition import MatrixPartition

__all__ = ["violaEngine", "MatrixPartition", "ShardedEMA", "gather_to_owner", "partial_gradient",
           "replicate_tensor", "write_from_owner"]
