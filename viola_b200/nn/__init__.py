"""FP8 neural-network modules: Linear, gated MLP and the expert (grouped) linear."""

from .linear import Linear
from .mlp import MLP
from .grouped import GroupedLinear

__all__ = ["Linear", "MLP", "GroupedLinear"]
