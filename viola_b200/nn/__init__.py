"""FP8 neural-network modules: Linear, gated MLP and the expert (grouped) linear."""

from .linear import Linear
from .mlp import MLP
from .grouped import GroupedLinear
from .fused import activation_linear, gated_residual, norm_modulate_linear, norm_modulate_mlp

__all__ = ["Linear", "MLP", "GroupedLinear", "gated_residual", "norm_modulate_linear", "norm_modulate_mlp",
           "activation_linear"]
