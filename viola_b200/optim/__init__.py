"""Optimizers: whole-matrix base class, FP8-momentum Muon and the master-weight binder."""

from .matrix import MatrixOptimizer
from .muon import FP8Muon
from .master_weights import bind_optimizer

__all__ = ["MatrixOptimizer", "FP8Muon", "bind_optimizer"]
