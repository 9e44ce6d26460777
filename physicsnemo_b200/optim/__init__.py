"""Optimizers: ``Muon``, ``CombinedOptimizer`` and the one-launch ``FusedAdam`` / ``FusedAdamW``."""
from .combined_optimizer import CombinedOptimizer
from .fused_adam import FusedAdam, FusedAdamW, grad_global_norm
from .muon import Muon

__all__ = ["CombinedOptimizer", "Muon", "FusedAdam", "FusedAdamW", "grad_global_norm"]
