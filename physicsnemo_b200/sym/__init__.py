"""Symbolic PDE residuals on tensors: SymPy equations, a dependency graph, numerical gradient nodes."""
from .eq.gradients import GradientCalculator, compute_connectivity_tensor
from .eq.pde import PDE
from .eq.phy_informer import PhysicsInformer

__all__ = ["GradientCalculator", "PDE", "PhysicsInformer", "compute_connectivity_tensor"]
