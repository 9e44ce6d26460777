from .legacy_samplers import deterministic_sampler, stochastic_sampler
from .samplers import sample
from .solvers import (SOLVERS, EDMStochasticEulerSolver, EDMStochasticHeunSolver, EulerSolver, HeunSolver, Solver)

__all__ = ["sample", "Solver", "EulerSolver", "HeunSolver", "EDMStochasticEulerSolver", "EDMStochasticHeunSolver",
           "SOLVERS", "deterministic_sampler", "stochastic_sampler"]
