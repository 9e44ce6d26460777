"""PDE residuals of a symbolic system evaluated on tensors with a chosen numerical derivative.

Parity: ``physicsnemo/sym/eq/phy_informer.py`` (``PhysicsInformer``: ``required_inputs``,
``forward``; methods ``finite_difference``, ``spectral``, ``least_squares``, ``autodiff``,
``meshless_finite_difference``; up to second-order derivatives in ``x, y, z``; derivatives along
any other symbol, e.g. time, are inputs the caller supplies).

Construction compiles the equations once (SymPy → tensor callables with shared sub-expressions),
builds one gradient node per differentiated variable and order, and schedules everything into a
``Graph``; ``forward`` is a walk over that fixed module list, so a training loop can capture it in
a CUDA graph together with the model step.
"""
from __future__ import annotations

import logging
import math
from itertools import combinations
from typing import Dict, List, Optional, Union

import torch

from ..computation import Computation
from ..constants import split_derivative
from ..graph import Graph
from .gradients import GradientCalculator, compute_connectivity_tensor
from .pde import PDE

logger = logging.getLogger(__name__)

_SPACE = ("x", "y", "z")
_METHODS = ("finite_difference", "spectral", "least_squares", "autodiff", "meshless_finite_difference")


class PhysicsInformer:
    def __init__(self, required_outputs: List[str], equations: PDE, grad_method: str,
                 fd_dx: Union[float, List[float]] = 0.001, bounds: List[float] | None = None,
                 compute_connectivity: bool = True, detach_names: List[str] | None = None,
                 device: Optional[str] = None):
        self.required_outputs = list(required_outputs)
        self.equations = equations
        self.dim = equations.dim
        self.grad_method = grad_method
        self.fd_dx = fd_dx
        self.bounds = list(bounds) if bounds is not None else [2 * math.pi] * 3
        self.compute_connectivity = compute_connectivity
        self.device = device if device is not None else torch.device("cpu")
        self.grad_calc = GradientCalculator(device=self.device)
        self.computations = self.equations.make_computations(detach_names=detach_names)
        available = [c.outputs[0] for c in self.computations]
        for name in self.required_outputs:
            if name not in available:
                raise ValueError(f"{name} not in equation outputs. Choose from {available}")
        self.require_mixed_derivs = False
        self._first, self._second, self._supplied = self._classify_derivatives()
        self.graph = self._create_graph()

    # ---- analysis of the requested equations ----------------------------------------------------
    def _selected(self):
        return [c for c in self.computations if c.outputs[0] in self.required_outputs]

    def _classify_derivatives(self):
        """Variables needing first / second spatial derivatives, and derivative keys the caller must supply."""
        first, second, supplied = set(), set(), set()
        for comp in self._selected():
            for key in comp.derivatives:
                var, wrt = split_derivative(key)
                if len(wrt) > 2:
                    raise ValueError("Only up to second-order PDEs are supported")
                foreign = [w for w in wrt if w not in _SPACE]
                if foreign:
                    logger.warning("Derivative w.r.t %s detected — must be supplied manually.", foreign[0])
                    supplied.add(key)
                    continue
                if len(wrt) == 2 and wrt[0] != wrt[1]:
                    self.require_mixed_derivs = True
                (first if len(wrt) == 1 else second).add(var)
        return first, second, supplied

    def _extract_derivatives(self):
        return set(self._first), set(self._second), set(self._supplied)

    @property
    def required_inputs(self) -> List[str]:
        names = set(self._first) | set(self._second) | set(self._supplied)
        for comp in self._selected():
            names.update(comp.inputs)
        inputs = list(names)
        if self.grad_method == "meshless_finite_difference":
            inputs = self._expand_for_meshless_fd(inputs)
        elif self.grad_method == "autodiff":
            inputs.append("coordinates")
        elif self.grad_method == "least_squares":
            inputs.append("coordinates")
            inputs += ["nodes", "edges"] if self.compute_connectivity else ["connectivity_tensor"]
        return inputs

    def _expand_for_meshless_fd(self, names: List[str]) -> List[str]:
        out = list(names)
        axes = _SPACE[:self.dim]
        for name in names:
            for a in axes:
                out += [f"{name}>>{a}::1", f"{name}>>{a}::-1"]
        return out

    # ---- graph construction ---------------------------------------------------------------------
    def _derivative_keys(self, var: str, dim: int, order: int, return_mixed_derivs: bool = False) -> List[str]:
        keys = [var + ("__" + a) * order for a in _SPACE[:dim]]
        if return_mixed_derivs and order == 2:
            for i, j in combinations(range(dim), 2):
                keys += [f"{var}__{_SPACE[i]}__{_SPACE[j]}", f"{var}__{_SPACE[j]}__{_SPACE[i]}"]
        return keys

    def _gradient_kwargs(self) -> dict:
        if self.grad_method in ("finite_difference", "meshless_finite_difference"):
            return {"dx": self.fd_dx}
        if self.grad_method == "spectral":
            return {"ell": self.bounds}
        return {}

    def _create_diff_node(self, var: str, dim: int, order: int) -> Computation | None:
        if self.grad_method not in _METHODS:
            return None
        mixed = self.require_mixed_derivs and order == 2
        module = self.grad_calc.get_gradient_module(self.grad_method, var, dim=dim, order=order,
                                                    return_mixed_derivs=mixed, **self._gradient_kwargs())
        return Computation([var], self._derivative_keys(var, dim, order, self.require_mixed_derivs), module,
                           name=f"{self.grad_method} d^{order} {var}")

    def _create_diff_nodes(self, variables, dim: int, order: int) -> List[Computation]:
        nodes = [self._create_diff_node(v, dim, order) for v in sorted(variables)]
        return [n for n in nodes if n is not None]

    def _create_graph(self) -> Graph:
        diff_nodes = self._create_diff_nodes(self._first, self.dim, 1) + self._create_diff_nodes(self._second, self.dim, 2)
        return Graph(self.computations, list(self.required_inputs), list(self.required_outputs),
                     diff_nodes=diff_nodes).to(self.device)

    # ---- evaluation -----------------------------------------------------------------------------
    def forward(self, inputs: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        inputs = dict(inputs)
        if self.grad_method == "least_squares" and self.compute_connectivity:
            inputs["connectivity_tensor"] = compute_connectivity_tensor(inputs["nodes"], inputs["edges"])
        return self.graph(inputs)

    __call__ = forward
