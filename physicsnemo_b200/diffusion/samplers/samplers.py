"""Generic sampling loop (parity: ``physicsnemo/diffusion/samplers/samplers.py:74-427``)."""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Union

import torch
from torch import Tensor

from .solvers import SOLVERS, Solver


def sample(denoiser, xN: Tensor, noise_scheduler, num_steps: int, solver: Union[str, Solver] = "heun",
           time_steps: Optional[Tensor] = None, solver_options: Optional[Dict[str, Any]] = None,
           time_eval: Optional[List[int]] = None):
    """Integrate ``denoiser`` from the latent ``xN`` down to ``t = 0``.

    ``solver`` is a name (``"euler"``, ``"heun"``, ``"edm_stochastic_euler"``, ``"edm_stochastic_heun"``) or a
    ``Solver`` instance; ``time_steps`` overrides the scheduler's discretisation; ``time_eval`` lists
    step indices whose states are returned (as a list) instead of the final sample.
    """
    solver_options = solver_options or {}
    if isinstance(solver, str):
        if solver not in SOLVERS:
            raise ValueError(f"Unknown solver '{solver}'. Available solvers: " + ", ".join(f'"{k}"' for k in SOLVERS))
        solver_ = SOLVERS[solver](denoiser, **solver_options)
    else:
        if solver_options:
            raise ValueError("solver_options must be None when solver is a Solver instance.")
        solver_ = solver
    if time_steps is not None:
        t_steps = time_steps.to(device=xN.device, dtype=xN.dtype)
    else:
        t_steps = noise_scheduler.timesteps(num_steps, device=xN.device, dtype=xN.dtype)
    grad = torch.is_grad_enabled()
    n_steps = len(t_steps) - 1
    if time_eval is not None:
        bad = [i for i in time_eval if i < 0 or i >= n_steps]
        if bad:
            raise ValueError(f"time_eval contains out-of-range indices {bad}; valid indices are in range(0, {n_steps}).")
    samples: List[Tensor] = []
    x = xN
    for i in range(n_steps):
        B = x.shape[0]
        x = solver_.step(x, t_steps[i].expand(B), t_steps[i + 1].expand(B))
        if not grad:
            x = x.detach()
        if time_eval is not None and i in time_eval:
            samples.append(x.clone())
    return samples if time_eval is not None else x
