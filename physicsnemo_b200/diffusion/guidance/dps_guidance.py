"""Diffusion posterior sampling (DPS) guidance.

Parity: ``physicsnemo/diffusion/guidance/dps_guidance.py`` — ``DPSScorePredictor`` wraps an ``x0`` predictor and adds
guidance terms to the converted score; a guidance is any callable ``(x, t, x_0) -> tensor like x`` returning the gradient
of a log-likelihood with respect to ``x`` *through* the predictor.  The two stock guidances use

    log p(y | x_t) ≈ − ρ(t) · ‖A(x̂₀(x_t)) − y‖ₚᵖ,    ρ(t) = 1 / (2 (σ_y² + γ σ(t)² / α(t)²)),

with ``A`` an arbitrary observation operator (``ModelConsistencyDPSGuidance``) or a mask on the state itself
(``DataConsistencyDPSGuidance``).
"""
from __future__ import annotations

from typing import Callable, Protocol, Sequence, runtime_checkable

import torch
from torch import Tensor


def _as_broadcastable(x, y: Tensor) -> Tensor:
    x = torch.as_tensor(x)
    try:
        ok = torch.broadcast_shapes(x.shape, y.shape) == y.shape
    except RuntimeError:
        ok = False
    if not ok:
        raise ValueError(f"First tensor of shape {tuple(x.shape)} must broadcast to the second tensor of shape {tuple(y.shape)}.")
    return x


def _needs_autograd(name: str) -> None:
    if not torch.compiler.is_compiling() and torch.is_inference_mode_enabled():
        raise RuntimeError(f"{name} requires autograd but torch inference mode is enabled. Wrap the calling code with "
                           "'with torch.inference_mode(False):' or 'with torch.no_grad():' instead.")


@runtime_checkable
class DPSGuidance(Protocol):
    def __call__(self, x: Tensor, t: Tensor, x_0: Tensor) -> Tensor: ...


class DPSScorePredictor:
    """Score predictor ``score(x̂₀(x, t), x, t) + Σ guidance(x, t, x̂₀)``; ``x`` is re-attached to autograd on every call."""

    def __init__(self, x0_predictor: Callable[[Tensor, Tensor], Tensor], x0_to_score_fn: Callable[[Tensor, Tensor, Tensor], Tensor],
                 guidances: DPSGuidance | Sequence[DPSGuidance]) -> None:
        self.x0_predictor, self.x0_to_score_fn = x0_predictor, x0_to_score_fn
        self.guidances = list(guidances) if isinstance(guidances, Sequence) and not isinstance(guidances, str) else [guidances]

    def __call__(self, x: Tensor, t: Tensor) -> Tensor:
        _needs_autograd("DPSScorePredictor")
        x = x.detach().requires_grad_(True)
        with torch.enable_grad():
            x_0 = self.x0_predictor(x, t)
            total = torch.zeros_like(x)
            for guidance in self.guidances:
                total = total + guidance(x, t, x_0)
        return self.x0_to_score_fn(x_0, x, t) + total


class _ConsistencyGuidance:
    def __init__(self, y, std_y, norm, gamma, sigma_fn, alpha_fn, retain_graph, create_graph):
        self.y = y
        self.std_y, self.gamma = _as_broadcastable(std_y, y), _as_broadcastable(gamma, y)
        if sigma_fn is None and bool((self.gamma > 0).any()):
            raise ValueError("sigma_fn must be provided when gamma > 0")
        self._loss_fn = (lambda a, b, p=norm: (a - b).abs().pow(p)) if isinstance(norm, int) else norm
        self.sigma_fn = sigma_fn if sigma_fn is not None else torch.zeros_like
        self.alpha_fn = alpha_fn if alpha_fn is not None else torch.ones_like
        self.retain_graph, self.create_graph = retain_graph, create_graph

    def _residual(self, x_0: Tensor, y: Tensor) -> Tensor:
        raise NotImplementedError

    def __call__(self, x: Tensor, t: Tensor, x_0: Tensor) -> Tensor:
        _needs_autograd(type(self).__name__)
        y, std_y, gamma = (v.to(dtype=x.dtype, device=x.device) for v in (self.y, self.std_y, self.gamma))
        with torch.enable_grad():
            loss = self._residual(x_0, y)
            t_bc = t.reshape((-1,) + (1,) * (loss.ndim - 1))
            rho = 1.0 / (2.0 * (std_y ** 2 + gamma * self.sigma_fn(t_bc) ** 2 / self.alpha_fn(t_bc) ** 2))
            grad = torch.autograd.grad((rho * loss).sum(), x, retain_graph=self.retain_graph, create_graph=self.create_graph)[0]
        return -grad


class ModelConsistencyDPSGuidance(_ConsistencyGuidance):
    """Guidance towards observations ``y ≈ A(x₀)`` of a differentiable observation operator ``A``."""

    def __init__(self, observation_operator: Callable[[Tensor], Tensor], y: Tensor, std_y, norm=2, gamma=0.0, sigma_fn=None, alpha_fn=None,
                 retain_graph: bool = False, create_graph: bool = False) -> None:
        super().__init__(y, std_y, norm, gamma, sigma_fn, alpha_fn, retain_graph, create_graph)
        self.observation_operator = observation_operator

    def _residual(self, x_0, y):
        return self._loss_fn(self.observation_operator(x_0), y)


class DataConsistencyDPSGuidance(_ConsistencyGuidance):
    """Guidance towards point observations of the state itself: ``y ≈ x₀`` where ``mask`` is true."""

    def __init__(self, mask: Tensor, y: Tensor, std_y, norm=2, gamma=0.0, sigma_fn=None, alpha_fn=None, retain_graph: bool = False,
                 create_graph: bool = False) -> None:
        super().__init__(y, std_y, norm, gamma, sigma_fn, alpha_fn, retain_graph, create_graph)
        self.mask = mask.float()

    def _residual(self, x_0, y):
        return self.mask.to(dtype=x_0.dtype, device=x_0.device) * self._loss_fn(x_0, y)
