"""ODE / SDE solvers stepping a denoiser from ``t_cur`` to ``t_next``.

Parity: ``physicsnemo/diffusion/samplers`` — ``Solver`` protocol (``base.py``), ``EulerSolver``
(``euler.py``), ``HeunSolver`` (``heun.py:28-137``; second-order with parameter ``alpha``, Euler on
the final step to ``t = 0``), ``EDMStochasticEulerSolver`` / ``EDMStochasticHeunSolver`` (churn:
temporarily raise the noise level by ``gamma`` inside ``[S_min, S_max]``, then step).
"""
from __future__ import annotations

import math
from typing import Callable, Optional, Protocol, runtime_checkable

import torch
from torch import Tensor


@runtime_checkable
class Solver(Protocol):
    def step(self, x: Tensor, t_cur: Tensor, t_next: Tensor) -> Tensor: ...


def _bc(t, x):
    return t.contiguous().reshape((-1,) + (1,) * (x.ndim - 1))


class EulerSolver:
    def __init__(self, denoiser) -> None:
        self.denoiser = denoiser

    def step(self, x, t_cur, t_next):
        return x + (_bc(t_next, x) - _bc(t_cur, x)) * self.denoiser(x, t_cur.contiguous())


class HeunSolver:
    def __init__(self, denoiser, alpha: float = 1.0) -> None:
        if not 0 < alpha <= 1:
            raise ValueError(f"alpha must be in (0, 1], got {alpha}")
        self.denoiser, self.alpha = denoiser, alpha

    def step(self, x, t_cur, t_next):
        t_cur, t_next = t_cur.contiguous(), t_next.contiguous()
        tc, tn = _bc(t_cur, x), _bc(t_next, x)
        h = tn - tc
        d_cur = self.denoiser(x, t_cur)
        t_prime = (tc + self.alpha * h).reshape(x.shape[0])
        x_prime = x + self.alpha * h * d_cur
        mask = (tn != 0).to(x.dtype)
        d_prime = self.denoiser(x_prime, torch.where(t_prime == 0, t_cur, t_prime))
        w_cur, w_prime = 1 - 1 / (2 * self.alpha), 1 / (2 * self.alpha)
        x_heun = x + h * (w_cur * d_cur + w_prime * d_prime)
        return mask * x_heun + (1 - mask) * (x + h * d_cur)


class _EDMStochasticBase:
    def __init__(self, denoiser, S_churn: float = 0, S_min: float = 0, S_max: float = float("inf"),
                 S_noise: float = 1, num_steps: int = 18, sigma_fn: Optional[Callable] = None,
                 sigma_inv_fn: Optional[Callable] = None, diffusion_fn: Optional[Callable] = None) -> None:
        self.denoiser = denoiser
        self.S_churn, self.S_min, self.S_max, self.S_noise, self.num_steps = S_churn, S_min, S_max, S_noise, num_steps
        if (sigma_fn is None) != (sigma_inv_fn is None):
            raise ValueError("sigma_fn and sigma_inv_fn must both be provided or both None.")
        self.sigma_fn = sigma_fn or (lambda t: t)
        self.sigma_inv_fn = sigma_inv_fn or (lambda s: s)
        self.diffusion_fn = diffusion_fn or (lambda x, t: 2 * t.reshape(-1, *([1] * (x.ndim - 1))))

    def _churn(self, x, t_cur):
        tc = _bc(t_cur, x)
        gamma_base = min(self.S_churn / self.num_steps, math.sqrt(2) - 1)
        sigma_cur = self.sigma_fn(tc)
        mask = (sigma_cur >= self.S_min) & (sigma_cur <= self.S_max)
        gamma = torch.where(mask, gamma_base, 0.0)
        t_hat = self.sigma_inv_fn(sigma_cur + gamma * sigma_cur)
        g_sq = self.diffusion_fn(x, t_cur)
        safe = torch.where(tc == 0, torch.ones_like(tc), tc)
        scale = (t_hat ** 2 - tc ** 2).clamp(min=0).sqrt() * self.S_noise * (g_sq / (2 * safe)).sqrt()
        scale = torch.where(tc == 0, torch.zeros_like(scale), scale)
        return x + scale * torch.randn_like(x), t_hat


class EDMStochasticEulerSolver(_EDMStochasticBase):
    def step(self, x, t_cur, t_next):
        t_cur, t_next = t_cur.contiguous(), t_next.contiguous()
        x_hat, t_hat = self._churn(x, t_cur)
        d_cur = self.denoiser(x_hat, t_hat.reshape(x.shape[0]))
        return x_hat + (_bc(t_next, x) - t_hat) * d_cur


class EDMStochasticHeunSolver(_EDMStochasticBase):
    def __init__(self, denoiser, alpha: float = 1.0, **kwargs) -> None:
        super().__init__(denoiser, **kwargs)
        if not 0 < alpha <= 1:
            raise ValueError(f"alpha must be in (0, 1], got {alpha}")
        self.alpha = alpha

    def step(self, x, t_cur, t_next):
        t_cur, t_next = t_cur.contiguous(), t_next.contiguous()
        x_hat, t_hat = self._churn(x, t_cur)
        tn = _bc(t_next, x)
        h = tn - t_hat
        t_hat_flat = t_hat.reshape(x.shape[0])
        d_cur = self.denoiser(x_hat, t_hat_flat)
        t_prime = (t_hat + self.alpha * h).reshape(x.shape[0])
        x_prime = x_hat + self.alpha * h * d_cur
        mask = (tn != 0).to(x.dtype)
        d_prime = self.denoiser(x_prime, torch.where(t_prime == 0, t_hat_flat, t_prime))
        w_cur, w_prime = 1 - 1 / (2 * self.alpha), 1 / (2 * self.alpha)
        x_heun = x_hat + h * (w_cur * d_cur + w_prime * d_prime)
        return mask * x_heun + (1 - mask) * (x_hat + h * d_cur)


SOLVERS = {"euler": EulerSolver, "heun": HeunSolver, "edm_stochastic_euler": EDMStochasticEulerSolver,
           "edm_stochastic_heun": EDMStochasticHeunSolver}
