"""Noise schedulers.

Parity: ``physicsnemo/diffusion/noise_schedulers`` — the ``NoiseScheduler`` protocol
(``base.py:29-259``), ``LinearGaussianNoiseScheduler`` (``linear_gaussian.py:31-985``:
``x_t = alpha(t) x_0 + sigma(t) eps``; drift ``alpha'/alpha · x``; squared diffusion
``2 sigma' sigma − 2 (alpha'/alpha) sigma²``; conversions x0 ↔ score ↔ epsilon; ODE / SDE
denoisers), and the concrete EDM (``edm.py:26-266``), EDM log-uniform, VP, VE, iDDPM and
Student-t EDM schedules.
"""
from __future__ import annotations

import math
from abc import ABC, abstractmethod
from typing import Any, Literal, Protocol, Tuple, runtime_checkable

import torch
from torch import Tensor


@runtime_checkable
class NoiseScheduler(Protocol):
    def sample_time(self, N: int, *, device=None, dtype=None) -> Tensor: ...
    def add_noise(self, x0: Tensor, time: Tensor) -> Tensor: ...
    def timesteps(self, num_steps: int, *, device=None, dtype=None) -> Tensor: ...
    def init_latents(self, spatial_shape: Tuple[int, ...], tN: Tensor, *, device=None, dtype=None) -> Tensor: ...
    def get_denoiser(self, **kwargs: Any): ...
    def loss_weight(self, t: Tensor) -> Tensor: ...


def _bc(t: Tensor, x: Tensor) -> Tensor:
    return t.reshape((-1,) + (1,) * (x.ndim - 1))


class LinearGaussianNoiseScheduler(ABC):
    """Base of schedules with a linear-Gaussian perturbation kernel."""

    @abstractmethod
    def sigma(self, t: Tensor) -> Tensor: ...
    @abstractmethod
    def sigma_inv(self, sigma: Tensor) -> Tensor: ...
    @abstractmethod
    def sigma_dot(self, t: Tensor) -> Tensor: ...
    @abstractmethod
    def alpha(self, t: Tensor) -> Tensor: ...
    @abstractmethod
    def alpha_dot(self, t: Tensor) -> Tensor: ...
    @abstractmethod
    def timesteps(self, num_steps: int, *, device=None, dtype=None) -> Tensor: ...
    @abstractmethod
    def sample_time(self, N: int, *, device=None, dtype=None) -> Tensor: ...
    @abstractmethod
    def loss_weight(self, t: Tensor) -> Tensor: ...

    # ---- SDE coefficients
    def drift(self, x: Tensor, t: Tensor) -> Tensor:
        tb = _bc(t, x)
        return (self.alpha_dot(tb) / self.alpha(tb)) * x

    def diffusion(self, x: Tensor, t: Tensor) -> Tensor:
        tb = _bc(t, x)
        s, sd, a, ad = self.sigma(tb), self.sigma_dot(tb), self.alpha(tb), self.alpha_dot(tb)
        return 2 * sd * s - 2 * (ad / a) * s ** 2

    # ---- conversions between parameterisations
    def x0_to_score(self, x0: Tensor, x_t: Tensor, t: Tensor) -> Tensor:
        tb = _bc(t, x_t)
        return (self.alpha(tb) * x0 - x_t) / self.sigma(tb) ** 2

    def score_to_x0(self, score: Tensor, x_t: Tensor, t: Tensor) -> Tensor:
        tb = _bc(t, x_t)
        return (x_t + self.sigma(tb) ** 2 * score) / self.alpha(tb)

    def epsilon_to_score(self, epsilon: Tensor, t: Tensor) -> Tensor:
        return -epsilon / self.sigma(_bc(t, epsilon))

    def score_to_epsilon(self, score: Tensor, t: Tensor) -> Tensor:
        return -self.sigma(_bc(t, score)) * score

    def epsilon_to_x0(self, epsilon: Tensor, x_t: Tensor, t: Tensor) -> Tensor:
        tb = _bc(t, x_t)
        return (x_t - self.sigma(tb) * epsilon) / self.alpha(tb)

    def x0_to_epsilon(self, x0: Tensor, x_t: Tensor, t: Tensor) -> Tensor:
        tb = _bc(t, x_t)
        return (x_t - self.alpha(tb) * x0) / self.sigma(tb)

    # ---- sampling side
    def get_denoiser(self, *, score_predictor=None, x0_predictor=None, epsilon_predictor=None,
                     denoising_type: Literal["ode", "sde"] = "ode", **kwargs: Any):
        if sum(p is not None for p in (score_predictor, x0_predictor, epsilon_predictor)) != 1:
            raise ValueError("Exactly one of 'score_predictor', 'x0_predictor', or 'epsilon_predictor' must be provided.")
        if x0_predictor is not None:
            score_fn = lambda x, t: self.x0_to_score(x0_predictor(x, t), x, t)  # noqa: E731
        elif epsilon_predictor is not None:
            score_fn = lambda x, t: self.epsilon_to_score(epsilon_predictor(x, t), t)  # noqa: E731
        else:
            score_fn = score_predictor
        if denoising_type not in ("ode", "sde"):
            raise ValueError(f"denoising_type must be 'ode' or 'sde', got '{denoising_type}'")
        factor = 0.5 if denoising_type == "ode" else 1.0

        def denoiser(x: Tensor, t: Tensor) -> Tensor:
            return self.drift(x, t) - factor * self.diffusion(x, t) * score_fn(x, t)

        return denoiser

    def add_noise(self, x0: Tensor, time: Tensor) -> Tensor:
        tb = _bc(time, x0)
        return self.alpha(tb) * x0 + self.sigma(tb) * torch.randn_like(x0)

    def init_latents(self, spatial_shape: Tuple[int, ...], tN: Tensor, *, device=None, dtype=None) -> Tensor:
        noise = torch.randn(tN.shape[0], *spatial_shape, device=device, dtype=dtype)
        return self.sigma(tN.reshape((-1,) + (1,) * len(spatial_shape))) * noise


class EDMNoiseScheduler(LinearGaussianNoiseScheduler):
    """EDM: ``sigma(t) = t``, ``alpha = 1``; Karras rho-schedule; log-normal training times."""

    def __init__(self, sigma_min: float = 0.002, sigma_max: float = 80.0, rho: float = 7.0, sigma_data=0.5,
                 P_mean: float = -1.2, P_std: float = 1.2):
        self.sigma_min, self.sigma_max, self.rho = sigma_min, sigma_max, rho
        self.sigma_data = sigma_data if isinstance(sigma_data, Tensor) else torch.as_tensor(sigma_data, dtype=torch.float32)
        self._per_channel = self.sigma_data.ndim > 0
        self.P_mean, self.P_std = P_mean, P_std

    def sigma(self, t): return t
    def sigma_inv(self, sigma): return sigma
    def sigma_dot(self, t): return torch.ones_like(t)
    def alpha(self, t): return torch.ones_like(t)
    def alpha_dot(self, t): return torch.zeros_like(t)

    def timesteps(self, num_steps, *, device=None, dtype=None):
        i = torch.arange(num_steps, dtype=dtype, device=device)
        hi, lo = self.sigma_max ** (1 / self.rho), self.sigma_min ** (1 / self.rho)
        t = (hi + i / (num_steps - 1) * (lo - hi)) ** self.rho
        return torch.cat([t, torch.zeros(1, dtype=dtype, device=device)])

    def sample_time(self, N, *, device=None, dtype=None):
        return (torch.randn(N, device=device, dtype=dtype) * self.P_std + self.P_mean).exp()

    def loss_weight(self, t):
        sigma = self.sigma(t)
        sd = self.sigma_data.to(device=sigma.device, dtype=sigma.dtype)
        if self._per_channel:
            sigma, sd = sigma.unsqueeze(-1), sd.unsqueeze(0)
        return (sigma ** 2 + sd ** 2) / (sigma * sd) ** 2


class EDMLogUniformNoiseScheduler(EDMNoiseScheduler):
    """EDM schedule whose training noise levels are log-uniform in ``[sigma_min, sigma_max]``."""

    def __init__(self, sigma_min: float = 0.002, sigma_max: float = 80.0, rho: float = 7.0, sigma_data=0.5):
        super().__init__(sigma_min=sigma_min, sigma_max=sigma_max, rho=rho, sigma_data=sigma_data)

    def sample_time(self, N, *, device=None, dtype=None):
        u = torch.rand(N, device=device, dtype=dtype)
        lo, hi = math.log(self.sigma_min), math.log(self.sigma_max)
        return (lo + u * (hi - lo)).exp()


class VPNoiseScheduler(LinearGaussianNoiseScheduler):
    """Variance preserving SDE: ``alpha = exp(-½(½ β_d t² + β_min t))``, ``sigma = sqrt(1 − alpha²)``."""

    def __init__(self, beta_min: float = 0.1, beta_d: float = 19.1, epsilon_s: float = 1e-3, t_max: float = 1.0):
        self.beta_min, self.beta_d, self.epsilon_s, self.t_max = beta_min, beta_d, epsilon_s, t_max

    def alpha(self, t): return torch.exp(-0.5 * (0.5 * self.beta_d * t ** 2 + self.beta_min * t))
    def alpha_dot(self, t): return -0.5 * (self.beta_min + self.beta_d * t) * self.alpha(t)
    def sigma(self, t): return torch.sqrt(1 - self.alpha(t) ** 2)
    def sigma_dot(self, t): return -self.alpha(t) * self.alpha_dot(t) / self.sigma(t)

    def sigma_inv(self, sigma):
        log_term = torch.log(1 - sigma ** 2 + 1e-8)
        disc = self.beta_min ** 2 - 2 * self.beta_d * log_term
        return (-self.beta_min + torch.sqrt(disc.clamp(min=0))) / self.beta_d

    def timesteps(self, num_steps, *, device=None, dtype=None):
        i = torch.arange(num_steps, dtype=dtype, device=device)
        t = self.t_max + i / (num_steps - 1) * (self.epsilon_s - self.t_max)
        return torch.cat([t, torch.zeros(1, dtype=dtype, device=device)])

    def sample_time(self, N, *, device=None, dtype=None):
        return self.epsilon_s + torch.rand(N, device=device, dtype=dtype) * (self.t_max - self.epsilon_s)

    def loss_weight(self, t): return (self.alpha(t) / self.sigma(t)) ** 2


class VENoiseScheduler(LinearGaussianNoiseScheduler):
    """Variance exploding SDE: ``sigma(t) = sqrt(t)``, ``alpha = 1``."""

    def __init__(self, sigma_min: float = 0.02, sigma_max: float = 100.0):
        self.sigma_min, self.sigma_max = sigma_min, sigma_max

    def sigma(self, t): return t.sqrt()
    def sigma_inv(self, sigma): return sigma ** 2
    def sigma_dot(self, t): return 0.5 / t.sqrt()
    def alpha(self, t): return torch.ones_like(t)
    def alpha_dot(self, t): return torch.zeros_like(t)

    def timesteps(self, num_steps, *, device=None, dtype=None):
        i = torch.arange(num_steps, dtype=dtype, device=device)
        ratio = self.sigma_min ** 2 / self.sigma_max ** 2
        t = (self.sigma_max ** 2) * (ratio ** (i / (num_steps - 1)))
        return torch.cat([t, torch.zeros(1, dtype=dtype, device=device)])

    def sample_time(self, N, *, device=None, dtype=None):
        u = torch.rand(N, device=device, dtype=dtype)
        return self.sigma_inv(self.sigma_min * torch.exp(u * math.log(self.sigma_max / self.sigma_min)))

    def loss_weight(self, t): return 1 / self.sigma(t) ** 2


class IDDPMNoiseScheduler(LinearGaussianNoiseScheduler):
    """Improved-DDPM cosine schedule expressed as noise levels ``u_j`` (``sigma(t) = t``)."""

    def __init__(self, sigma_min: float = 0.002, sigma_max: float = 81.0, C_1: float = 0.001, C_2: float = 0.008,
                 M: int = 1000):
        self.sigma_min, self.sigma_max, self.C_1, self.C_2, self.M = sigma_min, sigma_max, C_1, C_2, M
        self._u = self._compute_u_schedule()

    def _compute_u_schedule(self) -> Tensor:
        u = torch.zeros(self.M + 1)
        for j in range(self.M, 0, -1):
            a_j = math.sin(0.5 * math.pi * j / self.M / (self.C_2 + 1)) ** 2
            a_jm1 = math.sin(0.5 * math.pi * (j - 1) / self.M / (self.C_2 + 1)) ** 2
            u[j - 1] = ((u[j] ** 2 + 1) / max(a_jm1 / a_j, self.C_1) - 1).sqrt()
        return u

    def sigma(self, t): return t
    def sigma_inv(self, sigma): return sigma
    def sigma_dot(self, t): return torch.ones_like(t)
    def alpha(self, t): return torch.ones_like(t)
    def alpha_dot(self, t): return torch.zeros_like(t)

    def _levels(self, device, dtype):
        u = self._u.to(device=device, dtype=dtype)
        return u[torch.logical_and(u >= self.sigma_min, u <= self.sigma_max)]

    def timesteps(self, num_steps, *, device=None, dtype=None):
        uf = self._levels(device, dtype)
        i = torch.arange(num_steps, dtype=dtype, device=device)
        idx = ((len(uf) - 1) / (num_steps - 1) * i).round().to(torch.int64)
        return torch.cat([uf[idx], torch.zeros(1, dtype=dtype, device=device)])

    def sample_time(self, N, *, device=None, dtype=None):
        uf = self._levels(device, dtype)
        return uf[torch.randint(0, len(uf), (N,), device=device)]

    def loss_weight(self, t): return 1 / self.sigma(t) ** 2


class StudentTEDMNoiseScheduler(EDMNoiseScheduler):
    """EDM schedule with heavy-tailed (Student-t, ``nu`` degrees of freedom) noise for extremes."""

    def __init__(self, sigma_min: float = 0.002, sigma_max: float = 80.0, rho: float = 7.0, sigma_data=0.5,
                 P_mean: float = -1.2, P_std: float = 1.2, nu: float = 10.0):
        super().__init__(sigma_min, sigma_max, rho, sigma_data, P_mean, P_std)
        if nu <= 2:
            raise ValueError(f"nu must be > 2 for a finite variance, got {nu}")
        self.nu = nu

    def _student_t(self, shape, device, dtype) -> Tensor:
        normal = torch.randn(shape, device=device, dtype=dtype)
        chi2 = torch.distributions.Chi2(torch.tensor(self.nu, device=device)).sample((shape[0],)).to(dtype)
        kappa = chi2 / self.nu
        return normal / torch.sqrt(kappa).reshape((-1,) + (1,) * (len(shape) - 1))

    def add_noise(self, x0, time):
        return x0 + self.sigma(_bc(time, x0)) * self._student_t(tuple(x0.shape), x0.device, x0.dtype)

    def init_latents(self, spatial_shape, tN, *, device=None, dtype=None):
        noise = self._student_t((tN.shape[0], *spatial_shape), device, dtype or torch.float32)
        return self.sigma(tN.reshape((-1,) + (1,) * len(spatial_shape))) * noise
