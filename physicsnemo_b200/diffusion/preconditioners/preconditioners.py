"""Affine preconditioners: ``D(x, t) = c_skip x + c_out F(c_in x, c_noise, condition)``.

Parity: ``physicsnemo/diffusion/preconditioners/preconditioners.py`` —
``BaseAffinePreconditioner`` (``:62-531``) and ``VP`` (``:534``), ``VE`` (``:684``), ``iDDPM``
(``:791``), ``EDM`` (``:933-1106``; per-channel ``sigma_data`` buffer).  The wrapped network lives
under ``model`` so state-dict keys gain the ``model.`` prefix.  Coefficients stay plain
(replicated) tensors when ``x`` is a ``ShardTensor``.
"""
from __future__ import annotations

import math
from abc import ABC, abstractmethod
from typing import Any, Sequence, Tuple

import torch

from ...core.meta import ModelMetaData
from ...core.module import Module


class BaseAffinePreconditioner(Module, ABC):
    def __init__(self, model: Module, meta: ModelMetaData | None = None) -> None:
        super().__init__()
        self.meta = meta
        self.model = model

    @abstractmethod
    def compute_coefficients(self, t: torch.Tensor, /) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
        """Return ``(c_in, c_noise, c_out, c_skip)`` for noise level(s) ``t`` (broadcastable to ``x``)."""

    def sigma(self, t: torch.Tensor) -> torch.Tensor:
        return t

    def _validate_input(self, x: torch.Tensor) -> None:
        pass

    def forward(self, x: torch.Tensor, t: torch.Tensor, condition=None, **model_kwargs: Any) -> torch.Tensor:
        if not torch.compiler.is_compiling():
            B = x.shape[0]
            if tuple(t.shape) != (B,):
                raise ValueError(f"Expected t to have shape ({B},) matching batch size of x, but got {t.shape}.")
            if isinstance(condition, torch.Tensor) and condition.shape[0] != B:
                raise ValueError(f"Condition tensor has batch size {condition.shape[0]} but expected {B} to match x.")
            self._validate_input(x)
        sigma_t = self.sigma(t).reshape((-1,) + (1,) * (x.ndim - 1))
        c_in, c_noise, c_out, c_skip = self.compute_coefficients(sigma_t)
        if condition is not None:
            F_x = self.model(c_in * x, c_noise.flatten(), condition=condition, **model_kwargs)
        else:
            F_x = self.model(c_in * x, c_noise.flatten(), **model_kwargs)
        return c_skip * x + c_out * F_x


class VPPreconditioner(BaseAffinePreconditioner):
    def __init__(self, model: Module, beta_d: float = 19.9, beta_min: float = 0.1, M: int = 1000) -> None:
        super().__init__(model)
        self.register_buffer("beta_d", torch.tensor(beta_d))
        self.register_buffer("beta_min", torch.tensor(beta_min))
        self.register_buffer("M", torch.tensor(M))

    def sigma(self, t):
        return ((0.5 * self.beta_d * (t ** 2) + self.beta_min * t).exp() - 1).sqrt()

    def compute_coefficients(self, sigma):
        c_skip = torch.ones_like(sigma)
        c_out = -sigma
        c_in = 1 / (sigma ** 2 + 1).sqrt()
        t = ((self.beta_min ** 2 + 2 * self.beta_d * (1 + sigma ** 2).log()).sqrt() - self.beta_min) / self.beta_d
        return c_in, (self.M - 1) * t, c_out, c_skip


class VEPreconditioner(BaseAffinePreconditioner):
    def __init__(self, model: Module) -> None:
        super().__init__(model)

    def compute_coefficients(self, t):
        return torch.ones_like(t), (0.5 * t).log(), t, torch.ones_like(t)


class IDDPMPreconditioner(BaseAffinePreconditioner):
    def __init__(self, model: Module, C_1: float = 0.001, C_2: float = 0.008, M: int = 1000) -> None:
        super().__init__(model)
        self.register_buffer("C_1", torch.tensor(C_1))
        self.register_buffer("C_2", torch.tensor(C_2))
        self.register_buffer("M", torch.tensor(M))
        u = torch.zeros(M + 1)
        for j in range(M, 0, -1):
            a_j = math.sin(0.5 * math.pi * j / M / (C_2 + 1)) ** 2
            a_jm1 = math.sin(0.5 * math.pi * (j - 1) / M / (C_2 + 1)) ** 2
            u[j - 1] = ((u[j] ** 2 + 1) / max(a_jm1 / a_j, C_1) - 1).sqrt()
        self.register_buffer("u", u)

    def compute_coefficients(self, t):
        c_skip = torch.ones_like(t)
        c_out = -t
        c_in = 1 / (t ** 2 + 1).sqrt()
        idx = torch.cdist(t.reshape(1, -1, 1), self.u.reshape(1, -1, 1)).argmin(2).reshape(t.shape)
        return c_in, self.M - 1 - idx, c_out, c_skip


class EDMPreconditioner(BaseAffinePreconditioner):
    """EDM scalings; ``sigma_data`` may be a scalar or one value per channel."""

    def __init__(self, model: Module, sigma_data=0.5) -> None:
        super().__init__(model)
        if isinstance(sigma_data, torch.Tensor):
            sd = sigma_data.detach().to(dtype=torch.float32).reshape(-1)
        elif isinstance(sigma_data, Sequence) and not isinstance(sigma_data, str):
            sd = torch.as_tensor(list(sigma_data), dtype=torch.float32)
        else:
            sd = torch.as_tensor(float(sigma_data))
        if sd.ndim > 0 and sd.numel() == 1:
            sd = sd.squeeze()
        self.register_buffer("sigma_data", sd)
        self._sigma_data_channels = sd.numel() if sd.ndim > 0 else 0

    def _validate_input(self, x):
        C = self._sigma_data_channels
        if C > 0 and x.ndim >= 2 and x.shape[1] != C:
            raise ValueError(
                f"EDMPreconditioner has per-channel sigma_data with {C} channels, but input x has {x.shape[1]} "
                f"channels (shape {tuple(x.shape)}).")

    def _reshape_sigma_data(self, t):
        sd = self.sigma_data
        if self._sigma_data_channels > 0:
            sd = sd.view(1, -1, *([1] * (t.ndim - 2)))
        return sd

    def compute_coefficients(self, t):
        sd = self._reshape_sigma_data(t)
        c_skip = sd ** 2 / (t ** 2 + sd ** 2)
        c_out = t * sd / (t ** 2 + sd ** 2).sqrt()
        c_in = 1 / (sd ** 2 + t ** 2).sqrt()
        return c_in, t.log() / 4, c_out, c_skip
