"""Affine preconditioners: ``D(x, t) = c_skip x + c_out F(c_in x, c_noise, condition)``.

Parity: ``physicsnemo/diffusion/preconditioners/preconditioners.py`` —
``BaseAffinePreconditioner`` (``:62-531``) and ``VP`` (``:534``), ``VE`` (``:684``), ``iDDPM``
(``:791``), ``EDM`` (``:933-1106``; per-channel ``sigma_data`` buffer).  The wrapped network lives
under ``model`` so state-dict keys gain the ``model.`` prefix.

Sharded activations (reference ``:482-531``): the four coefficients are always computed on plain tensors — a noise
level that arrives as a replicated distributed tensor, or a buffer that FSDP turned into one, is unwrapped first.
They multiply a ``ShardTensor`` as plain tensors (its dispatch treats a plain operand as replicated); for a genuine
``DTensor`` activation they are wrapped as replicated tensors on the activation's mesh.
"""
from __future__ import annotations

import math
from abc import ABC, abstractmethod
from typing import Any, Sequence, Tuple

import torch

from ...core.meta import ModelMetaData
from ...core.module import Module

Coefficients = Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]


def _plain(value: torch.Tensor) -> torch.Tensor:
    """The ordinary tensor behind a (replicated) distributed tensor; other tensors pass through."""
    gather = getattr(value, "full_tensor", None)
    return gather() if callable(gather) else value


def _is_true_dtensor(x) -> bool:
    try:
        from torch.distributed.tensor import DTensor
    except Exception:  # pragma: no cover - torch without distributed tensors
        return False
    if not isinstance(x, DTensor):
        return False
    from ...parallel.shard_tensor import ShardTensor

    return not isinstance(x, ShardTensor)


def _replicated_like(value: torch.Tensor, activation) -> torch.Tensor:
    from torch.distributed.tensor import DTensor, Replicate

    mesh = activation.device_mesh
    return DTensor.from_local(value, mesh, [Replicate()] * mesh.ndim, run_check=False)


class BaseAffinePreconditioner(Module, ABC):
    """``forward(x, t, condition)`` with ``t`` of shape ``[B]``; subclasses supply the coefficients (and ``sigma(t)``)."""

    def __init__(self, model: Module, meta: ModelMetaData | None = None) -> None:
        super().__init__()
        self.meta = meta
        self.model = model

    @abstractmethod
    def compute_coefficients(self, t: torch.Tensor, /) -> Coefficients:
        """Return ``(c_in, c_noise, c_out, c_skip)`` for noise level(s) ``t`` (broadcastable to ``x``)."""

    def sigma(self, t: torch.Tensor) -> torch.Tensor:
        """Noise level of time ``t`` (identity unless the parametrisation has its own schedule)."""
        return t

    def _validate_input(self, x: torch.Tensor) -> None:
        """Hook for subclass-specific checks of ``x`` (skipped while ``torch.compile`` traces)."""

    def _check_call(self, x, t, condition) -> None:
        batch = x.shape[0]
        if t.ndim != 1 or t.shape[0] != batch:
            raise ValueError(f"one noise level per sample is required: x holds {batch} samples, t has shape {tuple(t.shape)}")
        if isinstance(condition, torch.Tensor):
            cond_batch = condition.shape[0]
        else:                                              # TensorDict-like containers expose ``batch_size``
            sizes = getattr(condition, "batch_size", None)
            cond_batch = sizes[0] if sizes else None
        if cond_batch is not None and cond_batch != batch:
            raise ValueError(f"the condition holds {cond_batch} samples but x holds {batch}")
        self._validate_input(x)

    def _coefficients_for(self, x, t) -> Coefficients:
        per_sample = (x.shape[0],) + (1,) * (x.ndim - 1)
        level = _plain(self.sigma(t).reshape(per_sample))
        coeffs = tuple(_plain(c) for c in self.compute_coefficients(level))
        if _is_true_dtensor(x):
            coeffs = tuple(_replicated_like(c, x) for c in coeffs)
        return coeffs

    def forward(self, x: torch.Tensor, t: torch.Tensor, condition=None, **model_kwargs: Any) -> torch.Tensor:
        if not torch.compiler.is_compiling():
            self._check_call(x, t, condition)
        c_in, c_noise, c_out, c_skip = self._coefficients_for(x, t)
        if condition is not None:
            model_kwargs = dict(model_kwargs, condition=condition)
        raw = self.model(c_in * x, c_noise.flatten(), **model_kwargs)
        return c_skip * x + c_out * raw


def _unit_variance_scale(sigma: torch.Tensor) -> torch.Tensor:
    """``1 / sqrt(1 + sigma²)``: the input scale of the variance-preserving family."""
    return torch.rsqrt(sigma.square() + 1)


class VPPreconditioner(BaseAffinePreconditioner):
    """Variance preserving: ``sigma(t) = sqrt(exp(½ β_d t² + β_min t) − 1)``; the network sees ``(M − 1) t(σ)``."""

    def __init__(self, model: Module, beta_d: float = 19.9, beta_min: float = 0.1, M: int = 1000) -> None:
        super().__init__(model)
        for name, value in (("beta_d", beta_d), ("beta_min", beta_min), ("M", M)):
            self.register_buffer(name, torch.tensor(value))

    def sigma(self, t):
        exponent = t * (self.beta_min + 0.5 * self.beta_d * t)
        return torch.sqrt(torch.expm1(exponent))

    def _time_of(self, sigma):
        """Inverse of ``sigma(t)``: the positive root of ½ β_d t² + β_min t = log(1 + σ²)."""
        discriminant = self.beta_min.square() + 2 * self.beta_d * torch.log1p(sigma.square())
        return (discriminant.sqrt() - self.beta_min) / self.beta_d

    def compute_coefficients(self, sigma):
        return _unit_variance_scale(sigma), (self.M - 1) * self._time_of(sigma), sigma.neg(), torch.ones_like(sigma)


class VEPreconditioner(BaseAffinePreconditioner):
    """Variance exploding: no input scaling, ``c_noise = log(σ / 2)``, output scaled by ``σ``."""

    def __init__(self, model: Module) -> None:
        super().__init__(model)

    def compute_coefficients(self, t):
        one = torch.ones_like(t)
        return one, torch.log(t / 2), t, one


def _iddpm_noise_table(M: int, C_1: float, C_2: float) -> torch.Tensor:
    """``u[0..M]`` of the improved-DDPM cosine schedule, ``u[M] = 0``.  With ``v = u² + 1`` the recurrence
    ``u[j-1] = sqrt((u[j]² + 1) / max(ᾱ[j-1] / ᾱ[j], C_1) − 1)`` is ``v[j-1] = v[j] / clip[j]``, i.e. a reversed
    cumulative product."""
    j = torch.arange(M + 1, dtype=torch.float64)
    alpha_bar = torch.sin(0.5 * math.pi * j / M / (C_2 + 1)).square()
    clip = torch.clamp(alpha_bar[:-1] / alpha_bar[1:], min=C_1)              # clip[j-1] belongs to step j = 1 .. M
    v = torch.ones(M + 1, dtype=torch.float64)
    v[:-1] = torch.flip(torch.cumprod(torch.flip(1.0 / clip, dims=[0]), dim=0), dims=[0])
    return torch.sqrt(torch.clamp(v - 1.0, min=0.0)).to(torch.float32)


class IDDPMPreconditioner(BaseAffinePreconditioner):
    """Improved DDPM: VP-style scalings; ``c_noise`` is the index of the nearest level of the discrete schedule."""

    def __init__(self, model: Module, C_1: float = 0.001, C_2: float = 0.008, M: int = 1000) -> None:
        super().__init__(model)
        for name, value in (("C_1", C_1), ("C_2", C_2), ("M", M)):
            self.register_buffer(name, torch.tensor(value))
        self.register_buffer("u", _iddpm_noise_table(M, C_1, C_2))

    def compute_coefficients(self, t):
        nearest = (t.reshape(-1, 1) - self.u.reshape(1, -1)).abs().argmin(dim=1).reshape(t.shape)
        return _unit_variance_scale(t), self.M - 1 - nearest, t.neg(), torch.ones_like(t)


def _as_sigma_data(value) -> torch.Tensor:
    """Scalar (0-d) or per-channel (1-d) float32 tensor from a number, a sequence or a tensor."""
    if isinstance(value, torch.Tensor):
        out = value.detach().float().flatten()
    elif isinstance(value, Sequence) and not isinstance(value, str):
        out = torch.tensor([float(v) for v in value])
    else:
        return torch.tensor(float(value))
    return out[0].clone() if out.numel() == 1 else out


class EDMPreconditioner(BaseAffinePreconditioner):
    """EDM scalings; ``sigma_data`` may be a scalar or one value per channel."""

    def __init__(self, model: Module, sigma_data=0.5) -> None:
        super().__init__(model)
        self.register_buffer("sigma_data", _as_sigma_data(sigma_data))
        self._sigma_data_channels = self.sigma_data.numel() if self.sigma_data.ndim else 0

    def _validate_input(self, x):
        expected = self._sigma_data_channels
        if expected and x.ndim > 1 and x.shape[1] != expected:
            raise ValueError(f"sigma_data was given for {expected} channels; x of shape {tuple(x.shape)} has {x.shape[1]}")

    def _reshape_sigma_data(self, t):
        """``sigma_data`` broadcastable against ``t`` of shape ``[B, 1, ...]``: per-channel values go to dim 1."""
        if not self._sigma_data_channels:
            return self.sigma_data
        return self.sigma_data.reshape((1, -1) + (1,) * (t.ndim - 2))

    def compute_coefficients(self, t):
        data = _plain(self._reshape_sigma_data(t))
        total_var = t.square() + data.square()
        inv_std = torch.rsqrt(total_var)
        return inv_std, 0.25 * torch.log(t), t * data * inv_std, data.square() / total_var
