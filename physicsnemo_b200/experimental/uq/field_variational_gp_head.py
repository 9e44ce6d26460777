"""Point-wise multitask variational GP head for field regression with per-point uncertainty.

Parity: ``physicsnemo/experimental/uq/field_variational_gp_head.py`` (``FieldVariationalGPHead``,
``FieldVariationalGPPrediction``).  The reference builds on GPyTorch (an independent-multitask variational strategy, a
Matérn ARD kernel, ``VariationalELBO``); GPyTorch is not installed here, so — like the scalar ``VariationalGPHead`` next to
it — this head is written directly in PyTorch: one sparse variational GP per output channel (own inducing points,
whitened variational distribution, Matérn-½ / 3⁄2 / 5⁄2 ARD kernel with a hard lengthscale interval), evaluated only at
the marginals, so a field of N points costs O(N · M) per channel instead of an N × N covariance.

Features ``(..., D)`` → optional DKL MLP → optional ``l2_radial`` normalisation (unit direction plus the batch-standardised
magnitude as one extra kernel dimension) → GP.  Observation noise is one learned scalar per channel, or, with
``noise_mlp_hidden``, an MLP of the GP-input features that modulates that floor per point (heteroscedastic), clamped to
``noise_std_range``.  ``forward_and_loss`` returns the predictive mean and the negative ELBO per data point
(expected Gaussian log-likelihood minus KL / ``n_train``); ``predict`` returns mean, total variance, interval and the
epistemic (latent-function) variance.
"""
from __future__ import annotations

import math
from typing import List, Literal, NamedTuple, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .variational_gp_head import _VariationalGPLayer, _inv_softplus


class FieldVariationalGPPrediction(NamedTuple):
    """All fields ``(..., num_tasks)``: mean, total variance (epistemic + observation noise), interval bounds, and the
    latent-function variance alone (the signal for "where is the model uncertain")."""

    mean: torch.Tensor
    variance: torch.Tensor
    lower: torch.Tensor
    upper: torch.Tensor
    epistemic_variance: torch.Tensor


def _marginals(layer: _VariationalGPLayer, x: torch.Tensor, jitter: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """Mean and variance of ``q(f(x))`` at every row of ``x`` ``[N, D]`` (no cross-covariances)."""
    Z = layer.inducing_points.to(x.dtype)
    M = Z.shape[0]
    Kzz = layer.kernel(Z, Z) + jitter * torch.eye(M, dtype=x.dtype, device=x.device)
    A = torch.linalg.solve_triangular(torch.linalg.cholesky(Kzz), layer.kernel(Z, x), upper=False)      # [M, N]
    Lq = layer.scale_tril().to(x.dtype)
    mean = layer.constant_mean.to(x.dtype) + A.t() @ layer.variational_mean.to(x.dtype)
    prior_var = layer.outputscale.to(x.dtype).expand(x.shape[0])                                       # k(x, x) of a Matérn kernel
    var = prior_var - A.square().sum(0) + (Lq.t() @ A).square().sum(0)
    return mean, var.clamp_min(0)


def _mlp(widths: Sequence[int], out: Optional[int] = None) -> nn.Sequential:
    layers: List[nn.Module] = []
    for a, b in zip(widths[:-1], widths[1:]):
        layers += [nn.Linear(a, b), nn.ReLU()]
    if out is not None:
        layers.append(nn.Linear(widths[-1], out))
    return nn.Sequential(*layers)


class FieldVariationalGPHead(nn.Module):
    def __init__(self, input_dim: int, *, n_train: int, num_tasks: int = 4, n_inducing: int = 256,
                 inducing_points: Optional[torch.Tensor] = None, lengthscale_range: Tuple[float, float] = (0.01, 10.0),
                 lengthscale_prior: Optional[Tuple[float, float]] = None, outputscale_prior: Optional[Tuple[float, float]] = None,
                 matern_nu: float = 2.5, mlp_hidden: Optional[List[int]] = None, feature_norm: Literal["none", "l2_radial"] = "none",
                 use_double: bool = True, jitter: Tuple[float, float] = (1e-3, 1e-4), confidence_z: float = 1.96,
                 noise_mlp_hidden: Optional[List[int]] = None, noise_std_range: Tuple[float, float] = (1e-3, 10.0)) -> None:
        super().__init__()
        if feature_norm not in ("none", "l2_radial"):
            raise ValueError(f"feature_norm is 'none' or 'l2_radial', got {feature_norm!r}")
        self.num_tasks, self._num_data = num_tasks, int(n_train)
        self._use_double, self._jitter, self._confidence_z, self._feature_norm = use_double, jitter, confidence_z, feature_norm
        self.feature_extractor = _mlp([input_dim, *mlp_hidden]) if mlp_hidden else None
        gp_dim = mlp_hidden[-1] if mlp_hidden else input_dim
        self._radial_bn = nn.BatchNorm1d(1, affine=False) if feature_norm == "l2_radial" else None
        gp_dim += 1 if self._radial_bn is not None else 0
        self.gp_input_dim = gp_dim
        Z = self._init_inducing(inducing_points, n_inducing, gp_dim, num_tasks)
        self.gp_layer = nn.ModuleList(_VariationalGPLayer(Z[k], gp_dim, lengthscale_range, matern_nu) for k in range(num_tasks))
        self.raw_noise = nn.Parameter(torch.full((num_tasks,), _inv_softplus(0.6932 - 1e-4)))          # noise = 1e-4 + softplus(raw)
        self._priors = {"lengthscale": lengthscale_prior, "outputscale": outputscale_prior}
        self._noise_range = (float(noise_std_range[0]), float(noise_std_range[1]))
        self.noise_head = None
        if noise_mlp_hidden:
            self.noise_head = _mlp([gp_dim, *noise_mlp_hidden], out=num_tasks)
            nn.init.zeros_(self.noise_head[-1].weight)            # starts as the homoscedastic model (modulation 1)
            nn.init.zeros_(self.noise_head[-1].bias)
        if use_double:
            self.gp_layer.double()
            self.raw_noise.data = self.raw_noise.data.double()

    @staticmethod
    def _init_inducing(given, n_inducing: int, gp_dim: int, num_tasks: int) -> torch.Tensor:
        if given is None:
            return torch.randn(num_tasks, n_inducing, gp_dim)
        if given.shape[-1] != gp_dim:
            raise ValueError(f"inducing points have width {given.shape[-1]}, the kernel input has {gp_dim} "
                             "(pass them through transform_features first)")
        return given.clone() if given.ndim == 3 else given.unsqueeze(0).repeat(num_tasks, 1, 1)

    # ------------------------------------------------------------- features
    @property
    def heteroscedastic(self) -> bool:
        return self.noise_head is not None

    @staticmethod
    def _flatten_points(t: torch.Tensor) -> torch.Tensor:
        return t.reshape(-1, t.shape[-1])

    def transform_features(self, features: torch.Tensor) -> torch.Tensor:
        """Features as the kernel sees them: ``(..., D)`` → ``(N, gp_input_dim)``."""
        x = self._flatten_points(features)
        if self.feature_extractor is not None:
            x = self.feature_extractor(x)
        if self._radial_bn is not None:
            norm = x.norm(dim=-1, keepdim=True)
            x = torch.cat([x / norm.clamp_min(1e-12), self._radial_bn(norm)], dim=-1)
        return x.double() if self._use_double else x

    @torch.no_grad()
    def set_inducing_points(self, features: torch.Tensor) -> None:
        """Seed the inducing points of every channel from real (transformed) features: a random subset of the rows."""
        x = self.transform_features(features)
        M = self.gp_layer[0].inducing_points.shape[0]
        if x.shape[0] < M:
            raise ValueError(f"{M} inducing points need at least as many feature rows, got {x.shape[0]}")
        for layer in self.gp_layer:
            pick = torch.randperm(x.shape[0], device=x.device)[:M]
            layer.inducing_points.copy_(x[pick].to(layer.inducing_points.dtype))

    def _pointwise_noise_var(self, x: torch.Tensor) -> torch.Tensor:
        floor = (1e-4 + F.softplus(self.raw_noise)).to(x.dtype)                                   # [tasks]
        if self.noise_head is None:
            return floor.expand(x.shape[0], -1)
        std = floor.sqrt() * torch.exp(self.noise_head(x.to(self.noise_head[0].weight.dtype)).to(x.dtype))
        return std.clamp(*self._noise_range).square()

    def _latent(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        jit = self._jitter[1] if x.dtype == torch.float64 else self._jitter[0]
        stats = [_marginals(layer, x, jit) for layer in self.gp_layer]
        return torch.stack([m for m, _ in stats], dim=-1), torch.stack([v for _, v in stats], dim=-1)     # [N, tasks] each

    def _log_prior(self) -> torch.Tensor:
        total = self.raw_noise.new_zeros(())
        for name, prior in self._priors.items():
            if prior is None:
                continue
            a, b = prior
            for layer in self.gp_layer:
                v = getattr(layer, name)
                total = total + ((a - 1) * v.log() - b * v).sum()
        return total

    # --------------------------------------------------------------- public
    def forward(self, features: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Latent mean and variance per point and channel, ``(..., num_tasks)`` each."""
        mean, var = self._latent(self.transform_features(features))
        shape = (*features.shape[:-1], self.num_tasks)
        return mean.reshape(shape).to(features.dtype), var.reshape(shape).to(features.dtype)

    def forward_and_loss(self, features: torch.Tensor, targets: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """``(predictive mean (..., tasks), negative ELBO per data point)``."""
        x = self.transform_features(features)
        mean, var = self._latent(x)
        y = self._flatten_points(targets).to(mean.dtype)
        s2 = self._pointwise_noise_var(x)
        ell = -0.5 * (math.log(2 * math.pi) + s2.log() + ((y - mean).square() + var) / s2)
        kl = sum(layer.kl_divergence() for layer in self.gp_layer)
        prior = self._log_prior() if not self.heteroscedastic else 0.0           # the hand-built hetero objective carries no prior term
        elbo = ell.sum(-1).mean() - (kl - prior) / self._num_data
        return mean.reshape(*features.shape[:-1], self.num_tasks).to(features.dtype), (-elbo).to(features.dtype)

    def loss(self, features: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        return self.forward_and_loss(features, targets)[1]

    @torch.no_grad()
    def predict(self, features: torch.Tensor) -> FieldVariationalGPPrediction:
        was_training = self.training
        self.eval()
        try:
            x = self.transform_features(features)
            mean, epi = self._latent(x)
            total = epi + self._pointwise_noise_var(x)
            half = self._confidence_z * total.sqrt()
            shape, dt = (*features.shape[:-1], self.num_tasks), features.dtype
            out = (mean, total, mean - half, mean + half, epi)
            return FieldVariationalGPPrediction(*(t.reshape(shape).to(dt) for t in out))
        finally:
            if was_training:
                self.train()
