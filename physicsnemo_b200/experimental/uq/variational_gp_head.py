"""Sparse variational Gaussian-process head for uncertainty on top of a learned embedding.

Parity: ``physicsnemo/experimental/uq/variational_gp_head.py`` (``VariationalGPHead``, ``GPPrediction``): optional MLP
feature extractor → SVGP with ``n_inducing`` learnable inducing points, constant mean, scaled Matérn-ν ARD kernel with
interval-constrained length scales, Gaussian likelihood; ``loss`` is the negative ELBO normalised per datum
(``E_q[log p(y|f)]`` averaged over the batch minus ``KL / n_train``), ``predict`` returns mean, variance (with observation
noise) and a ``± z σ`` band.  The reference builds this on gpytorch; gpytorch is not available here, so the model is
written out with the whitened Cholesky parameterisation (``u = L_zz v``, ``q(v) = N(m, L_q L_qᵀ)``):

    A = L_zz⁻¹ K_zx,   mean = c + Aᵀ m,   cov = K_xx − Aᵀ A + Aᵀ L_q L_qᵀ A,
    KL = ½ (tr(L_q L_qᵀ) + mᵀ m − M − 2 Σ log diag L_q).
"""
from __future__ import annotations

import math
from typing import NamedTuple, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F


class GPPrediction(NamedTuple):
    mean: torch.Tensor
    variance: torch.Tensor
    lower: torch.Tensor
    upper: torch.Tensor


class GPDistribution(NamedTuple):
    """Latent-function posterior at the query points."""

    mean: torch.Tensor
    covariance_matrix: torch.Tensor

    @property
    def variance(self) -> torch.Tensor:
        return self.covariance_matrix.diagonal(dim1=-2, dim2=-1)


def _inv_softplus(x: float) -> float:
    return math.log(math.expm1(x))


class _VariationalGPLayer(nn.Module):
    def __init__(self, inducing_points: torch.Tensor, input_dim: int, lengthscale_range=(0.01, 10.0), matern_nu: float = 2.5):
        super().__init__()
        if matern_nu not in (0.5, 1.5, 2.5):
            raise ValueError("matern_nu must be 0.5, 1.5 or 2.5")
        M = inducing_points.shape[0]
        self.nu, self.ls_lo, self.ls_hi = matern_nu, float(lengthscale_range[0]), float(lengthscale_range[1])
        self.inducing_points = nn.Parameter(inducing_points.clone())
        self.variational_mean = nn.Parameter(torch.zeros(M))
        self.chol_variational_covar = nn.Parameter(torch.eye(M))
        self.constant_mean = nn.Parameter(torch.zeros(()))
        init_ls = min(max(math.log(2.0), self.ls_lo * 1.01), self.ls_hi * 0.99)                # same default scale as softplus(0)
        frac = (init_ls - self.ls_lo) / (self.ls_hi - self.ls_lo)
        self.raw_lengthscale = nn.Parameter(torch.full((input_dim,), math.log(frac / (1 - frac))))
        self.raw_outputscale = nn.Parameter(torch.zeros(()))

    @property
    def lengthscale(self) -> torch.Tensor:
        return self.ls_lo + (self.ls_hi - self.ls_lo) * torch.sigmoid(self.raw_lengthscale)

    @property
    def outputscale(self) -> torch.Tensor:
        return F.softplus(self.raw_outputscale)

    def kernel(self, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        ls = self.lengthscale.to(a.dtype)
        r = torch.cdist(a / ls, b / ls).clamp_min(1e-15)
        if self.nu == 0.5:
            k = torch.exp(-r)
        elif self.nu == 1.5:
            s = math.sqrt(3.0) * r
            k = (1 + s) * torch.exp(-s)
        else:
            s = math.sqrt(5.0) * r
            k = (1 + s + s * s / 3.0) * torch.exp(-s)
        return self.outputscale.to(a.dtype) * k

    def scale_tril(self) -> torch.Tensor:
        L = torch.tril(self.chol_variational_covar)
        d = L.diagonal()
        return L - torch.diag(d) + torch.diag(d.abs().clamp_min(1e-8))

    def forward(self, x: torch.Tensor, jitter: float) -> GPDistribution:
        Z = self.inducing_points.to(x.dtype)
        M = Z.shape[0]
        Kzz = self.kernel(Z, Z) + jitter * torch.eye(M, dtype=x.dtype, device=x.device)
        Lzz = torch.linalg.cholesky(Kzz)
        A = torch.linalg.solve_triangular(Lzz, self.kernel(Z, x), upper=False)                 # [M, N]
        Lq = self.scale_tril().to(x.dtype)
        mean = self.constant_mean.to(x.dtype) + A.t() @ self.variational_mean.to(x.dtype)
        SA = Lq.t() @ A
        cov = self.kernel(x, x) - A.t() @ A + SA.t() @ SA
        return GPDistribution(mean, cov)

    def kl_divergence(self) -> torch.Tensor:
        Lq, m = self.scale_tril(), self.variational_mean
        return 0.5 * (Lq.square().sum() + m.square().sum() - m.numel() - 2.0 * Lq.diagonal().log().sum())


class VariationalGPHead(nn.Module):
    def __init__(self, input_dim: int = 32, *, n_train: int, n_inducing: int = 64, inducing_points: torch.Tensor | None = None,
                 lengthscale_range: tuple[float, float] = (0.01, 10.0), lengthscale_prior=None, outputscale_prior=None, matern_nu: float = 2.5,
                 mlp_hidden: Sequence[int] | None = None, use_double: bool = True, jitter: tuple[float, float] = (1e-4, 1e-6),
                 confidence_z: float = 1.96):
        super().__init__()
        self._use_double, self._jitter, self._confidence_z, self.n_train = use_double, jitter, confidence_z, n_train
        if mlp_hidden:
            layers, d = [], input_dim
            for h in mlp_hidden:
                layers += [nn.Linear(d, h), nn.ReLU()]
                d = h
            self.feature_extractor, gp_dim = nn.Sequential(*layers), mlp_hidden[-1]
        else:
            self.feature_extractor, gp_dim = None, input_dim
        if inducing_points is None:
            inducing_points = torch.randn(n_inducing, gp_dim)
        elif inducing_points.shape[-1] != gp_dim and self.feature_extractor is not None:
            with torch.no_grad():
                inducing_points = self.feature_extractor(inducing_points)
        self.gp_layer = _VariationalGPLayer(inducing_points, gp_dim, lengthscale_range, matern_nu)
        self.raw_noise = nn.Parameter(torch.tensor(_inv_softplus(0.6932 - 1e-4)))              # noise = 1e-4 + softplus(raw)
        self._priors = {"lengthscale": lengthscale_prior, "outputscale": outputscale_prior}   # Gamma(concentration, rate) or None
        if use_double:
            self.gp_layer.double()
            self.raw_noise.data = self.raw_noise.data.double()

    @property
    def noise(self) -> torch.Tensor:
        return 1e-4 + F.softplus(self.raw_noise)

    def _features(self, embedding: torch.Tensor) -> torch.Tensor:
        if self.feature_extractor is not None:
            embedding = self.feature_extractor(embedding)
        return embedding.double() if self._use_double else embedding

    def _latent(self, embedding: torch.Tensor) -> GPDistribution:
        x = self._features(embedding)
        return self.gp_layer(x, self._jitter[1] if x.dtype == torch.float64 else self._jitter[0])

    def forward(self, embedding: torch.Tensor) -> GPDistribution:
        d = self._latent(embedding)
        return GPDistribution(d.mean.to(embedding.dtype), d.covariance_matrix.to(embedding.dtype))

    def _log_prior(self) -> torch.Tensor:
        total = self.raw_noise.new_zeros(())
        for name, prior in self._priors.items():
            if prior is not None:
                v, (a, b) = getattr(self.gp_layer, name), prior
                total = total + ((a - 1) * v.log() - b * v).sum()                             # Gamma log-density up to a constant
        return total

    def forward_and_loss(self, embedding: torch.Tensor, target: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        d = self._latent(embedding)
        y, s2 = target.to(d.mean.dtype), self.noise.to(d.mean.dtype)
        ell = -0.5 * (math.log(2 * math.pi) + s2.log() + ((y - d.mean).square() + d.variance) / s2)
        elbo = ell.mean() - (self.gp_layer.kl_divergence() - self._log_prior()) / self.n_train
        return d.mean.to(embedding.dtype), (-elbo).to(embedding.dtype)

    def loss(self, embedding: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        return self.forward_and_loss(embedding, target)[1]

    @torch.no_grad()
    def predict(self, embedding: torch.Tensor) -> GPPrediction:
        was_training = self.training
        self.eval()
        try:
            d = self._latent(embedding)
            var = d.variance.clamp_min(0) + self.noise.to(d.mean.dtype)
            half = self._confidence_z * var.sqrt()
            dt = embedding.dtype
            return GPPrediction(d.mean.to(dt), var.to(dt), (d.mean - half).to(dt), (d.mean + half).to(dt))
        finally:
            if was_training:
                self.train()
