"""Gaussian mixture density model in tensor operations, for density-based geometry guardrails.

Parity: ``physicsnemo/experimental/guardrails/geometry/gmm_torch.py`` (``TorchGMM``: full-covariance EM with
``reg_covar``, ``max_iter``, ``tol``, ``score_samples`` = log-density per sample, ``get_state`` / ``set_state``).
Responsibilities, weighted covariances and Cholesky factors are batched over the components, so one EM iteration is a
handful of batched matrix products on whatever device the data lives on.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn


class TorchGMM(nn.Module):
    def __init__(self, n_components: int, reg_covar: float = 1e-6, max_iter: int = 100, tol: float = 1e-3, device=None, random_state: int | None = 0):
        super().__init__()
        self.n_components, self.reg_covar, self.max_iter, self.tol = n_components, reg_covar, max_iter, tol
        self.device_, self.random_state = torch.device(device) if device is not None else None, random_state
        self.weights_ = self.means_ = self.covariances_ = self.precisions_cholesky_ = None
        self.converged_, self.n_iter_, self.lower_bound_ = False, 0, -math.inf

    def _prep(self, X) -> torch.Tensor:
        X = torch.as_tensor(X)
        X = X.to(self.device_ if self.device_ is not None else X.device)
        return X.double() if X.dtype not in (torch.float32, torch.float64) else X

    def _init(self, X: torch.Tensor) -> None:
        n, d = X.shape
        gen = torch.Generator(device="cpu")
        if self.random_state is not None:
            gen.manual_seed(self.random_state)
        centres = [X[int(torch.randint(n, (1,), generator=gen))]]
        for _ in range(1, self.n_components):                                  # k-means++ seeding
            d2 = torch.cdist(X, torch.stack(centres)).square().amin(dim=1).clamp_min(0)
            p = (d2 / d2.sum().clamp_min(1e-30)).cpu().double()
            centres.append(X[int(torch.multinomial(p, 1, generator=gen))])
        self.means_ = torch.stack(centres)
        self.weights_ = X.new_full((self.n_components,), 1.0 / self.n_components)
        cov = torch.cov(X.t()).reshape(d, d) + self.reg_covar * torch.eye(d, dtype=X.dtype, device=X.device)
        self.covariances_ = cov.unsqueeze(0).repeat(self.n_components, 1, 1)
        self._update_precisions()

    def _update_precisions(self) -> None:
        L = torch.linalg.cholesky(self.covariances_)
        eye = torch.eye(L.shape[-1], dtype=L.dtype, device=L.device).expand_as(L)
        self.precisions_cholesky_ = torch.linalg.solve_triangular(L, eye, upper=False).transpose(-1, -2)   # P with Σ⁻¹ = P Pᵀ

    def _log_prob(self, X: torch.Tensor) -> torch.Tensor:
        d = X.shape[1]
        y = torch.einsum("nkd,kde->nke", X.unsqueeze(1) - self.means_.unsqueeze(0), self.precisions_cholesky_)
        log_det = self.precisions_cholesky_.diagonal(dim1=-2, dim2=-1).log().sum(-1)
        return -0.5 * (d * math.log(2 * math.pi) + y.square().sum(-1)) + log_det

    def _e_step(self, X):
        weighted = self._log_prob(X) + self.weights_.log()
        norm = torch.logsumexp(weighted, dim=1)
        return torch.exp(weighted - norm.unsqueeze(1)), float(norm.mean())

    def _m_step(self, X, resp) -> None:
        nk = resp.sum(0) + 10 * torch.finfo(X.dtype).eps
        self.weights_ = nk / nk.sum()
        self.means_ = (resp.t() @ X) / nk.unsqueeze(1)
        diff = X.unsqueeze(1) - self.means_.unsqueeze(0)
        cov = torch.einsum("nk,nkd,nke->kde", resp, diff, diff) / nk.reshape(-1, 1, 1)
        self.covariances_ = cov + self.reg_covar * torch.eye(X.shape[1], dtype=X.dtype, device=X.device)
        self._update_precisions()

    @torch.no_grad()
    def fit(self, X) -> "TorchGMM":
        X = self._prep(X)
        if X.ndim != 2 or X.shape[0] < self.n_components:
            raise ValueError("X must be (n_samples, n_features) with at least n_components samples")
        self._init(X)
        prev = -math.inf
        for it in range(1, self.max_iter + 1):
            resp, bound = self._e_step(X)
            self._m_step(X, resp)
            self.n_iter_, self.lower_bound_ = it, bound
            if abs(bound - prev) < self.tol:
                self.converged_ = True
                break
            prev = bound
        return self

    @torch.no_grad()
    def score_samples(self, X) -> torch.Tensor:
        if self.means_ is None:
            raise RuntimeError("fit the model before scoring")
        X = self._prep(X).to(self.means_)
        return torch.logsumexp(self._log_prob(X) + self.weights_.log(), dim=1)

    def score(self, X) -> torch.Tensor:
        return self.score_samples(X).mean()

    def get_state(self) -> dict:
        return {k: getattr(self, k).detach().cpu() for k in ("weights_", "means_", "covariances_", "precisions_cholesky_")}

    def set_state(self, state: dict, device=None) -> None:
        for k, v in state.items():
            setattr(self, k, torch.as_tensor(v).to(device if device is not None else "cpu"))
