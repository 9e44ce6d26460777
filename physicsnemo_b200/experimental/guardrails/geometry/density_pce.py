"""Polynomial-chaos density model: Mahalanobis distance in a Hermite-polynomial feature space of PCA coordinates.

Counterpart of ``physicsnemo/experimental/guardrails/geometry/density_pce.py`` (``TorchPCEDensityModel`` :37).
Fit: standardise, PCA (95 % of the variance unless ``n_components`` is given), expand the PCA coordinates in products
of probabilists' Hermite polynomials up to total degree ``poly_degree``, and store mean and (regularised) covariance of
the expansion.  Score: Mahalanobis distance of a sample's expansion; larger is more anomalous.  The expansion is built
from one table of per-dimension polynomials gathered with a multi-index matrix (a single ``prod`` over dimensions).
"""

from __future__ import annotations

from itertools import product
from typing import Optional, Union

import numpy as np
import torch

__all__ = ["TorchPCEDensityModel"]

_STATE = ("n_features_in_", "n_pca_components_", "hermite_degree_", "pca_mean_", "pca_std_", "pca_components_",
          "pca_explained_variance_ratio_", "poly_mean_", "poly_cov_", "poly_cov_inv_", "training_scores_")


class TorchPCEDensityModel:
    def __init__(self, n_components: Optional[int] = None, poly_degree: int = 2, interaction_only: bool = False,
                 random_state: Optional[int] = 0, device: Union[str, torch.device] = "cpu"):
        self.n_components, self.poly_degree, self.interaction_only, self.random_state = n_components, poly_degree, interaction_only, random_state
        self.device = torch.device(device)
        if random_state is not None:
            torch.manual_seed(random_state)
        for k in _STATE:
            setattr(self, k, None)

    def _prep(self, X) -> torch.Tensor:
        if isinstance(X, np.ndarray):
            X = torch.from_numpy(X)
        elif not isinstance(X, torch.Tensor):
            raise TypeError(f"X must be np.ndarray or torch.Tensor, got {type(X)}")
        return X.float().to(self.device)

    # ---- Hermite expansion -----------------------------------------------------------------------------------
    def _multi_indices(self, n_dims: int) -> torch.Tensor:
        top = 1 if self.interaction_only else self.poly_degree
        idx = [i for i in product(range(top + 1), repeat=n_dims) if 0 < sum(i) <= self.poly_degree]
        return torch.tensor([(0,) * n_dims] + idx, dtype=torch.long, device=self.device)           # [terms, dims]

    def _hermite_table(self, X: torch.Tensor) -> torch.Tensor:
        """``He_k(x)`` for ``k = 0 .. poly_degree``: ``[degree + 1, n, dims]`` by the three-term recurrence."""
        table = [torch.ones_like(X), X]
        for n in range(1, self.poly_degree):
            table.append(X * table[-1] - n * table[-2])
        return torch.stack(table[:self.poly_degree + 1])

    def _generate_hermite_features(self, X: torch.Tensor) -> torch.Tensor:
        idx = self._multi_indices(X.shape[1])
        table = self._hermite_table(X)                                                            # [K, n, d]
        picked = table[idx.t()[:, None, :], torch.arange(X.shape[0], device=X.device)[None, :, None],
                       torch.arange(X.shape[1], device=X.device)[:, None, None]]                   # [d, n, terms]
        return picked.prod(dim=0)

    # ---- fit / score --------------------------------------------------------------------------------------------
    def _project(self, X: torch.Tensor) -> torch.Tensor:
        return ((X - self.pca_mean_) / self.pca_std_) @ self.pca_components_

    def fit(self, X) -> "TorchPCEDensityModel":
        X = self._prep(X)
        if X.ndim != 2:
            raise ValueError(f"X must be 2D array, got shape {X.shape}")
        if X.shape[0] < 10:
            raise ValueError(f"Need at least 10 samples for fitting, got {X.shape[0]}")
        self.n_features_in_ = X.shape[1]
        self.pca_mean_ = X.mean(dim=0, keepdim=True)
        self.pca_std_ = X.std(dim=0, keepdim=True).clamp(min=1e-8)
        Z = (X - self.pca_mean_) / self.pca_std_
        _, S, Vt = torch.linalg.svd(Z, full_matrices=False)
        var = S ** 2 / (X.shape[0] - 1)
        self.pca_explained_variance_ratio_ = var / var.sum()
        if self.n_components is None:
            keep = int(torch.searchsorted(torch.cumsum(self.pca_explained_variance_ratio_, 0), torch.tensor(0.95, device=self.device))) + 1
            keep = min(keep, X.shape[1])
        else:
            keep = min(self.n_components, X.shape[0], X.shape[1])
        self.pca_components_ = Vt[:keep].T.contiguous()
        self.n_pca_components_, self.hermite_degree_ = keep, self.poly_degree
        H = self._generate_hermite_features(Z @ self.pca_components_)
        self.poly_mean_ = H.mean(dim=0)
        Hc = H - self.poly_mean_
        self.poly_cov_ = Hc.T @ Hc / (X.shape[0] - 1) + 1e-6 * torch.eye(H.shape[1], device=self.device)
        self.poly_cov_inv_ = torch.linalg.inv(self.poly_cov_)
        self.training_scores_ = self._compute_scores(H)
        return self

    def _compute_scores(self, H: torch.Tensor) -> torch.Tensor:
        Hc = H - self.poly_mean_
        return torch.sqrt(((Hc @ self.poly_cov_inv_) * Hc).sum(dim=1).clamp(min=0))

    def score(self, X) -> torch.Tensor:
        if self.pca_components_ is None:
            raise RuntimeError("Model must be fitted before scoring")
        return self._compute_scores(self._generate_hermite_features(self._project(self._prep(X))))

    def percentiles(self, scores) -> np.ndarray:
        """Percentage of training scores at or below each score."""
        if self.training_scores_ is None or len(self.training_scores_) == 0:
            raise RuntimeError("Model must be fitted before computing percentiles")
        s = self._prep(scores) if not isinstance(scores, torch.Tensor) else scores.to(self.device)
        return (100.0 * (self.training_scores_[None, :] <= s[:, None]).sum(dim=1).float() / len(self.training_scores_)).cpu().numpy()

    # ---- persistence --------------------------------------------------------------------------------------------
    def get_state(self) -> dict:
        out = {"n_components": self.n_components, "poly_degree": self.poly_degree, "interaction_only": self.interaction_only}
        for k in _STATE:
            v = getattr(self, k)
            out[k] = v.detach().cpu().numpy() if isinstance(v, torch.Tensor) else v
        return out

    def set_state(self, state: dict, device: Union[str, torch.device] = "cpu") -> None:
        self.device = torch.device(device)
        scalar = lambda v: v.item() if isinstance(v, np.ndarray) and v.ndim == 0 else v  # noqa: E731
        self.n_components = scalar(state.get("n_components"))
        self.poly_degree, self.interaction_only = int(scalar(state["poly_degree"])), bool(scalar(state["interaction_only"]))
        for k in _STATE:
            v = scalar(state.get(k))
            setattr(self, k, torch.as_tensor(v).float().to(self.device) if isinstance(v, np.ndarray) else (None if v is None else int(v)))
