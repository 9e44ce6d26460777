"""Density model behind the geometry guardrail: Gaussian mixture or polynomial-chaos, one interface.

Counterpart of ``physicsnemo/experimental/guardrails/geometry/density_model.py`` (``GeometryDensityModel`` :30).
``score`` returns an anomaly score per sample (negative log-likelihood for the mixture, Mahalanobis distance for the
polynomial-chaos model; larger is more anomalous); ``percentiles`` ranks scores against those of the training set.
"""

from __future__ import annotations

from typing import Optional, Union

import numpy as np
import torch

from ..gmm import TorchGMM
from .density_pce import TorchPCEDensityModel

__all__ = ["GeometryDensityModel"]

_HYPER = ("method", "gmm_components", "pce_components", "poly_degree", "interaction_only", "random_state")


class GeometryDensityModel:
    def __init__(self, method: str = "gmm", gmm_components: int = 1, pce_components: Optional[int] = None, poly_degree: int = 2,
                 interaction_only: bool = False, random_state: Optional[int] = 0, device: Union[str, torch.device] = "cpu"):
        self.method = method.lower()
        if self.method not in ("gmm", "pce"):
            raise ValueError(f"method must be 'gmm' or 'pce', got '{self.method}'")
        self.gmm_components, self.pce_components, self.poly_degree = gmm_components, pce_components, poly_degree
        self.interaction_only, self.random_state, self.device = interaction_only, random_state, torch.device(device)
        self.ref_scores: Optional[torch.Tensor] = None
        self.model = self._make()

    def _make(self):
        if self.method == "gmm":
            return TorchGMM(n_components=self.gmm_components, device=self.device, random_state=self.random_state)
        return TorchPCEDensityModel(n_components=self.pce_components, poly_degree=self.poly_degree, interaction_only=self.interaction_only,
                                    random_state=self.random_state, device=self.device)

    def _prep(self, X) -> torch.Tensor:
        if isinstance(X, np.ndarray):
            X = torch.from_numpy(X)
        elif not isinstance(X, torch.Tensor):
            raise TypeError(f"X must be np.ndarray or torch.Tensor, got {type(X)}")
        return X.float().to(self.device)

    def fit(self, X) -> None:
        X = self._prep(X)
        self.model.fit(X)
        self.ref_scores = self.score(X)

    def score(self, X) -> torch.Tensor:
        X = self._prep(X)
        return -self.model.score_samples(X) if self.method == "gmm" else self.model.score(X)

    def percentiles(self, scores) -> np.ndarray:
        if self.ref_scores is None or len(self.ref_scores) == 0:
            raise RuntimeError("Density model not fitted. Call fit() before computing percentiles.")
        s = (torch.from_numpy(scores) if isinstance(scores, np.ndarray) else scores).to(self.ref_scores)
        return (100.0 * (self.ref_scores[None, :] <= s[:, None]).sum(dim=1).float() / len(self.ref_scores)).cpu().numpy()

    def get_state(self) -> dict:
        state = {k: getattr(self, k) for k in _HYPER}
        state["ref_scores"] = None if self.ref_scores is None else self.ref_scores.detach().cpu().numpy()
        for k, v in self.model.get_state().items():
            state[f"{self.method}_{k}"] = v.numpy() if isinstance(v, torch.Tensor) else v
        return state

    def set_state(self, state: dict, device: Union[str, torch.device] = "cpu") -> None:
        scalar = lambda v: v.item() if isinstance(v, np.ndarray) and v.ndim == 0 else v  # noqa: E731
        for k in _HYPER:
            if k in state:
                setattr(self, k, scalar(state[k]))
        self.method, self.device = str(self.method), torch.device(device)
        self.ref_scores = torch.as_tensor(np.asarray(state["ref_scores"])).float().to(self.device)
        self.model = self._make()
        prefix = f"{self.method}_"
        inner = {k[len(prefix):]: v for k, v in state.items() if k.startswith(prefix)}
        if self.method == "gmm":
            inner = {k: torch.as_tensor(np.asarray(v)) for k, v in inner.items()}
        self.model.set_state(inner, device=self.device)
