"""Weighted reductions (parity: ``physicsnemo/metrics/general/reduction.py``)."""
from abc import ABC

import torch
from torch import Tensor


class WeightedStatistic(ABC):
    """Holds normalised positive weights and aligns them with the reduced dimension of an input."""

    def __init__(self, weights: Tensor):
        if not bool(torch.all(weights > 0.0)):
            raise ValueError("Expected all weights to be positive.")
        self.weights = self._normalize(weights)

    def _normalize(self, weights: Tensor) -> Tensor:
        return weights / weights.sum()

    def __call__(self, x: Tensor, dim: int) -> Tensor:
        w = self.weights
        if w.ndim == 1:
            if x.shape[dim] != w.numel():
                raise ValueError("Expected inputs and weights to have the same size along the reduction dimension "
                                 f"but have dimensions {x.shape[dim]} and {w.numel()}.")
            shape = [1] * x.ndim
            shape[dim % x.ndim] = w.numel()
            return w.reshape(shape)
        if x.ndim != w.ndim or x.shape[dim] != w.shape[dim]:
            raise ValueError("Expected inputs and weights to have compatible shapes.")
        return w


class WeightedMean(WeightedStatistic):
    def __call__(self, x: Tensor, dim: int, keepdims: bool = False) -> Tensor:
        w = super().__call__(x, dim)
        return torch.sum(x * w, dim=dim, keepdim=keepdims)


class WeightedVariance(WeightedStatistic):
    """Weighted variance with the ``(n-1)/n`` correction over the non-zero weights."""

    def __init__(self, weights: Tensor):
        super().__init__(weights)
        self.wm = WeightedMean(self.weights)

    def __call__(self, x: Tensor, dim: int, keepdims: bool = False) -> Tensor:
        w = super().__call__(x, dim)
        centre = self.wm(x, dim, keepdims=True)
        nnz = torch.sum(w > 0.0)
        return torch.sum(w * (x - centre) ** 2, dim=dim, keepdim=keepdims) * nnz / (nnz - 1.0)
