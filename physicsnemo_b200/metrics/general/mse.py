"""Mean squared error metrics (parity: ``physicsnemo/metrics/general/mse.py``)."""
from typing import Union

import torch
from torch import Tensor


def mse(pred: Tensor, target: Tensor, dim: int = None, weights: Tensor = None, eps: float = 1e-8) -> Union[Tensor, float]:
    """(Weighted) mean squared error over ``dim`` (all dims when ``None``)."""
    se = (pred - target) ** 2
    if weights is None:
        return torch.mean(se, dim=dim)
    w = torch.broadcast_to(weights.to(device=se.device, dtype=se.dtype), se.shape)
    if dim is None:
        return (w * se).sum() / w.sum().clamp_min(eps)
    return (w * se).sum(dim=dim) / w.sum(dim=dim).clamp_min(eps)


def rmse(pred: Tensor, target: Tensor, dim: int = None, weights: Tensor = None, eps: float = 1e-8) -> Union[Tensor, float]:
    return torch.sqrt(mse(pred, target, dim=dim, weights=weights, eps=eps))
