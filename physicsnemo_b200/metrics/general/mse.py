"""Mean squared error metrics (parity: ``physicsnemo/metrics/general/mse.py``)."""
from typing import Optional, Union

import torch
from torch import Tensor


def _reduce(values: Tensor, dim: Optional[int]) -> Tensor:
    return values.sum() if dim is None else values.sum(dim=dim)


def mse(pred: Tensor, target: Tensor, dim: int = None, weights: Tensor = None, eps: float = 1e-8) -> Union[Tensor, float]:
    """(Weighted) mean squared error over ``dim`` (all dims when ``None``).

    With ``weights`` (broadcastable to the inputs) the result is ``Σ w e² / max(Σ w, eps)``."""
    err2 = torch.square(pred - target)
    if weights is None:
        return err2.mean() if dim is None else err2.mean(dim=dim)
    w = weights.to(err2).expand_as(err2)
    total = _reduce(w, dim)
    return _reduce(err2 * w, dim) / torch.clamp(total, min=eps)


def rmse(pred: Tensor, target: Tensor, dim: int = None, weights: Tensor = None, eps: float = 1e-8) -> Union[Tensor, float]:
    """Square root of :func:`mse` with the same arguments."""
    return mse(pred, target, dim, weights, eps).sqrt()
