"""Relative errors (parity: ``physicsnemo/metrics/general/relative_error.py``): per-sample ratios of
error and target energy, reduced over the batch."""
from typing import Optional

import torch
from torch import Tensor


def _check(pred: Tensor, target: Tensor) -> None:
    if pred.shape != target.shape:
        raise ValueError(f"pred and target must have the same shape, got {tuple(pred.shape)} and {tuple(target.shape)}")
    if pred.ndim < 1:
        raise ValueError("pred and target must have at least a batch dimension")


def _ratio(pred, target, power, batch_dim, eps, reduction):
    _check(pred, target)
    dims = [d for d in range(pred.ndim) if d != batch_dim % pred.ndim]
    num = ((pred - target).abs() ** 2).sum(dim=dims)
    den = (target.abs() ** 2).sum(dim=dims).clamp_min(eps)
    r = num / den
    if power == 0.5:
        r = r.sqrt()
    if reduction == "mean":
        return r.mean()
    if reduction == "sum":
        return r.sum()
    if reduction == "none":
        return r
    raise ValueError(f"unknown reduction {reduction}")


def relative_mse(pred: Tensor, target: Tensor, batch_dim: int = 0, eps: float = 1e-12, reduction: str = "mean") -> Tensor:
    """``||pred - target||² / ||target||²`` per sample."""
    return _ratio(pred, target, 1.0, batch_dim, eps, reduction)


def relative_l2(pred: Tensor, target: Tensor, batch_dim: int = 0, eps: float = 1e-12, reduction: str = "mean") -> Tensor:
    """``||pred - target|| / ||target||`` per sample."""
    return _ratio(pred, target, 0.5, batch_dim, eps, reduction)
