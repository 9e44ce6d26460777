"""Anomaly correlation coefficient (parity: ``physicsnemo/metrics/climate/acc.py``)."""
import torch
from torch import Tensor

from .reduction import _compute_lat_weights


def acc(pred: Tensor, target: Tensor, climatology: Tensor, lat: Tensor) -> Tensor:
    """Latitude-weighted correlation of the anomalies of ``pred`` and ``target`` over the last two dims."""
    for t in (pred, target, climatology):
        if t.ndim <= 2:
            raise AssertionError("Expected predictions to have at least two dimensions")
    w = _compute_lat_weights(lat)[:, None]
    pa, ta = pred - climatology, target - climatology
    norm = (w * torch.ones_like(pa)).sum(dim=(-2, -1), keepdim=True)
    pa = pa - (w * pa).sum(dim=(-2, -1), keepdim=True) / norm
    ta = ta - (w * ta).sum(dim=(-2, -1), keepdim=True) / norm
    cov = (w * pa * ta).sum(dim=(-2, -1))
    return cov / torch.sqrt((w * pa * pa).sum(dim=(-2, -1)) * (w * ta * ta).sum(dim=(-2, -1)))
