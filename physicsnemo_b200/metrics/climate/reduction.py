"""Latitude-weighted reductions on (…, lat, lon) fields (parity: ``physicsnemo/metrics/climate/reduction.py``)."""
import torch
from torch import Tensor

from ..general.reduction import WeightedMean, WeightedVariance


def _compute_lat_weights(lat: Tensor) -> Tensor:
    """``|cos(lat°)|`` normalised to sum one."""
    w = torch.cos(torch.deg2rad(lat)).abs()
    return w / w.sum()


def zonal_mean(x: Tensor, lat: Tensor, dim: int = -2, keepdims: bool = False) -> Tensor:
    return WeightedMean(_compute_lat_weights(lat))(x, dim=dim, keepdims=keepdims)


def zonal_var(x: Tensor, lat: Tensor, std: bool = False, dim: int = -2, keepdims: bool = False) -> Tensor:
    v = WeightedVariance(_compute_lat_weights(lat))(x, dim=dim, keepdims=keepdims)
    return v.sqrt() if std else v


def _need_2d(x: Tensor) -> None:
    if x.ndim < 2:
        raise AssertionError("Expected x to have at least two dimensions, with the last two dimensions representing lat and lon respectively")


def global_mean(x: Tensor, lat: Tensor, keepdims: bool = False) -> Tensor:
    _need_2d(x)
    return zonal_mean(x, lat, dim=-2, keepdims=keepdims).mean(dim=-1, keepdim=keepdims)


def global_var(x: Tensor, lat: Tensor, std: bool = False, keepdims: bool = False) -> Tensor:
    _need_2d(x)
    centre = global_mean(x, lat, keepdims=True)
    v = zonal_mean((x - centre) ** 2, lat, dim=-2, keepdims=keepdims).mean(dim=-1, keepdim=keepdims)
    return v.sqrt() if std else v
