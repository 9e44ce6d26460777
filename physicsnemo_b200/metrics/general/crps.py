"""Continuous ranked probability score (parity: ``physicsnemo/metrics/general/crps.py``).

Three estimators: the kernel form ``E|X − y| − ½ E|X − X'|`` on a sorted ensemble (exact, O(m log m)), the closed form
for a Gaussian forecast, and the integral of the squared difference between an empirical CDF on bins and the step
function at the observation.
"""
import math
from typing import Union

import numpy as np
import torch
from torch import Tensor

from .histogram import cdf as cdf_function

_METHODS = ("kernel", "sort", "histogram")


def _as_tensor_like(obs, like: Tensor) -> Tensor:
    return torch.from_numpy(obs).to(like.device) if isinstance(obs, np.ndarray) else obs


def _kernel_crps_implementation(pred: Tensor, obs: Tensor, biased: bool) -> Tensor:
    """Ensemble members along the LAST axis.  The pair term ``½ E|X − X'|`` of a sorted sample is the weighted sum
    ``Σ_i (2i − m − 1) x_(i) / norm`` with ``norm = m²`` (biased) or ``m (m − 1)`` (fair)."""
    members = pred.shape[-1]
    distance_to_obs = (pred - obs.unsqueeze(-1)).abs().mean(dim=-1)
    ordered = pred.sort(dim=-1).values
    rank = torch.arange(members, device=pred.device, dtype=pred.dtype)
    weight = (2.0 * rank - (members - 1)) / float(members * members if biased else members * (members - 1))
    return distance_to_obs - (ordered * weight).sum(dim=-1)


def kcrps(pred: Tensor, obs: Tensor, dim: int = 0, biased: bool = True):
    """Kernel CRPS of an ensemble whose members run along ``dim``."""
    return _kernel_crps_implementation(pred.movedim(dim, -1), obs, biased)


def _crps_gaussian(mean: Tensor, std: Tensor, obs) -> Tensor:
    """``σ [ z (2Φ(z) − 1) + 2φ(z) − 1/√π ]`` with ``z = (y − μ)/σ``."""
    obs = _as_tensor_like(obs, mean)
    for name, other in (("standard deviation", std), ("observation", obs)):
        if other.shape != mean.shape:
            raise ValueError(f"the {name} has shape {tuple(other.shape)} but the mean has shape {tuple(mean.shape)}")
    z = (obs - mean) / std
    density = torch.exp(-0.5 * z * z) / math.sqrt(2.0 * math.pi)
    two_cdf_minus_one = torch.erf(z / math.sqrt(2.0))
    return std * (z * two_cdf_minus_one + 2.0 * density - 1.0 / math.sqrt(math.pi))


def _crps_from_cdf(bin_edges: Tensor, cdf: Tensor, obs) -> Tensor:
    """``∫ (F(x) − 1[x ≥ y])² dx`` on equally spaced bins: ``bin_edges`` ``[B + 1, ...]``, ``cdf`` ``[B, ...]``."""
    obs = _as_tensor_like(obs, cdf)
    trailing = bin_edges.shape[1:]
    if cdf.shape[1:] != trailing:
        raise ValueError(f"bins {tuple(bin_edges.shape)} and cdf {tuple(cdf.shape)} differ beyond their first dimension")
    if obs.shape != trailing:
        raise ValueError(f"observations {tuple(obs.shape)} do not match the bins' trailing shape {tuple(trailing)}")
    if bin_edges.shape[0] - 1 != cdf.shape[0]:
        raise ValueError(f"{bin_edges.shape[0]} bin edges need {bin_edges.shape[0] - 1} cdf values, got {cdf.shape[0]}")
    width = bin_edges[1] - bin_edges[0]
    centres = (bin_edges[:-1] + bin_edges[1:]) / 2
    step = (centres >= obs).to(torch.int32)
    return ((cdf - step).abs().square() * width).sum(dim=0)


def _crps_from_counts(bin_edges: Tensor, counts: Tensor, obs) -> Tensor:
    empirical = (counts / counts.sum(dim=0)).cumsum(dim=0)
    return _crps_from_cdf(bin_edges, empirical, obs)


def crps(pred: Tensor, obs, dim: int = 0, method: str = "kernel") -> Tensor:
    """CRPS of an ensemble forecast; ``method`` is one of "kernel" / "sort" (exact) or "histogram" (binned CDF)."""
    if method not in _METHODS:
        raise ValueError(f"unknown CRPS method {method!r}; choose from {', '.join(_METHODS)}")
    obs = torch.as_tensor(obs, device=pred.device, dtype=pred.dtype)
    if method != "histogram":
        return kcrps(pred, obs, dim=dim)
    members = pred.shape[dim]
    edges, values = cdf_function(pred.movedim(dim, 0), bins=max(int(np.sqrt(members)), 100))
    return _crps_from_cdf(edges, values, obs)
