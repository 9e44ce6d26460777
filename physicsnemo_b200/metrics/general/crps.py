"""Continuous ranked probability score (parity: ``physicsnemo/metrics/general/crps.py``)."""
from typing import Union

import numpy as np
import torch
from torch import Tensor

from .histogram import cdf as cdf_function


def _kernel_crps_implementation(pred: Tensor, obs: Tensor, biased: bool) -> Tensor:
    """``E|X − y| − ½ E|X − X'|`` with the spread term evaluated on the sorted ensemble in O(m log m)."""
    skill = torch.abs(pred - obs[..., None]).mean(-1)
    pred, _ = torch.sort(pred)
    m = pred.size(-1)
    i = torch.arange(1, m + 1, device=pred.device, dtype=pred.dtype)
    denom = m * m if biased else m * (m - 1)
    spread = torch.sum((2 * i - m - 1) / denom * pred, dim=-1)
    return skill - spread


def kcrps(pred: Tensor, obs: Tensor, dim: int = 0, biased: bool = True):
    """Kernel CRPS of an ensemble along ``dim``."""
    return _kernel_crps_implementation(torch.movedim(pred, dim, -1), obs, biased=biased)


def _crps_gaussian(mean: Tensor, std: Tensor, obs) -> Tensor:
    if isinstance(obs, np.ndarray):
        obs = torch.from_numpy(obs).to(mean.device)
    if mean.shape != std.shape:
        raise ValueError(f"Mean and standard deviation must have compatible shapes but found {mean.shape} and {std.shape}.")
    if mean.shape != obs.shape:
        raise ValueError(f"Mean and obs must have compatible shapes but found {mean.shape} and {obs.shape}.")
    d = (obs - mean) / std
    phi = torch.exp(-0.5 * d ** 2) / (2 * torch.pi) ** 0.5
    Phi = torch.erf(d / 2 ** 0.5)
    return std * (2 * phi + d * Phi - 1.0 / torch.pi ** 0.5)


def _crps_from_cdf(bin_edges: Tensor, cdf: Tensor, obs) -> Tensor:
    if isinstance(obs, np.ndarray):
        obs = torch.from_numpy(obs).to(cdf.device)
    if bin_edges.shape[1:] != cdf.shape[1:]:
        raise ValueError(f"Expected bins and cdf to have compatible non-zeroth dimensions but have shapes {bin_edges.shape[1:]} and {cdf.shape[1:]}.")
    if bin_edges.shape[1:] != obs.shape:
        raise ValueError(f"Expected bins and observations to have compatible broadcasting dimensions but have shapes {bin_edges.shape[1:]} and {obs.shape}.")
    if bin_edges.shape[0] != cdf.shape[0] + 1:
        raise ValueError(f"Expected zeroth dimension of cdf to be equal to the zeroth dimension of bins + 1 but have shapes {bin_edges.shape[0]} and {cdf.shape[0]}+1.")
    dbins = bin_edges[1] - bin_edges[0]
    mids = 0.5 * (bin_edges[1:] + bin_edges[:-1])
    heaviside = torch.ge(mids, obs).int()
    return torch.sum(torch.abs(cdf - heaviside) ** 2 * dbins, dim=0)


def _crps_from_counts(bin_edges: Tensor, counts: Tensor, obs) -> Tensor:
    cdf_hat = torch.cumsum(counts / torch.sum(counts, dim=0), dim=0)
    return _crps_from_cdf(bin_edges, cdf_hat, obs)


def crps(pred: Tensor, obs, dim: int = 0, method: str = "kernel") -> Tensor:
    """CRPS of an ensemble forecast: ``method`` in {"kernel", "sort", "histogram"}."""
    if method not in ["kernel", "sort", "histogram"]:
        raise ValueError("Method must either be 'kernel', 'sort' or 'histogram'.")
    n = pred.shape[dim]
    obs = torch.as_tensor(obs, device=pred.device, dtype=pred.dtype)
    if method in ["kernel", "sort"]:
        return kcrps(pred, obs, dim=dim)
    pred = torch.movedim(pred, dim, 0)
    bin_edges, c = cdf_function(pred, bins=max(int(np.sqrt(n)), 100))
    return _crps_from_cdf(bin_edges, c, obs)
