"""Wasserstein distances (parity: ``physicsnemo/metrics/general/wasserstein.py``)."""
from warnings import warn

import torch
from torch import Tensor

from . import histogram


def _psd_sqrt(m: Tensor) -> Tensor:
    vals, vecs = torch.linalg.eigh(m)
    if torch.any(vals < 0.0):
        warn("Warning! Some eigenvalues are less than zero and matrix is not positive definite.")
        vals = vals.clamp_min(0.0)
    return (vecs * vals.sqrt().unsqueeze(-2)) @ vecs.transpose(-2, -1)


def wasserstein_from_normal(mu0: Tensor, sigma0: Tensor, mu1: Tensor, sigma1: Tensor) -> Tensor:
    """Squared 2-Wasserstein distance of two Gaussians (variances, or covariance matrices in the last two dims)."""
    if sigma0.ndim == mu0.ndim:
        return (mu0 - mu1) ** 2 + (sigma0 + sigma1 - 2 * torch.sqrt(sigma0 * sigma1))
    root0 = _psd_sqrt(sigma0)
    cross = _psd_sqrt(root0 @ sigma1 @ root0)
    tr = torch.diagonal(sigma0 + sigma1 - 2 * cross, dim1=-2, dim2=-1).sum(-1)
    return torch.linalg.vector_norm(mu0 - mu1, dim=-1) ** 2 + tr


def wasserstein_from_cdf(bin_edges: Tensor, cdf_x: Tensor, cdf_y: Tensor) -> Tensor:
    return torch.sum(torch.abs(cdf_x - cdf_y) * (bin_edges[1] - bin_edges[0]), dim=0)


def wasserstein_from_samples(x: Tensor, y: Tensor, bins: int = 10) -> Tensor:
    """1-Wasserstein distance of two sample sets along dim 0, from their binned CDFs."""
    edges, cx = histogram.cdf(x, bins=bins)
    _, cy = histogram.cdf(y, bins=edges)
    return wasserstein_from_cdf(edges, cx, cy)
