"""Rank histograms and the rank probability score (parity: ``physicsnemo/metrics/general/calibration.py``)."""
from typing import Union

import numpy as np
import torch
from torch import Tensor

from .histogram import histogram, linspace


def find_rank(bin_edges: Tensor, counts: Tensor, obs: Union[Tensor, np.ndarray]) -> Tensor:
    """Fraction of the histogram mass at or below the observation."""
    if isinstance(obs, np.ndarray):
        obs = torch.from_numpy(obs).to(counts.device)
    if bin_edges.shape[1:] != counts.shape[1:]:
        raise ValueError(f"Expected bins and counts to have compatible non-zeroth dimensions but have shapes {bin_edges.shape[1:]} and {counts.shape[1:]}.")
    if bin_edges.shape[1:] != obs.shape:
        raise ValueError(f"Expected bins and observations to have compatible broadcasting dimensions but have shapes {bin_edges.shape[1:]} and {obs.shape}.")
    if bin_edges.shape[0] != counts.shape[0] + 1:
        raise ValueError(f"Expected zeroth dimension of counts to be equal to the zeroth dimension of bins + 1 but have shapes {bin_edges.shape[0]} and {counts.shape[0]}+1.")
    total = counts.sum(dim=0)[0]
    mids = 0.5 * (bin_edges[1:] + bin_edges[:-1])
    return torch.sum(counts * (mids <= obs[None]), dim=0) / total


def _rank_probability_score_from_counts(rank_bin_edges: Tensor, rank_counts: Tensor) -> Tensor:
    c = torch.cumsum(rank_counts, dim=0)
    c = c / c[-1]
    upper = rank_bin_edges[1:]
    return torch.sum((c - upper) ** 2, dim=0) / torch.sum((1.0 - upper) ** 2, dim=0)


def rank_probability_score(ranks: Tensor) -> Tensor:
    """Distance of the rank CDF (10 bins on [0, 1]) from the uniform one, normalised to [0, 1]."""
    zero = torch.zeros_like(ranks[0])
    edges, counts = histogram(ranks, bins=linspace(zero, zero + 1.0, 10))
    return _rank_probability_score_from_counts(edges, counts)
