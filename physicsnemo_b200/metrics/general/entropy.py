"""Entropy of binned distributions (parity: ``physicsnemo/metrics/general/entropy.py``)."""
import math

import torch
from torch import Tensor


def _check(p: Tensor, bin_edges: Tensor) -> None:
    if bin_edges.shape[1:] != p.shape[1:]:
        raise ValueError(f"Expected bins and pdf to have compatible non-zeroth dimensions but have shapes {bin_edges.shape[1:]} and {p.shape[1:]}.")
    if bin_edges.shape[0] != p.shape[0] + 1:
        raise ValueError(f"Expected zeroth dimension of cdf to be equal to the zeroth dimension of bins + 1 but have shapes {bin_edges.shape[0]} and {p.shape[0]}+1.")


def _density(p: Tensor, mids: Tensor) -> Tensor:
    return p / torch.trapz(p, mids, dim=0) + 1e-8


def entropy_from_counts(p: Tensor, bin_edges: Tensor, normalized: bool = True) -> Tensor:
    """Differential entropy of a histogram; ``normalized`` maps [delta-like, uniform] to [0, 1]."""
    _check(p, bin_edges)
    mids = 0.5 * (bin_edges[1:] + bin_edges[:-1])
    d = _density(p, mids)
    ent = torch.trapz(-d * torch.log(d), mids, dim=0)
    if not normalized:
        return ent
    width = bin_edges[1] - bin_edges[0]
    hi = torch.log(bin_edges[-1] - bin_edges[0])
    lo = 0.5 + 0.5 * torch.log(2 * math.pi * width ** 2)
    return (ent - lo) / (hi - lo)


def relative_entropy_from_counts(p: Tensor, q: Tensor, bin_edges: Tensor) -> Tensor:
    """KL(p ‖ q) of two histograms on the same bins."""
    _check(p, bin_edges)
    if p.shape != q.shape:
        raise ValueError(f"Expected p and q to have compatible shapes but have shapes {p.shape} and {q.shape}.")
    mids = 0.5 * (bin_edges[1:] + bin_edges[:-1])
    dp, dq = _density(p, mids), _density(q, mids)
    return torch.trapz(dp * torch.log(dp / dq), mids, dim=0)
