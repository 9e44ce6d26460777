"""Extreme forecast index and normalised entropy (parity: ``physicsnemo/metrics/climate/efi.py``)."""
import math

import torch
from torch import Tensor

from ..general.entropy import entropy_from_counts
from ..general.histogram import normal_cdf


def _efi_integral(reference_cdf: Tensor, pred_cdf: Tensor) -> Tensor:
    kernel = (reference_cdf - pred_cdf) / torch.sqrt(1e-8 + reference_cdf * (1.0 - reference_cdf))
    return 2.0 / math.pi * torch.trapz(kernel, reference_cdf, dim=0)


def efi_gaussian(pred_cdf: Tensor, bin_edges: Tensor, climatology_mean: Tensor, climatology_std: Tensor) -> Tensor:
    """EFI against a Gaussian climatology evaluated at the right bin edges."""
    return _efi_integral(normal_cdf(climatology_mean, climatology_std, bin_edges, grid="right"), pred_cdf)


def efi(bin_edges: Tensor, counts: Tensor, quantiles: Tensor) -> Tensor:
    """EFI of a forecast histogram against climatological ``quantiles`` given on the same bins."""
    mass = counts * (bin_edges[1:] - bin_edges[:-1])
    return _efi_integral(quantiles, torch.cumsum(mass, dim=0) / mass.sum(dim=0))


def normalized_entropy(pred_pdf: Tensor, bin_edges: Tensor, climatology_pdf: Tensor) -> Tensor:
    if pred_pdf.shape != climatology_pdf.shape:
        raise ValueError("Prediction PDF and Climatological PDF must have the same shapes"
                         f"but recieved {pred_pdf.shape} and {climatology_pdf.shape}.")
    return 1.0 - entropy_from_counts(pred_pdf, bin_edges) / entropy_from_counts(climatology_pdf, bin_edges)
