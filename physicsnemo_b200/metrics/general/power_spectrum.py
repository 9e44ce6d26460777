"""Radially binned 2-D power spectrum (parity: ``physicsnemo/metrics/general/power_spectrum.py``)."""
from typing import Tuple

import torch


def _batch_weighted_histogram(data_tensor: torch.Tensor, num_classes: int = -1, weights: torch.Tensor = None) -> torch.Tensor:
    """Per-row weighted histogram of non-negative values into ``num_classes`` equal bins of [0, max]."""
    top = data_tensor.max()
    nc = int(top + 1) if num_classes <= 0 else num_classes
    out = torch.zeros((*data_tensor.shape[:-1], nc), dtype=data_tensor.dtype, device=data_tensor.device)
    w = weights if weights is not None else torch.ones((), dtype=out.dtype, device=out.device).expand(data_tensor.shape)
    out.scatter_add_(-1, ((data_tensor * nc) // (top + 1)).long(), w)
    return out


def power_spectrum(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(k, power)``: mean of ``|FFT2(x)|²`` (ortho) over rings of the shifted wavenumber plane."""
    lead, (h, w) = x.shape[:-2], x.shape[-2:]
    x = x.reshape(-1, h, w)
    nb = x.shape[0]
    pw = torch.fft.fftshift(torch.fft.fftn(x, dim=(-2, -1), norm="ortho").abs() ** 2, dim=(-2, -1)).float()
    iy, ix = torch.meshgrid(torch.arange(h, device=x.device), torch.arange(w, device=x.device), indexing="ij")
    radius = torch.hypot(iy - h // 2, ix - w / 2).float().flatten()
    order = torch.argsort(radius)
    radius = radius[order]
    pw = pw.reshape(nb, -1)[:, order]
    nbins = min(h // 2, w // 2)
    edges = torch.linspace(0, radius.max() + 1, nbins)
    centres = 0.5 * (edges[1:] + edges[:-1])
    rr = radius.expand(nb, -1).contiguous()
    total = _batch_weighted_histogram(rr, weights=pw, num_classes=nbins - 1)
    count = _batch_weighted_histogram(rr, num_classes=nbins - 1)
    return centres, (total / count).reshape(*lead, nbins - 1)
