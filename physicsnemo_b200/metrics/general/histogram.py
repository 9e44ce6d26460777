"""Histograms, CDFs and their streaming / distributed accumulation.

Parity: ``physicsnemo/metrics/general/histogram.py`` — ``linspace`` (tensor end points),
``histogram`` / ``cdf`` over the leading (ensemble) dimension with per-location bins, ``normal_pdf`` /
``normal_cdf``, and the ``Histogram`` accumulator (``:364-653``) whose bin edges are agreed across
ranks by MIN / MAX all-reduces and whose counts are summed.
"""
from __future__ import annotations

from typing import List, Tuple, Union

import torch
import torch.distributed as dist
from torch import Tensor


def linspace(start: Tensor, stop: Tensor, num: int) -> Tensor:
    """``num + 1`` points from ``start`` to ``stop`` (tensors of equal shape) along a new leading dim."""
    steps = torch.arange(num + 1, dtype=start.dtype, device=start.device) / num
    steps = steps.reshape(-1, *([1] * start.ndim))
    return start[None] + steps * (stop - start)[None]


@torch.jit.ignore
def _low_memory_bin_reduction_counts(inputs: Tensor, bin_edges: Tensor, counts: Tensor, number_of_bins: int) -> Tensor:
    for j in range(number_of_bins):
        hi = bin_edges[j + 1]
        lo = bin_edges[j]
        inside = (inputs >= lo[None]) & ((inputs < hi[None]) if j < number_of_bins - 1 else (inputs <= hi[None]))
        counts[j] += inside.sum(dim=0)
    return counts


def _count_bins(inputs: Tensor, bin_edges: Tensor, counts: Tensor = None, cdf: bool = False) -> Tensor:
    nb = bin_edges.shape[0] - 1
    if counts is None:
        counts = torch.zeros((nb, *inputs.shape[1:]), dtype=torch.int64, device=inputs.device)
    counts = _low_memory_bin_reduction_counts(inputs, bin_edges, counts, nb)
    return counts


def _get_mins_maxs(*inputs: Tensor, axis: int = 0) -> Tuple[Tensor, Tensor]:
    lo = inputs[0].amin(dim=axis)
    hi = inputs[0].amax(dim=axis)
    for t in inputs[1:]:
        lo, hi = torch.minimum(lo, t.amin(dim=axis)), torch.maximum(hi, t.amax(dim=axis))
    return lo, hi


def _update_bins_counts(inputs: Tensor, bin_edges: Tensor, counts: Tensor) -> Tuple[Tensor, Tensor]:
    """Extend the bin range (keeping the bin width) to cover ``inputs`` and add their counts."""
    nb = bin_edges.shape[0] - 1
    lo, hi = _get_mins_maxs(inputs)
    width = bin_edges[1] - bin_edges[0]
    start, end = bin_edges[0], bin_edges[-1]
    left = torch.clamp(torch.ceil((start - lo) / width), min=0).amax().long().item()
    right = torch.clamp(torch.ceil((hi - end) / width), min=0).amax().long().item()
    if left or right:
        new_start = start - left * width
        new_edges = new_start[None] + torch.arange(nb + left + right + 1, device=inputs.device,
                                                   dtype=bin_edges.dtype).reshape(-1, *([1] * start.ndim)) * width[None]
        new_counts = torch.zeros((nb + left + right, *counts.shape[1:]), dtype=counts.dtype, device=counts.device)
        new_counts[left:left + nb] = counts
        bin_edges, counts = new_edges, new_counts
    counts = _count_bins(inputs, bin_edges, counts)
    return bin_edges, counts


def _compute_counts_cdf(*inputs: Tensor, bins: Union[int, Tensor] = 10, counts: Tensor = None, cdf: bool = False):
    if isinstance(bins, int):
        lo, hi = _get_mins_maxs(*inputs)
        same = hi == lo
        hi = torch.where(same, hi + 0.5, hi)
        lo = torch.where(same, lo - 0.5, lo)
        bin_edges = linspace(lo, hi, bins)
    else:
        bin_edges = bins
    for t in inputs:
        counts = _count_bins(t, bin_edges, counts)
    if cdf:
        c = torch.cumsum(counts, dim=0).to(inputs[0].dtype)
        return bin_edges, c / c[-1].clamp_min(1)
    return bin_edges, counts


def histogram(*inputs: Tensor, bins: Union[int, Tensor] = 10, counts: Tensor = None, verbose: bool = False):
    """Counts of the values along dim 0 in ``bins`` bins per location: ``(bin_edges, counts)``."""
    return _compute_counts_cdf(*inputs, bins=bins, counts=counts, cdf=False)


def cdf(*inputs: Tensor, bins: Union[int, Tensor] = 10, counts: Tensor = None, verbose: bool = False):
    """Empirical CDF of the values along dim 0: ``(bin_edges, cdf)``."""
    return _compute_counts_cdf(*inputs, bins=bins, counts=counts, cdf=True)


def normal_pdf(mean: Tensor, std: Tensor, bin_edges: Tensor, grid: str = "midpoint") -> Tensor:
    pts = _grid(bin_edges, grid)
    return torch.exp(-0.5 * ((pts - mean[None]) / std[None]) ** 2) / (std[None] * (2 * torch.pi) ** 0.5)


def normal_cdf(mean: Tensor, std: Tensor, bin_edges: Tensor, grid: str = "midpoint") -> Tensor:
    pts = _grid(bin_edges, grid)
    return 0.5 * (1 + torch.erf((pts - mean[None]) / (std[None] * 2 ** 0.5)))


def _grid(bin_edges: Tensor, grid: str) -> Tensor:
    if grid == "midpoint":
        return 0.5 * (bin_edges[1:] + bin_edges[:-1])
    if grid == "left":
        return bin_edges[:-1]
    if grid == "right":
        return bin_edges[1:]
    raise ValueError("This type of grid is not defined. Choose one of {'midpoint', 'left', 'right'}.")


class Histogram:
    """Streaming histogram over batches (and ranks): ``__call__`` starts it, ``update`` extends it,
    ``finalize(cdf=False)`` returns ``(bin_edges, pdf or cdf)``."""

    def __init__(self, input_shape, bins: Union[int, Tensor] = 10, tol: float = 1e-2, device="cpu",
                 dtype=torch.float32):
        self.input_shape = tuple(input_shape)
        self.device, self.dtype, self.tol = torch.device(device), dtype, tol
        if isinstance(bins, int):
            self.number_of_bins = bins
            self.bin_edges = None
        else:
            self.number_of_bins = bins.shape[0] - 1
            self.bin_edges = bins.to(self.device)
        self.counts = torch.zeros((self.number_of_bins, *self.input_shape), dtype=torch.int64, device=self.device)

    def _distributed(self) -> bool:
        return dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1

    def __call__(self, inputs: Tensor):
        if self.bin_edges is None:
            lo, hi = _get_mins_maxs(inputs)
            if self._distributed():
                dist.all_reduce(lo, op=dist.ReduceOp.MIN)
                dist.all_reduce(hi, op=dist.ReduceOp.MAX)
            same = hi == lo
            self.bin_edges = linspace(torch.where(same, lo - 0.5, lo), torch.where(same, hi + 0.5, hi), self.number_of_bins)
        self.counts = torch.zeros((self.bin_edges.shape[0] - 1, *self.input_shape), dtype=torch.int64, device=self.device)
        self.counts = _count_bins(inputs, self.bin_edges, self.counts)
        if self._distributed():
            dist.all_reduce(self.counts, op=dist.ReduceOp.SUM)
        self.number_of_bins = self.bin_edges.shape[0] - 1
        return self.bin_edges, self.counts

    def update(self, inputs: Tensor):
        if self.bin_edges is None:
            return self(inputs)
        if self._distributed():
            lo, hi = _get_mins_maxs(inputs)
            dist.all_reduce(lo, op=dist.ReduceOp.MIN)
            dist.all_reduce(hi, op=dist.ReduceOp.MAX)
            probe = torch.stack([lo, hi])
            edges, counts = _update_bins_counts(probe, self.bin_edges, self.counts)
            counts = counts - _count_bins(probe, edges)  # the probe only widens the range
            local = _count_bins(inputs, edges)
            dist.all_reduce(local, op=dist.ReduceOp.SUM)
            self.bin_edges, self.counts = edges, counts + local
        else:
            self.bin_edges, self.counts = _update_bins_counts(inputs, self.bin_edges, self.counts)
        self.number_of_bins = self.bin_edges.shape[0] - 1
        return self.bin_edges, self.counts

    def finalize(self, cdf: bool = False):
        total = self.counts.sum(dim=0).clamp_min(1)
        if cdf:
            return self.bin_edges, torch.cumsum(self.counts, dim=0).to(self.dtype) / total
        width = self.bin_edges[1] - self.bin_edges[0]
        return self.bin_edges, self.counts.to(self.dtype) / (total * width)
