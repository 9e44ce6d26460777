"""Mean aggregation of observation features onto ``(batch, pixel, bucket)`` cells followed by a bucket-mixing MLP.

Counterpart of ``physicsnemo/experimental/models/healda/scatter_aggregator.py`` (``scatter_mean`` :44,
``ScatterAggregator`` :123).  Sums and counts are accumulated with one ``index_add`` each (no NaN sentinel pass).
"""

from __future__ import annotations

import math
from typing import Tuple

import torch

__all__ = ["scatter_mean", "ScatterAggregator"]


def scatter_mean(x: torch.Tensor, index: torch.Tensor, shape: Tuple[int, ...], fill_value: float = float("nan")):
    """Mean of the rows of ``x`` ``[N, C]`` per cell of a grid of ``shape``; ``index`` ``[N, len(shape)]``.

    Returns ``(mean [*shape, C] with fill_value in empty cells, present [*shape] bool)``.
    """
    strides = torch.tensor([math.prod(shape[i + 1:]) for i in range(len(shape))], device=index.device)
    flat = (index * strides).sum(dim=-1)
    cells, C = math.prod(shape), x.shape[1]
    total = torch.zeros(cells, C, dtype=x.dtype, device=x.device).index_add_(0, flat, x)
    count = torch.zeros(cells, dtype=x.dtype, device=x.device).index_add_(0, flat, torch.ones_like(flat, dtype=x.dtype))
    present = count > 0
    mean = torch.where(present[:, None], total / count.clamp(min=1)[:, None], torch.full_like(total, fill_value))
    return mean.view(*shape, C), present.view(shape)


class ScatterAggregator(torch.nn.Module):
    def __init__(self, in_dim: int, out_dim: int, nbuckets: int):
        super().__init__()
        self.in_dim, self.out_dim, self.nbuckets = in_dim, out_dim, nbuckets
        self.bucket_mixing_mlp = torch.nn.Sequential(torch.nn.Linear(nbuckets * in_dim + nbuckets, out_dim * 2), torch.nn.LayerNorm(out_dim * 2),
                                                     torch.nn.SiLU(), torch.nn.Linear(out_dim * 2, out_dim))

    def forward(self, x: torch.Tensor, batch_idx: torch.Tensor, pix: torch.Tensor, bucket_id: torch.Tensor, nbatch: int, npix: int) -> torch.Tensor:
        mean, has = scatter_mean(x, torch.stack([batch_idx, pix, bucket_id], dim=-1), (nbatch, npix, self.nbuckets), fill_value=0.0)
        return self.bucket_mixing_mlp(torch.cat([mean.view(nbatch, npix, -1), has.to(x.dtype)], dim=-1))
