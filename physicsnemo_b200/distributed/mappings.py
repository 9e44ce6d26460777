"""Tensor-parallel region mappings (Megatron style), groups looked up by name.

Parity: ``physicsnemo/distributed/mappings.py:27-138`` (four autograd functions ``copy_to`` / ``reduce_from`` /
``scatter_to`` / ``gather_from`` a parallel region).  Here the four are ONE autograd function that is handed the name
of its forward operation and of its backward operation out of {keep, sum, local chunk, gather}: every mapping is a pair
of mutually adjoint operations on the region's process group.
"""
from typing import Optional, Sequence

import torch

from . import utils as _u
from .manager import DistributedManager


class _Region:
    """The process group behind a region name and the tensor operations the mappings are made of."""

    def __init__(self, name: str):
        manager = DistributedManager()
        self.group = manager.group(name)
        self.size = manager.group_size(name)

    def keep(self, t: torch.Tensor, dim, shapes) -> torch.Tensor:
        return t

    def total(self, t: torch.Tensor, dim, shapes) -> torch.Tensor:
        return _u._reduce(t, group=self.group)

    def local_chunk(self, t: torch.Tensor, dim, shapes) -> torch.Tensor:
        return _u._split(t, dim, group=self.group)

    def gathered(self, t: torch.Tensor, dim, shapes) -> torch.Tensor:
        return _u.all_gather_v_wrapper(t, shapes, dim, group=self.group)


class _RegionMap(torch.autograd.Function):
    """``forward`` applies operation ``fwd`` of the region, ``backward`` applies ``bwd`` to the incoming gradient."""

    @staticmethod
    def forward(ctx, tensor, fwd: str, bwd: str, region: str, dim: Optional[int], shapes: Optional[Sequence[int]]):
        where = _Region(region)
        if dim is not None and shapes is None:            # chunk sizes along ``dim`` of the tensor that gets split
            shapes = _u.compute_split_shapes(tensor.shape[dim], where.size)
        ctx.plan = (bwd, region, dim, shapes)
        return getattr(where, fwd)(tensor, dim, shapes)

    @staticmethod
    def backward(ctx, grad):
        op, region, dim, shapes = ctx.plan
        return (getattr(_Region(region), op)(grad, dim, shapes),) + (None,) * 5


def copy_to_parallel_region(input, group):
    """Identity into the region; the gradients of the region's ranks are summed on the way back."""
    return _RegionMap.apply(input, "keep", "total", group, None, None)


def reduce_from_parallel_region(input, group):
    """Sum over the region's ranks; the gradient passes unchanged."""
    return _RegionMap.apply(input, "total", "keep", group, None, None)


def scatter_to_parallel_region(input, dim, group):
    """This rank's chunk of ``input`` along ``dim``; the gradient chunks are gathered back."""
    return _RegionMap.apply(input, "local_chunk", "gathered", group, dim, None)


def gather_from_parallel_region(input, dim, shapes, group):
    """All ranks' chunks (sizes ``shapes`` along ``dim``) concatenated; the gradient keeps this rank's chunk."""
    return _RegionMap.apply(input, "gathered", "local_chunk", group, dim, shapes)
