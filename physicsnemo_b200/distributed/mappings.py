"""Tensor-parallel region mappings (Megatron style), groups looked up by name.

Parity: ``physicsnemo/distributed/mappings.py:27-138``.
"""
import torch

from .manager import DistributedManager
from .utils import _reduce, _split, all_gather_v_wrapper, compute_split_shapes


class _CopyToParallelRegion(torch.autograd.Function):
    """Identity forward, all-reduce backward."""

    @staticmethod
    def forward(ctx, input_, group_):
        ctx.group = group_
        return input_

    @staticmethod
    def backward(ctx, grad_output):
        return _reduce(grad_output, group=DistributedManager().group(ctx.group)), None


class _ReduceFromParallelRegion(torch.autograd.Function):
    """All-reduce forward, identity backward."""

    @staticmethod
    def forward(ctx, input_, group_):
        return _reduce(input_, group=DistributedManager().group(group_))

    @staticmethod
    def backward(ctx, grad_output):
        return grad_output, None


class _ScatterToParallelRegion(torch.autograd.Function):
    """Keep the local chunk forward, all-gather backward."""

    @staticmethod
    def forward(ctx, input_, dim_, group_):
        ctx.dim, ctx.group = dim_, group_
        ctx.split_shapes = compute_split_shapes(input_.shape[dim_], DistributedManager().group_size(group_))
        return _split(input_, dim_, group=DistributedManager().group(group_))

    @staticmethod
    def backward(ctx, grad_output):
        return (all_gather_v_wrapper(grad_output, ctx.split_shapes, ctx.dim, group=DistributedManager().group(ctx.group)),
                None, None)


class _GatherFromParallelRegion(torch.autograd.Function):
    """All-gather forward, keep the local chunk backward."""

    @staticmethod
    def forward(ctx, input_, dim_, shapes_, group_):
        ctx.dim, ctx.group = dim_, group_
        return all_gather_v_wrapper(input_, shapes_, dim_, group=DistributedManager().group(group_))

    @staticmethod
    def backward(ctx, grad_output):
        return _split(grad_output, ctx.dim, group=DistributedManager().group(ctx.group)), None, None, None


def copy_to_parallel_region(input, group):
    return _CopyToParallelRegion.apply(input, group)


def reduce_from_parallel_region(input, group):
    return _ReduceFromParallelRegion.apply(input, group)


def scatter_to_parallel_region(input, dim, group):
    return _ScatterToParallelRegion.apply(input, dim, group)


def gather_from_parallel_region(input, dim, shapes, group):
    return _GatherFromParallelRegion.apply(input, dim, shapes, group)
