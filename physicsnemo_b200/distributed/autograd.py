"""Differentiable variable-size collectives.

Parity: ``physicsnemo/distributed/autograd.py`` — ``AllGatherVAutograd`` (``:33-80``),
``GatherVAutograd`` (``:83-131``), ``ScatterVAutograd`` (``:134-181``), ``IndexedAllToAllVAutograd``
(``:184-247``) and the functions ``all_gather_v``, ``gather_v``, ``scatter_v``,
``indexed_all_to_all_v`` (``:250-430``).
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from .utils import (
    all_gather_v_bwd_wrapper,
    all_gather_v_wrapper,
    gather_v_wrapper,
    indexed_all_to_all_v_wrapper,
    indexed_all_to_all_v_wrapper_bwd,
    scatter_v_wrapper,
)


class AllGatherVAutograd(torch.autograd.Function):
    """all-gather-v forward; backward sums the incoming gradient slices (reduce-scatter-v)."""

    @staticmethod
    def forward(ctx, tensor, sizes, dim=0, use_fp32=True, group=None):
        ctx.sizes, ctx.group, ctx.dim, ctx.use_fp32 = sizes, group, dim, use_fp32
        return all_gather_v_wrapper(tensor, sizes, dim=dim, group=group)

    @staticmethod
    def backward(ctx, grad_output):
        grad = None
        if ctx.needs_input_grad[0]:
            grad = all_gather_v_bwd_wrapper(grad_output, ctx.sizes, dim=ctx.dim, use_fp32=ctx.use_fp32, group=ctx.group)
        return grad, None, None, None, None


class GatherVAutograd(torch.autograd.Function):
    """gather-v forward; backward scatters the gradient back from ``dst``."""

    @staticmethod
    def forward(ctx, tensor, sizes, dim=0, dst=0, group=None):
        ctx.sizes, ctx.dim, ctx.src, ctx.group = sizes, dim, dst, group
        return gather_v_wrapper(tensor, sizes, dim=dim, dst=dst, group=group)

    @staticmethod
    def backward(ctx, grad_output):
        grad = scatter_v_wrapper(grad_output, ctx.sizes, dim=ctx.dim, src=ctx.src, group=ctx.group)
        if not ctx.needs_input_grad[0]:
            grad = None
        return grad, None, None, None, None


class ScatterVAutograd(torch.autograd.Function):
    """scatter-v forward; backward gathers the gradient on ``src``."""

    @staticmethod
    def forward(ctx, tensor, sizes, dim=0, src=0, group=None):
        ctx.tensor_shape = list(tensor.shape) if dist.get_rank(group=group) == src else None
        ctx.sizes, ctx.dim, ctx.dst, ctx.group = sizes, dim, src, group
        return scatter_v_wrapper(tensor, sizes, dim=dim, src=src, group=group)

    @staticmethod
    def backward(ctx, grad_output):
        grad = gather_v_wrapper(grad_output, ctx.sizes, dim=ctx.dim, dst=ctx.dst, group=ctx.group)
        if not ctx.needs_input_grad[0]:
            grad = None
        return grad, None, None, None, None


class IndexedAllToAllVAutograd(torch.autograd.Function):
    """indexed all-to-all-v forward; backward returns pieces to senders and ``index_add``s them."""

    @staticmethod
    def forward(ctx, tensor, indices, sizes, use_fp32=True, dim=0, group=None):
        ctx.sizes, ctx.use_fp32, ctx.group, ctx.dim = sizes, use_fp32, group, dim
        ctx.tensor_size_along_dim = tensor.size(dim)
        ctx.indices = indices
        return indexed_all_to_all_v_wrapper(tensor, indices, sizes, dim=dim, group=group)

    @staticmethod
    def backward(ctx, grad_output):
        grad = None
        if ctx.needs_input_grad[0]:
            grad = indexed_all_to_all_v_wrapper_bwd(
                grad_output, ctx.indices, ctx.sizes, tensor_size_along_dim=ctx.tensor_size_along_dim,
                use_fp32=ctx.use_fp32, dim=ctx.dim, group=ctx.group,
            )
        return grad, None, None, None, None, None


def all_gather_v(tensor: torch.Tensor, sizes: List[int], dim: int = 0, use_fp32: bool = True,
                 group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Differentiable all-gather of per-rank slices of different length along ``dim``."""
    return AllGatherVAutograd.apply(tensor, sizes, dim, use_fp32, group)


def gather_v(tensor: torch.Tensor, sizes: List[int], dim: int = 0, dst: int = 0,
             group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Differentiable gather-v onto rank ``dst``."""
    return GatherVAutograd.apply(tensor, sizes, dim, dst, group)


def scatter_v(tensor: torch.Tensor, sizes: List[int], dim: int = 0, src: int = 0,
              group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Differentiable scatter-v from rank ``src``."""
    return ScatterVAutograd.apply(tensor, sizes, dim, src, group)


def indexed_all_to_all_v(tensor: torch.Tensor, indices: List[torch.Tensor], sizes: List[List[int]],
                         use_fp32: bool = True, dim: int = 0,
                         group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Differentiable indexed all-to-all-v (the halo gather of partitioned graphs)."""
    return IndexedAllToAllVAutograd.apply(tensor, indices, sizes, use_fp32, dim, group)
