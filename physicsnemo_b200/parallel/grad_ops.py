"""Gradient reduction for replicated tensors that meet sharded activations.

Parity: ``physicsnemo/domain_parallel/shard_utils/grad_ops.py`` (``GradReducer``: identity
forward, all-reduce of the gradient over every sharded mesh dimension backward).  Every plain
tensor that requires grad (a parameter, or something computed from parameters) and enters an
operation together with a ShardTensor passes through ``reduce_grad_over_mesh``.

``defer_param_grad_reduction(True)`` switches the per-use all-reduce off; the caller then sums
all parameter gradients once per step with ``reduce_param_grads`` (one flat bucket).
"""
from __future__ import annotations

from typing import Iterable

import torch
import torch.distributed as dist

from . import collectives as C

_DEFER = [False]


def defer_param_grad_reduction(flag: bool = True) -> None:
    _DEFER[0] = bool(flag)


def reduce_grad_over_mesh(t: torch.Tensor, mesh) -> torch.Tensor:
    if _DEFER[0] or not torch.is_grad_enabled() or not t.requires_grad:
        return t
    for md in range(mesh.ndim):
        if mesh.size(md) > 1:
            t = C.GradAllReduce.apply(t, mesh.get_group(md))
    return t


@torch.no_grad()
def reduce_param_grads(params: Iterable[torch.Tensor], mesh) -> None:
    """Sum ``.grad`` of ``params`` over all ranks of ``mesh`` with one flat fp32 all-reduce per mesh dim."""
    grads = [p.grad for p in params if p.grad is not None]
    if not grads:
        return
    flat = torch.cat([g.reshape(-1).float() for g in grads])
    for md in range(mesh.ndim):
        if mesh.size(md) > 1:
            dist.all_reduce(flat, group=mesh.get_group(md))
    off = 0
    for g in grads:
        n = g.numel()
        g.copy_(flat[off:off + n].reshape(g.shape))
        off += n
