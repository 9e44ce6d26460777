"""Shared helpers of the ShardTensor handlers."""
from __future__ import annotations

from typing import Dict, Sequence, Tuple

import torch
from torch.distributed.tensor import Partial, Replicate, Shard

from ..grad_ops import reduce_grad_over_mesh
from ..shard_tensor import MissingShardPatch, ShardTensor
from ..spec import ShardTensorSpec

NO_TF = torch._C.DisableTorchFunctionSubclass


def is_st(x) -> bool:
    return isinstance(x, ShardTensor)


def local(x):
    return x._local_tensor if isinstance(x, ShardTensor) else x


def resolved(x: ShardTensor) -> ShardTensor:
    """``x`` with every Partial placement reduced to Replicate."""
    if x._spec.is_partial():
        return x.redistribute(placements=[Replicate() if isinstance(p, Partial) else p for p in x._spec.placements])
    return x


def param(t, mesh):
    """A replicated operand (weight / bias): gradient shares are summed over the mesh."""
    if t is None:
        return None
    if isinstance(t, ShardTensor):
        return resolved(t).full_tensor() if t._spec.sharded_tensor_dims() else resolved(t)._local_tensor
    return reduce_grad_over_mesh(t, mesh)


def wrap(local_out: torch.Tensor, mesh, placements: Sequence, sizes: Dict[int, Tuple[int, ...]]) -> ShardTensor:
    """Wrap a local result; the global shape follows from the per-rank extents."""
    gshape = list(local_out.shape)
    for md, p in enumerate(placements):
        if isinstance(p, Shard):
            gshape[p.dim] = sum(sizes[md])
    return ShardTensor(local_out, ShardTensorSpec(mesh, tuple(placements), torch.Size(gshape), local_out.dtype,
                                                  {md: tuple(s) for md, s in sizes.items()}))


def norm_dim(d: int, ndim: int) -> int:
    return d + ndim if d < 0 else d


def register(*funcs):
    def deco(handler):
        for f in funcs:
            if f is not None:
                ShardTensor.register_function_handler(f, handler)
        return handler

    return deco
