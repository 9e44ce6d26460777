"""Time <-> space resharding of ``[B, T, X, C]`` activations across a model-parallel group.

Counterpart of ``physicsnemo/experimental/models/healda/sharding.py`` (``shard_x`` :38, ``shard_t`` :73 and the
``ShardTensor`` variants :110-:139).  Temporal attention needs every time step of a pixel on one rank (space sharded);
spatial layers need every pixel of a time step (time sharded).  Both moves are one differentiable all-to-all whose
send buffer is laid out rank-major, so NCCL moves contiguous slabs over NVLink.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
from torch.distributed.nn.functional import all_to_all_single

__all__ = ["shard_x", "shard_t", "shard_x_shardtensor", "shard_t_shardtensor", "DATA_DIM", "MODEL_DIM"]

DATA_DIM = 0
MODEL_DIM = 1


def _exchange(slabs: torch.Tensor, group) -> torch.Tensor:
    """``slabs[r]`` goes to rank ``r``; returns the slabs received, ordered by source rank."""
    slabs = slabs.contiguous()
    return all_to_all_single(torch.empty_like(slabs), slabs, group=group)


def shard_x(tensor: torch.Tensor, group) -> torch.Tensor:
    """From time-sharded ``[B, T/n, X, C]`` to space-sharded ``[B, T, X/n, C]``."""
    n = dist.get_world_size(group)
    B, t, X, C = tensor.shape
    got = _exchange(tensor.view(B, t, n, X // n, C).permute(2, 0, 1, 3, 4), group)          # [n, B, t, X/n, C]
    return got.permute(1, 0, 2, 3, 4).reshape(B, n * t, X // n, C)


def shard_t(tensor: torch.Tensor, group) -> torch.Tensor:
    """From space-sharded ``[B, T, X/n, C]`` to time-sharded ``[B, T/n, X, C]``."""
    n = dist.get_world_size(group)
    B, T, x, C = tensor.shape
    got = _exchange(tensor.view(B, n, T // n, x, C).permute(1, 0, 2, 3, 4), group)          # [n, B, T/n, X/n, C]
    return got.permute(1, 2, 0, 3, 4).reshape(B, T // n, n * x, C)


def _reshard(tensor: torch.Tensor, mesh, from_dim: int, to_dim: int) -> torch.Tensor:
    from torch.distributed.tensor.placement_types import Shard

    from ....domain_parallel import ShardTensor

    return ShardTensor.from_local(tensor, mesh, [Shard(from_dim)]).redistribute(placements=[Shard(to_dim)]).to_local()


def shard_x_shardtensor(tensor: torch.Tensor, mesh) -> torch.Tensor:
    """``shard_x`` expressed as a ``ShardTensor`` redistribution over a 1-D mesh."""
    return _reshard(tensor, mesh, 1, 2)


def shard_t_shardtensor(tensor: torch.Tensor, mesh) -> torch.Tensor:
    """``shard_t`` expressed as a ``ShardTensor`` redistribution over a 1-D mesh."""
    return _reshard(tensor, mesh, 2, 1)
