"""Placement changes of a ``ShardTensor``.

Parity: ``physicsnemo/domain_parallel/_shard_redistribute.py`` — cases Partial→Replicate
(all-reduce), Shard→Replicate (all-gather-v without pad-to-max slicing on the result),
Replicate→Shard (local slice), Shard(i)→Shard(j) (one uneven all-to-all), Partial→Shard
(reduce then slice), Replicate→Partial (rank 0 keeps the value, others zero).  Each case is a
differentiable collective on the local shard (``collectives.py``).
"""
from __future__ import annotations

from typing import Tuple

import torch
import torch.distributed as dist
from torch.distributed.tensor import Partial, Replicate, Shard

from . import collectives as C
from .spec import ShardTensorSpec, chunk_sizes, mesh_coordinate


def redistribute_shard_tensor(st, target: Tuple):
    from .shard_tensor import ShardTensor

    spec: ShardTensorSpec = st._spec
    mesh = spec.mesh
    if len(target) != mesh.ndim:
        raise ValueError(f"need {mesh.ndim} placements, got {len(target)}")
    local = st._local_tensor
    placements = list(spec.placements)
    sizes = dict(spec.sharding_sizes)
    for md in range(mesh.ndim):
        cur, tgt = placements[md], target[md]
        if cur == tgt:
            continue
        group = mesh.get_group(md)
        n = mesh.size(md)
        coord = mesh_coordinate(mesh, md)
        if isinstance(cur, Partial):
            local = C.AllReduceSum.apply(local, group)
            cur = Replicate()
        if isinstance(cur, Shard) and isinstance(tgt, Shard):
            dst_sizes = chunk_sizes(spec.global_shape[tgt.dim], n)
            local = C.AllToAllDims.apply(local, cur.dim, tgt.dim, sizes[md], dst_sizes, group)
            sizes[md] = dst_sizes
            cur = tgt
        elif isinstance(cur, Shard):
            local = C.AllGatherV.apply(local, sizes[md], cur.dim, group)
            sizes.pop(md)
            cur = Replicate()
        if isinstance(cur, Replicate) and isinstance(tgt, Shard):
            dst_sizes = chunk_sizes(spec.global_shape[tgt.dim], n)
            start = sum(dst_sizes[:coord])
            local = C.SliceLocal.apply(local, start, dst_sizes[coord], tgt.dim)
            sizes[md] = dst_sizes
        elif isinstance(cur, Replicate) and isinstance(tgt, Partial):
            if coord != 0:
                local = local * 0
        placements[md] = tgt
    new_spec = ShardTensorSpec(mesh=mesh, placements=tuple(placements), global_shape=spec.global_shape,
                               dtype=local.dtype, sharding_sizes=sizes)
    return ShardTensor(local, new_spec)
