"""``ShardTensorSpec``: mesh, placements, global shape and the per-rank shard shapes.

Parity: ``physicsnemo/domain_parallel/_shard_tensor_spec.py`` — the spec carries, beyond
what DTensor records, the *actual* shape of every rank's shard along each sharded mesh
dimension (``_sharding_shapes``), so uneven shards are first-class.  Chunk sizes of an even
split follow ``compute_split_shapes`` (ceil-division chunks, floor fallback).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
from torch.distributed.device_mesh import DeviceMesh
from torch.distributed.tensor import Partial, Replicate, Shard

from ..distributed.utils import compute_split_shapes

Placement = (Shard, Replicate, Partial)


def mesh_coordinate(mesh: DeviceMesh, mesh_dim: int) -> int:
    return mesh.get_local_rank(mesh_dim)


@dataclass
class ShardTensorSpec:
    """Describes how a global tensor is laid out over ``mesh``.

    ``sharding_sizes[mesh_dim]`` lists the extent, along the tensor dimension sharded by that
    mesh dimension, of every rank of the mesh dimension (only for ``Shard`` placements).
    """

    mesh: DeviceMesh
    placements: Tuple
    global_shape: torch.Size
    dtype: torch.dtype
    sharding_sizes: Dict[int, Tuple[int, ...]] = field(default_factory=dict)

    # -------------------------------------------------------------- queries
    def shard_dim_of(self, mesh_dim: int) -> Optional[int]:
        p = self.placements[mesh_dim]
        return p.dim if isinstance(p, Shard) else None

    def mesh_dim_of(self, tensor_dim: int) -> Optional[int]:
        for md, p in enumerate(self.placements):
            if isinstance(p, Shard) and p.dim == tensor_dim:
                return md
        return None

    def sharded_tensor_dims(self):
        return [p.dim for p in self.placements if isinstance(p, Shard)]

    def is_partial(self) -> bool:
        return any(isinstance(p, Partial) for p in self.placements)

    def is_replicated(self) -> bool:
        return all(isinstance(p, Replicate) for p in self.placements)

    def local_shape(self) -> torch.Size:
        shape = list(self.global_shape)
        for md, p in enumerate(self.placements):
            if isinstance(p, Shard):
                shape[p.dim] = self.sharding_sizes[md][mesh_coordinate(self.mesh, md)]
        return torch.Size(shape)

    def offsets(self, mesh_dim: Optional[int] = None):
        """Start offset of this rank's shard along each sharded tensor dim (or one mesh dim)."""
        out = {}
        for md, p in enumerate(self.placements):
            if isinstance(p, Shard):
                sizes = self.sharding_sizes[md]
                out[md] = sum(sizes[: mesh_coordinate(self.mesh, md)])
        return out if mesh_dim is None else out.get(mesh_dim, 0)

    def sharding_shapes(self) -> Dict[int, Tuple[torch.Size, ...]]:
        """Full shard shapes of every rank along each sharded mesh dimension."""
        out = {}
        local = list(self.local_shape())
        for md, p in enumerate(self.placements):
            if isinstance(p, Shard):
                shapes = []
                for s in self.sharding_sizes[md]:
                    shp = list(local)
                    shp[p.dim] = s
                    shapes.append(torch.Size(shp))
                out[md] = tuple(shapes)
        return out

    # --------------------------------------------------------- construction
    def with_(self, **changes) -> "ShardTensorSpec":
        d = dict(mesh=self.mesh, placements=self.placements, global_shape=self.global_shape, dtype=self.dtype,
                 sharding_sizes=dict(self.sharding_sizes))
        d.update(changes)
        return ShardTensorSpec(**d)

    def __hash__(self):
        return hash((id(self.mesh), tuple(str(p) for p in self.placements), tuple(self.global_shape), self.dtype,
                     tuple(sorted(self.sharding_sizes.items()))))

    def _stable_hash(self) -> str:
        """Digest that is equal on every process and in every run for equal layouts (the in-process ``__hash__`` keys on
        the mesh object's identity).  Covers the mesh's shape, dimension names and device type, the placements, the
        global shape and dtype, the per-rank shard extents and this rank's local shape, so that an uneven layout and
        the even chunking of the same global shape do not collide.  Usable as a cache key across processes
        (reference: ``ShardTensorSpec._stable_hash``, ``_shard_tensor_spec.py:119``)."""
        import hashlib

        mesh = self.mesh
        parts = (tuple(mesh.mesh.shape), tuple(mesh.mesh_dim_names or ()), str(mesh.device_type),
                 tuple(repr(p) for p in self.placements), tuple(int(d) for d in self.global_shape), str(self.dtype),
                 tuple(sorted((int(k), tuple(int(x) for x in v)) for k, v in self.sharding_sizes.items())),
                 tuple(int(d) for d in self.local_shape()))
        return hashlib.sha256(repr(parts).encode()).hexdigest()

    def same_layout(self, other: "ShardTensorSpec") -> bool:
        return (self.mesh is other.mesh or self.mesh == other.mesh) and tuple(self.placements) == tuple(other.placements) \
            and self.sharding_sizes == other.sharding_sizes


def chunk_sizes(extent: int, parts: int) -> Tuple[int, ...]:
    return tuple(compute_split_shapes(extent, parts))


def infer_spec_from_local(local: torch.Tensor, mesh: DeviceMesh, placements: Sequence, sharding_shapes="infer",
                          global_shape: Optional[Sequence[int]] = None) -> ShardTensorSpec:
    """Build the spec of a tensor given this rank's shard.

    ``sharding_shapes``: ``"chunk"`` assumes the even split of ``global_shape`` (no
    communication); ``"infer"`` all-gathers the shard extents over each sharded mesh dimension;
    a dict ``{mesh_dim: (sizes or shapes per rank)}`` is taken as given.
    """
    placements = tuple(placements)
    if len(placements) != mesh.ndim:
        raise ValueError(f"need one placement per mesh dimension ({mesh.ndim}), got {len(placements)}")
    sizes: Dict[int, Tuple[int, ...]] = {}
    shape = list(local.shape)
    for md, p in enumerate(placements):
        if not isinstance(p, Shard):
            continue
        n = mesh.size(md)
        if isinstance(sharding_shapes, dict) and md in sharding_shapes:
            entry = sharding_shapes[md]
            sizes[md] = tuple(int(e[p.dim]) if not isinstance(e, int) else int(e) for e in entry)
        elif sharding_shapes == "chunk":
            if global_shape is None:
                raise ValueError('sharding_shapes="chunk" needs global_shape')
            sizes[md] = chunk_sizes(int(global_shape[p.dim]), n)
        else:  # infer by communication
            group = mesh.get_group(md)
            mine = torch.tensor([local.shape[p.dim]], dtype=torch.int64,
                                device=local.device if dist.get_backend(group) == "nccl" else "cpu")
            gathered = [torch.zeros_like(mine) for _ in range(n)]
            dist.all_gather(gathered, mine, group=group)
            sizes[md] = tuple(int(g.item()) for g in gathered)
        shape[p.dim] = sum(sizes[md])
    if global_shape is not None:
        shape = list(global_shape)
    return ShardTensorSpec(mesh=mesh, placements=placements, global_shape=torch.Size(shape), dtype=local.dtype,
                           sharding_sizes=sizes)
