"""``DomainMesh``: an interior (volume) mesh together with named boundary meshes and domain-level data
(parity: ``physicsnemo/mesh/domain_mesh.py``)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .mesh import Mesh


class DomainMesh:
    def __init__(self, interior: Mesh, boundaries: Optional[Dict[str, Mesh]] = None,
                 global_data: Optional[Dict[str, torch.Tensor]] = None) -> None:
        self.interior = interior
        self.boundaries: Dict[str, Mesh] = dict(boundaries or {})
        self.global_data = {k: torch.as_tensor(v) for k, v in dict(global_data or {}).items()}
        for name, b in self.boundaries.items():
            if b.n_spatial_dims != interior.n_spatial_dims:
                raise ValueError(f"boundary '{name}' has spatial dimension {b.n_spatial_dims}, interior has {interior.n_spatial_dims}")

    @classmethod
    def from_interior(cls, interior: Mesh, name: str = "boundary") -> "DomainMesh":
        return cls(interior, {name: interior.get_boundary_mesh()})

    @property
    def boundary_names(self):
        return list(self.boundaries)

    def to(self, *args, **kw) -> "DomainMesh":
        return DomainMesh(self.interior.to(*args, **kw), {k: v.to(*args, **kw) for k, v in self.boundaries.items()},
                          {k: v.to(*args, **kw) for k, v in self.global_data.items()})

    def merged_boundary(self) -> Mesh:
        return Mesh.merge(list(self.boundaries.values()))

    def split_boundary(self, name: str, predicate, new_names=("selected", "rest")) -> "DomainMesh":
        """Split one boundary by a predicate on its cell centroids (e.g. inlet / wall selection)."""
        b = self.boundaries[name]
        mask = predicate(b.cell_centroids)
        rest = {k: v for k, v in self.boundaries.items() if k != name}
        rest[new_names[0]], rest[new_names[1]] = b.slice_cells(mask), b.slice_cells(~mask)
        return DomainMesh(self.interior, rest, self.global_data)

    def statistics(self):
        return {"interior": self.interior.statistics, **{f"boundary/{k}": v.statistics for k, v in self.boundaries.items()}}

    def __repr__(self) -> str:
        return f"DomainMesh(interior={self.interior!r}, boundaries={ {k: v.n_cells for k, v in self.boundaries.items()} })"
