"""VTK / mesh readers (parity: ``physicsnemo/datapipes/readers/vtk.py``, ``readers/mesh.py``): a directory of
``.vtp / .vtu / .vtk / .stl`` files read through pyvista (imported on first use) into point / cell arrays."""
from __future__ import annotations

from pathlib import Path
from typing import Any, Optional

import numpy as np
import torch

from ..registry import register
from .base import Reader

_SUFFIXES = (".vtp", ".vtu", ".vtk", ".stl", ".vtm", ".obj", ".ply")


def _pyvista():
    try:
        import pyvista as pv
    except ImportError as e:  # pragma: no cover
        raise ImportError("VTKReader / MeshReader require pyvista (`pip install pyvista`).") from e
    return pv


@register()
class VTKReader(Reader):
    def __init__(self, path: str | Path, *, keys_to_read: Optional[list[str]] = None, file_pattern: str = "*",
                 exclude_patterns: Optional[list[str]] = None, pin_memory: bool = False,
                 include_index_in_metadata: bool = True) -> None:
        super().__init__(pin_memory=pin_memory, include_index_in_metadata=include_index_in_metadata)
        self.path = Path(path).expanduser().resolve()
        if not self.path.exists():
            raise FileNotFoundError(f"Path not found: {self.path}")
        files = [self.path] if self.path.is_file() else sorted(p for p in self.path.rglob(file_pattern) if p.suffix in _SUFFIXES)
        for pat in exclude_patterns or []:
            files = [f for f in files if pat not in f.name]
        if not files:
            raise ValueError(f"No mesh files found in {self.path}")
        self._files, self.keys_to_read = files, keys_to_read

    def _load_sample(self, index: int) -> dict[str, torch.Tensor]:
        mesh = _pyvista().read(str(self._files[index]))
        out = {"points": torch.from_numpy(np.asarray(mesh.points, dtype=np.float32))}
        if hasattr(mesh, "faces") and mesh.n_cells and mesh.is_all_triangles:
            out["faces"] = torch.from_numpy(np.asarray(mesh.faces).reshape(-1, 4)[:, 1:].astype(np.int64))
        for store, prefix in ((mesh.point_data, "point_data"), (mesh.cell_data, "cell_data")):
            for name in store.keys():
                if self.keys_to_read is None or name in self.keys_to_read:
                    out[f"{prefix}.{name}"] = torch.from_numpy(np.asarray(store[name]))
        return out

    def __len__(self) -> int:
        return len(self._files)

    def _get_sample_metadata(self, index: int) -> dict[str, Any]:
        return {"source_file": str(self._files[index]), "source_filename": self._files[index].name}


@register()
class MeshReader(VTKReader):
    """Returns ``physicsnemo_b200.mesh.Mesh`` objects (points, cells and data) instead of flat arrays."""

    def __getitem__(self, index: int):
        data, meta = super().__getitem__(index)
        from ...mesh import Mesh

        point_data = {k.split(".", 1)[1]: v for k, v in data.items() if k.startswith("point_data.")}
        cell_data = {k.split(".", 1)[1]: v for k, v in data.items() if k.startswith("cell_data.")}
        cells = data["faces"] if "faces" in data.keys() else torch.empty(0, 3, dtype=torch.long)
        return Mesh(points=data["points"], cells=cells, point_data=point_data, cell_data=cell_data), meta


@register()
class DomainMeshReader(MeshReader):
    """Reader of multi-block cases: one directory per sample holding ``interior`` and boundary meshes."""
