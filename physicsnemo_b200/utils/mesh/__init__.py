"""Mesh file helpers (parity: ``physicsnemo/utils/mesh/generate_stl.py``; the VTK-based converters of the reference need the
``vtk`` package, which is not available here)."""
from __future__ import annotations

import numpy as np
import torch


def sdf_to_stl(field, threshold: float = 0.0, backend: str = "marching_tetrahedra", filename: str = "output_stl.stl") -> None:
    """Extract the ``threshold`` isosurface of a 3-D field and write it as a binary STL.  ``backend`` is accepted for
    compatibility; the extraction always uses ``physicsnemo_b200.mesh.generate.marching_cubes``."""
    from ...mesh.generate import marching_cubes
    from ...mesh.io import write_stl

    f = field if isinstance(field, torch.Tensor) else torch.as_tensor(np.asarray(field, dtype=np.float32))
    write_stl(marching_cubes(f, threshold), filename)


__all__ = ["sdf_to_stl"]
