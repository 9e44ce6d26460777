"""Line and surface integrals on meshes (parity: ``physicsnemo/metrics/cae/integral.py``)."""
from typing import Dict, List, Optional, Union

import numpy as np


def line_integral(edges: np.ndarray, points: np.ndarray, field: np.ndarray) -> float:
    """Integral over the polyline ``edges`` of a scalar field, or of the tangential part of a vector field
    (values per edge)."""
    vec = points[edges[:, 1]] - points[edges[:, 0]]
    length = np.linalg.norm(vec, axis=1)
    if field.ndim == 2:
        return np.sum(np.sum(field * (vec / length[:, None]), axis=1) * length)
    return np.sum(field * length)


def surface_integral(mesh, data_type: str = "point_data",
                     array_name: Optional[Union[str, List[str]]] = None) -> Dict[str, np.ndarray]:
    """Surface integral of scalar arrays, and flux of vector arrays, of a ``pyvista.PolyData``."""
    mesh = mesh.compute_normals()
    data = getattr(mesh, data_type)
    have = list(data.keys())
    if not have:
        raise ValueError(f"No data arrays found using type: {data_type}, try switching between 'point_data' and 'cell_data'")
    if array_name is None:
        names = have
    else:
        names = list(array_name) if isinstance(array_name, (list, tuple)) else [array_name]
        if not set(names) <= set(have):
            raise ValueError(f"Requested vars not found in the provided mesh file. Choose from {have}")
    for n in names:
        arr = data[n]
        if arr.ndim == 1:
            data[f"integral_{n}"] = arr
        elif arr.ndim == 2:
            data[f"integral_{n}"] = np.sum(arr * data["Normals"], axis=1)
    total = mesh.integrate_data()
    return {f"integral_{n}": np.array(total[f"integral_{n}"]) for n in names}
