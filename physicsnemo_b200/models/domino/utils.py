"""Array helpers of the DoMINO workflow: scaling, sampling, padding, encodings, grids.

Parity: ``physicsnemo/models/domino/utils/utils.py`` (``calculate_center_of_mass`` ``:34`` …
``sample_points_on_mesh`` ``:1037``).  The scaling / grid / centre-of-mass / ``shuffle_array``
functions are the ones the DoMINO data pipe of this package uses; the rest complete the reference's
utility set for training and inference scripts.  The VTK readers of ``vtk_file_utils.py`` need
``vtk`` / ``pyvista`` (not installed); meshes enter through ``physicsnemo_b200.mesh.io`` instead.
"""
from __future__ import annotations

from pathlib import Path
from typing import Any, Optional, Sequence

import torch

from ...datapipes.cae.domino_datapipe import (calculate_center_of_mass, create_grid, shuffle_array, unnormalize,
                                              unstandardize)
from ...nn.functional import knn
from ...nn.functional.weighted_multinomial import weighted_multinomial

__all__ = ["calculate_center_of_mass", "normalize", "unnormalize", "standardize", "unstandardize",
           "calculate_normal_positional_encoding", "nd_interpolator", "pad", "pad_inp", "shuffle_array",
           "shuffle_array_without_sampling", "create_directory", "get_filenames", "calculate_pos_encoding", "combine_dict",
           "create_grid", "mean_std_sampling", "dict_to_device", "area_weighted_shuffle_array",
           "solution_weighted_shuffle_array", "sample_points_on_mesh"]


def normalize(field: torch.Tensor, max_val=None, min_val=None) -> torch.Tensor:
    """Map ``[min, max]`` to ``[-1, 1]``; missing bounds are taken per column from the data."""
    hi = field.amax(dim=0, keepdim=True) if max_val is None else max_val
    lo = field.amin(dim=0, keepdim=True) if min_val is None else min_val
    return 2.0 * (field - lo) / (hi - lo) - 1.0


def standardize(field: torch.Tensor, mean=None, std=None) -> torch.Tensor:
    """Zero mean, unit deviation per column; missing statistics are taken from the data."""
    mu = field.mean(dim=0, keepdim=True) if mean is None else mean
    sd = field.std(dim=0, keepdim=True) if std is None else std
    return (field - mu) / sd


def calculate_pos_encoding(nx: torch.Tensor, d: int = 8) -> list:
    """``[sin(x / 10000^{2k/d}), cos(x / 10000^{2k/d})]`` for ``k < d / 2``, as a flat list of tensors."""
    out = []
    for k in range(d // 2):
        scaled = nx / 10000 ** (2 * k / d)
        out += [scaled.sin(), scaled.cos()]
    return out


def calculate_normal_positional_encoding(coordinates_a: torch.Tensor, coordinates_b: Optional[torch.Tensor] = None,
                                         cell_dimensions: Sequence[float] = (1.0, 1.0, 1.0)) -> torch.Tensor:
    """Four-term sinusoidal encoding of each component of ``a`` (or ``a − b``) in cell units.

    The twelve encoded columns are concatenated axis by axis and then reinterpreted as ``(-1, 12)``
    rows, which is the (row-mixing) layout the reference's checkpoints were trained with.
    """
    v = coordinates_a if coordinates_b is None else coordinates_a - coordinates_b
    per_axis = [torch.cat(calculate_pos_encoding(v[:, a] / float(cell_dimensions[a]), d=4), dim=-1) for a in range(3)]
    return torch.cat(per_axis, dim=0).reshape(-1, 12)


def nd_interpolator(coordinates: torch.Tensor, field: torch.Tensor, grid: torch.Tensor, k: int = 2) -> torch.Tensor:
    """Mean of the field over the ``k`` nearest samples of every grid point."""
    return field[knn(coordinates, grid, k=k)[0]].mean(dim=1)


def _pad_rows(arr: torch.Tensor, n_points: int, value: float) -> torch.Tensor:
    missing = n_points - arr.shape[0]
    if missing <= 0:
        return arr
    return torch.cat([arr, arr.new_full((missing,) + tuple(arr.shape[1:]), value)])


def pad(arr: torch.Tensor, n_points: int, pad_value: float = 0.0) -> torch.Tensor:
    """Append constant rows to a ``(n, f)`` array until it has ``n_points`` rows."""
    return _pad_rows(arr, n_points, pad_value)


def pad_inp(arr: torch.Tensor, n_points: int, pad_value: float = 0.0) -> torch.Tensor:
    """The same for ``(n, h, w)`` arrays."""
    return _pad_rows(arr, n_points, pad_value)


def shuffle_array_without_sampling(arr: torch.Tensor):
    idx = torch.randperm(arr.shape[0])
    return arr[idx], idx


def create_directory(filepath) -> None:
    Path(filepath).mkdir(parents=True, exist_ok=True)


def get_filenames(filepath, exclude_dirs: bool = False) -> list:
    """Entry names of a directory; with ``exclude_dirs`` sub-directories are dropped except ``*.zarr`` stores."""
    root = Path(filepath)
    if not root.exists():
        raise FileNotFoundError(f"Directory {filepath} does not exist")
    return [p.name for p in root.iterdir() if not (exclude_dirs and p.is_dir() and not p.name.endswith(".zarr"))]


def combine_dict(old_dict: dict, new_dict: dict) -> dict:
    """Add the values of ``new_dict`` onto the matching keys of ``old_dict`` (in place)."""
    for key in old_dict:
        old_dict[key] += new_dict[key]
    return old_dict


def mean_std_sampling(field: torch.Tensor, mean: torch.Tensor, std: torch.Tensor, tolerance: float = 3.0) -> list:
    """Row indices where some component lies more than ``tolerance`` deviations from its mean (component by component)."""
    out = []
    for v in range(field.shape[-1]):
        far = ((field[:, v] - mean[v]).abs() > tolerance * std[v]).nonzero().squeeze(1)
        out += list(far)
    return out


def dict_to_device(state_dict: dict, device: Any, exclude_keys: Optional[list] = None) -> dict:
    skip = ["filename"] if exclude_keys is None else exclude_keys
    return {k: v.to(device) for k, v in state_dict.items() if k not in skip}


def _power_weighted(arr, n_points, weight, power):
    p = weight ** power
    return shuffle_array(arr, n_points, p / p.sum())


def area_weighted_shuffle_array(arr: torch.Tensor, n_points: int, area: torch.Tensor, area_factor: float = 1.0):
    """Sample rows with probability ∝ ``area ** area_factor``."""
    return _power_weighted(arr, n_points, area, area_factor)


def solution_weighted_shuffle_array(arr: torch.Tensor, n_points: int, solution: torch.Tensor, scaling_factor: float = 1.0):
    """Sample rows with probability ∝ ``solution ** scaling_factor``."""
    return _power_weighted(arr, n_points, solution, scaling_factor)


def sample_points_on_mesh(mesh_coordinates: torch.Tensor, mesh_faces: torch.Tensor, n_points: int,
                          mesh_areas: Optional[torch.Tensor] = None, mesh_normals: Optional[torch.Tensor] = None):
    """Uniform random points on a triangle surface: ``(points, face index, face area, face normal)`` per sample.

    Faces are drawn with replacement in proportion to their area; inside a face the point is
    ``(1 − √r₁) v₀ + √r₁ (1 − r₂) v₁ + √r₁ r₂ v₂``, which is uniform over the triangle.
    """
    faces = mesh_faces.reshape(-1, 3)
    if mesh_areas is None or mesh_normals is None:
        v0, v1, v2 = (mesh_coordinates[faces[:, i]] for i in range(3))
        cross = torch.linalg.cross(v1 - v0, v2 - v0, dim=1)
        length = torch.linalg.norm(cross, dim=1)
        mesh_normals = cross / length[:, None] if mesh_normals is None else mesh_normals
        mesh_areas = 0.5 * length if mesh_areas is None else mesh_areas
    picked = weighted_multinomial(mesh_areas, n_points, replacement=True)
    r1 = torch.rand(n_points, 1, device=mesh_coordinates.device).sqrt()
    r2 = torch.rand(n_points, 1, device=mesh_coordinates.device)
    bary = torch.stack([1.0 - r1, (1.0 - r2) * r1, r2 * r1], dim=1)                     # (n, 3, 1)
    points = (mesh_coordinates[faces[picked]] * bary).sum(dim=1)
    return points, picked, mesh_areas[picked], mesh_normals[picked]
