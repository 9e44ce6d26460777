"""Global shape descriptors of a surface mesh for geometry out-of-distribution detection.

Counterpart of ``physicsnemo/experimental/guardrails/geometry/feature_extraction.py`` (``extract_features`` :95),
``feature_schema.py`` (``FeatureSchema`` :31) and ``mesh_validation.py`` (``validate_mesh`` :28).  Twenty-two numbers per
mesh: centroid, the two leading principal axes (sign-fixed) and the three principal variances of the vertices, the
bounding-box extents, the per-axis second moments, the total area and the areas projected on the coordinate planes.
Everything is computed with tensor operations on the device of the mesh.
"""

from __future__ import annotations

import hashlib
from typing import List, Union

import numpy as np
import torch

from ....mesh import Mesh

__all__ = ["FEATURE_NAMES", "FEATURE_VERSION", "FeatureSchema", "extract_features", "feature_hash", "validate_mesh"]

FEATURE_VERSION = "v1.0"
FEATURE_NAMES: List[str] = (
    [f"centroid_{a}" for a in "xyz"] + [f"pca_axis1_{a}" for a in "xyz"] + [f"pca_axis2_{a}" for a in "xyz"]
    + ["pca_eig1", "pca_eig2", "pca_eig3"] + [f"extent_{a}" for a in "xyz"] + [f"moment_{a}" for a in "xyz"]
    + ["total_area", "area_xy", "area_xz", "area_yz"])


def feature_hash(names: List[str]) -> str:
    h = hashlib.sha256()
    for n in names:
        h.update(n.encode("utf-8"))
    return h.hexdigest()


class FeatureSchema:
    """Names, version and hash of the descriptor vector; ``validate_array`` checks a ``[n, dim]`` feature matrix."""

    names, version, hash, dim = FEATURE_NAMES, FEATURE_VERSION, feature_hash(FEATURE_NAMES), len(FEATURE_NAMES)

    @classmethod
    def validate_array(cls, X: np.ndarray) -> None:
        if X.ndim != 2:
            raise ValueError(f"Feature array must be 2D, got {X.ndim}D array with shape {X.shape}")
        if X.shape[1] != cls.dim:
            raise ValueError(f"Feature dimension mismatch: expected {cls.dim}, got {X.shape[1]}")


def validate_mesh(mesh: Mesh, min_verts: int = 4) -> None:
    """Raise ``ValueError`` for objects that are not meshes, have too few or non-finite vertices, or no area."""
    if not isinstance(mesh, Mesh):
        raise ValueError("Object is not a physicsnemo.mesh.Mesh")
    if mesh.n_points < min_verts:
        raise ValueError(f"Too few vertices: {mesh.n_points} < {min_verts}")
    if not bool(torch.isfinite(mesh.points).all()):
        raise ValueError("Non-finite vertex coordinates")
    areas = mesh.cell_areas
    total = float(areas.sum())
    if total <= 0:
        bad = int((areas <= 0).sum())
        raise ValueError(f"Non-positive surface area: {total:.2e}. Valid cells: {mesh.n_cells - bad}/{mesh.n_cells}, "
                         f"Degenerate cells: {bad}/{mesh.n_cells}")


def extract_features(mesh: Mesh, return_tensor: bool = False, skip_validation: bool = False) -> Union[np.ndarray, torch.Tensor]:
    if not skip_validation:
        validate_mesh(mesh)
    v = mesh.points
    if v.shape[0] < 4:
        raise ValueError("Insufficient points for PCA (need at least 4)")
    centroid = v.mean(dim=0)
    X = v - centroid
    _, S, Vt = torch.linalg.svd(X, full_matrices=False)                 # singular values come sorted
    eigvals = S ** 2 / (X.shape[0] - 1)
    axes = Vt.T * torch.where(Vt[:, 0] < 0, -1.0, 1.0)                   # first component of every axis non-negative
    areas, normals = mesh.cell_areas, mesh.cell_normals
    projected = (areas[:, None] * normals.abs()).sum(dim=0)             # on the yz, xz, xy planes
    feats = torch.cat([centroid, axes[:, :2].reshape(-1), eigvals[:3], v.amax(0) - v.amin(0), (X ** 2).mean(dim=0), areas.sum()[None],
                       projected.flip(0)])
    if feats.shape[0] != len(FEATURE_NAMES):
        raise RuntimeError(f"Feature length mismatch: expected {len(FEATURE_NAMES)}, got {feats.shape[0]}")
    return feats if return_tensor else feats.cpu().numpy()
