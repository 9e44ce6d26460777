"""Discrete calculus on simplicial meshes: gradient, divergence, curl, Laplacian and integrals of fields.

Parity: ``physicsnemo/mesh/calculus/{gradient,divergence,curl,laplacian,integration}.py``.  The building block is the
exact gradient of the piecewise-linear interpolant of a vertex field on every cell: with edge vectors ``E = [p_1 − p_0,
…, p_M − p_0]`` (M × D) and value differences ``d = [f_1 − f_0, …]`` the gradient is the minimum-norm solution of
``E g = d``, i.e. ``g = E⁺ d`` — it lies in the cell's tangent space, so the same formula serves triangles in 3-D,
tetrahedra, and edges.  Vertex values are area-weighted means of the incident cells' values; divergence and curl are
traces / antisymmetric parts of the gradient of a vector field; the Laplacian of a surface field is the cotangent
operator of ``mesh/operations.py``.
"""
from __future__ import annotations

import torch

from .mesh import Mesh
from .operations import cotangent_laplacian, vertex_areas


def _cell_pinv(mesh: Mesh) -> torch.Tensor:
    """``E⁺`` per cell: ``[n_cells, D, M]``."""
    p = mesh.points[mesh.cells]                              # [n_cells, M + 1, D]
    edges = p[:, 1:] - p[:, :1]                              # [n_cells, M, D]
    return torch.linalg.pinv(edges)


def cell_gradient(mesh: Mesh, point_values: torch.Tensor) -> torch.Tensor:
    """Gradient of the piecewise-linear interpolant of a vertex field on every cell.

    ``point_values``: ``[n_points]`` or ``[n_points, C]`` → ``[n_cells, D]`` or ``[n_cells, C, D]``."""
    f = point_values.reshape(mesh.n_points, -1)
    fc = f[mesh.cells]                                       # [n_cells, M + 1, C]
    d = fc[:, 1:] - fc[:, :1]                                # [n_cells, M, C]
    g = torch.einsum("ndm,nmc->ncd", _cell_pinv(mesh), d)    # [n_cells, C, D]
    return g[:, 0] if point_values.ndim == 1 else g


def cells_to_points(mesh: Mesh, cell_values: torch.Tensor) -> torch.Tensor:
    """Measure-weighted average of the incident cells' values at every vertex."""
    w = mesh.cell_areas
    V = mesh.cells.shape[1]
    flat = cell_values.reshape(mesh.n_cells, -1)
    num = torch.zeros(mesh.n_points, flat.shape[1], dtype=flat.dtype, device=flat.device)
    num.index_add_(0, mesh.cells.reshape(-1), (flat * w[:, None]).repeat_interleave(V, dim=0))
    den = torch.zeros(mesh.n_points, dtype=flat.dtype, device=flat.device).index_add_(0, mesh.cells.reshape(-1),
                                                                                      w.repeat_interleave(V))
    return (num / den.clamp_min(1e-30)[:, None]).reshape(mesh.n_points, *cell_values.shape[1:])


def gradient(mesh: Mesh, point_values: torch.Tensor, at: str = "points") -> torch.Tensor:
    """Gradient of a vertex field, on cells (exact for the linear interpolant) or averaged to the vertices."""
    g = cell_gradient(mesh, point_values)
    if at == "cells":
        return g
    if at != "points":
        raise ValueError("`at` is 'points' or 'cells'")
    return cells_to_points(mesh, g)


def divergence(mesh: Mesh, point_vectors: torch.Tensor, at: str = "points") -> torch.Tensor:
    """Divergence of a vertex vector field ``[n_points, D]``: trace of its (tangential) gradient."""
    if point_vectors.shape != (mesh.n_points, mesh.n_spatial_dims):
        raise ValueError(f"expected a [{mesh.n_points}, {mesh.n_spatial_dims}] vector field, got {tuple(point_vectors.shape)}")
    jac = cell_gradient(mesh, point_vectors)                 # [n_cells, D (component), D (direction)]
    div = jac.diagonal(dim1=1, dim2=2).sum(-1)
    return div if at == "cells" else cells_to_points(mesh, div)


def curl(mesh: Mesh, point_vectors: torch.Tensor, at: str = "points") -> torch.Tensor:
    """Curl of a vertex vector field: a scalar in 2-D, a vector in 3-D (from the antisymmetric part of the gradient)."""
    D = mesh.n_spatial_dims
    if point_vectors.shape != (mesh.n_points, D) or D not in (2, 3):
        raise ValueError("curl needs a [n_points, 2] or [n_points, 3] vector field")
    jac = cell_gradient(mesh, point_vectors)                 # J[c, i, j] = d v_i / d x_j
    if D == 2:
        c = jac[:, 1, 0] - jac[:, 0, 1]
    else:
        c = torch.stack([jac[:, 2, 1] - jac[:, 1, 2], jac[:, 0, 2] - jac[:, 2, 0], jac[:, 1, 0] - jac[:, 0, 1]], dim=-1)
    return c if at == "cells" else cells_to_points(mesh, c)


def laplacian(mesh: Mesh, point_values: torch.Tensor) -> torch.Tensor:
    """Laplace–Beltrami of a vertex field on a triangle mesh (cotangent weights, area-normalised)."""
    return cotangent_laplacian(mesh, point_values, normalize=True)


def integrate(mesh: Mesh, values: torch.Tensor, association: str = "point") -> torch.Tensor:
    """``∫ f`` over the mesh: vertex values with the barycentric dual areas, cell values with the cell measures."""
    if association == "point":
        w = vertex_areas(mesh)
        n = mesh.n_points
    elif association == "cell":
        w, n = mesh.cell_areas, mesh.n_cells
    else:
        raise ValueError("association is 'point' or 'cell'")
    flat = values.reshape(n, -1)
    return (flat * w[:, None]).sum(0).reshape(values.shape[1:])
