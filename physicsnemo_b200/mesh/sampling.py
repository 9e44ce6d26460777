"""Point location and data sampling on simplicial meshes.

Parity: ``physicsnemo/mesh/sampling/sample_data.py`` (``compute_barycentric_coordinates`` ``:138``,
``…_pairwise`` ``:173``, ``find_containing_cells`` ``:289``, ``find_all_containing_cells`` ``:362``,
``find_nearest_cells`` ``:405``, ``match_points`` ``:445``, ``sample_data_at_points`` ``:626``) and
``random_point_sampling.py`` (``sample_random_points_on_cells``).  Candidate (query, cell) pairs come
from a box test evaluated in query chunks (a dense boolean tile per chunk) instead of a tree walk;
the barycentric solve then runs once over the flat pair list.
"""
from __future__ import annotations

from typing import Dict, Literal, Optional

import torch

from .mesh import Mesh

_PAIR_BUDGET = 1 << 24          # booleans per box-test tile


def compute_barycentric_coordinates_pairwise(query_points: torch.Tensor, cell_vertices: torch.Tensor):
    """Barycentric coordinates of query ``i`` in simplex ``i``: ``(P, n + 1)`` and the distance to the simplex's affine hull ``(P,)``.

    Least squares on the edge matrix, so simplices of any codimension work; the residual tells how far
    off the manifold the query lies.
    """
    origin = cell_vertices[:, 0]
    edges = (cell_vertices[:, 1:] - origin[:, None]).transpose(1, 2)            # (P, d, n)
    rhs = (query_points - origin).unsqueeze(-1)
    if edges.shape[-1] == 0:
        rest = rhs.new_zeros(rhs.shape[0], 0)
        residual = torch.linalg.norm(rhs.squeeze(-1), dim=-1)
    else:
        gram = edges.transpose(1, 2) @ edges
        rest = (torch.linalg.pinv(gram) @ (edges.transpose(1, 2) @ rhs)).squeeze(-1)
        residual = torch.linalg.norm((edges @ rest.unsqueeze(-1) - rhs).squeeze(-1), dim=-1)
    return torch.cat([1 - rest.sum(dim=1, keepdim=True), rest], dim=1), residual


def compute_barycentric_coordinates(query_points: torch.Tensor, cell_vertices: torch.Tensor) -> torch.Tensor:
    """All pairs: ``(Q, d)`` queries against ``(C, n + 1, d)`` simplices → ``(Q, C, n + 1)``."""
    Q, C = query_points.shape[0], cell_vertices.shape[0]
    q = query_points[:, None, :].expand(Q, C, -1).reshape(Q * C, -1)
    v = cell_vertices[None].expand(Q, C, -1, -1).reshape(Q * C, *cell_vertices.shape[1:])
    return compute_barycentric_coordinates_pairwise(q, v)[0].reshape(Q, C, -1)


def _containing_pairs(mesh: Mesh, query_points: torch.Tensor, tolerance: float):
    """``(query index, cell index, barycentric coordinates)`` of every containment, sorted by query then cell."""
    verts = mesh.points[mesh.cells]
    lo, hi = verts.amin(dim=1) - tolerance, verts.amax(dim=1) + tolerance
    chunk = max(1, _PAIR_BUDGET // max(mesh.n_cells, 1))
    qs, cs, bs = [], [], []
    for start in range(0, query_points.shape[0], chunk):
        q = query_points[start:start + chunk]
        inside = ((q[:, None, :] >= lo[None]) & (q[:, None, :] <= hi[None])).all(dim=-1)
        qi, ci = inside.nonzero(as_tuple=True)
        if qi.numel() == 0:
            continue
        bary, residual = compute_barycentric_coordinates_pairwise(q[qi], verts[ci])
        ok = (bary >= -tolerance).all(dim=1) & (residual <= tolerance)
        qs.append(qi[ok] + start)
        cs.append(ci[ok])
        bs.append(bary[ok])
    if not qs:
        z = torch.zeros(0, dtype=torch.long, device=query_points.device)
        return z, z, query_points.new_zeros(0, mesh.cells.shape[1])
    return torch.cat(qs), torch.cat(cs), torch.cat(bs)


def find_all_containing_cells(mesh: Mesh, query_points: torch.Tensor, tolerance: float = 1e-6):
    """Every (query, cell) containment as flat lists ``(query_indices, cell_indices, barycentric_coords)``."""
    return _containing_pairs(mesh, query_points, tolerance)


def find_containing_cells(mesh: Mesh, query_points: torch.Tensor, tolerance: float = 1e-6):
    """First containing cell per query (``-1`` when outside) and its barycentric coordinates (NaN when outside)."""
    qi, ci, bary = _containing_pairs(mesh, query_points, tolerance)
    n = query_points.shape[0]
    cell = torch.full((n,), -1, dtype=torch.long, device=query_points.device)
    coords = query_points.new_full((n, mesh.cells.shape[1]), float("nan"))
    if qi.numel():
        first = torch.ones_like(qi, dtype=torch.bool)
        first[1:] = qi[1:] != qi[:-1]
        cell[qi[first]], coords[qi[first]] = ci[first], bary[first]
    return cell, coords


def find_nearest_cells(mesh: Mesh, query_points: torch.Tensor) -> torch.Tensor:
    """Index of the cell with the nearest centroid."""
    from ..nn.functional.neighbors import knn

    return knn(mesh.cell_centroids.float(), query_points.float(), k=1)[0][:, 0].long()


def match_points(points_a: torch.Tensor, points_b: torch.Tensor, tolerance: float = 1e-6) -> torch.Tensor:
    """For each point of ``a`` the index of a coincident point of ``b`` (within ``tolerance``), else ``-1``."""
    from ..nn.functional.neighbors import knn

    if points_b.shape[0] == 0:
        return torch.full((points_a.shape[0],), -1, dtype=torch.long, device=points_a.device)
    idx = knn(points_b.float(), points_a.float(), k=1)[0][:, 0].long()
    close = torch.linalg.norm(points_b[idx] - points_a, dim=1) <= tolerance
    return torch.where(close, idx, torch.full_like(idx, -1))


def sample_random_points_on_cells(mesh: Mesh, cell_indices=None, alpha: float = 1.0, generator=None) -> torch.Tensor:
    return mesh.sample_random_points_on_cells(cell_indices, alpha=alpha, generator=generator)


def _floating(t: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
    if t.is_floating_point() or t.is_complex():
        return t
    return t.to(torch.float64)


def sample_data_at_points(mesh: Mesh, query_points: torch.Tensor, data_source: Literal["cells", "points"] = "cells",
                          multiple_cells_strategy: Literal["mean", "nan"] = "mean", project_onto_nearest_cell: bool = False,
                          tolerance: float = 1e-6) -> Dict[str, torch.Tensor]:
    """Cell data of the containing cell, or point data interpolated with barycentric weights, at each query point.

    Outside the mesh the result is NaN.  A point inside several cells (on a shared facet) gets the mean
    over them, or NaN with ``multiple_cells_strategy="nan"``.  ``project_onto_nearest_cell`` replaces
    each query by the centroid of its nearest cell first (useful on surfaces, where exact on-manifold
    points are hard to supply).  Integer fields come back as float64 so that NaN can mark misses.
    """
    if data_source not in ("cells", "points"):
        raise ValueError(f"Invalid data_source={data_source!r}. Must be 'cells' or 'points'.")
    if multiple_cells_strategy not in ("mean", "nan"):
        raise ValueError(f"Invalid multiple_cells_strategy={multiple_cells_strategy!r}. Must be 'mean' or 'nan'.")
    if project_onto_nearest_cell and mesh.n_cells:
        query_points = mesh.cell_centroids[find_nearest_cells(mesh, query_points)]
    n = query_points.shape[0]
    qi, ci, bary = _containing_pairs(mesh, query_points, tolerance)
    hits = torch.zeros(n, dtype=torch.long, device=query_points.device).index_add_(0, qi, torch.ones_like(qi))
    out: Dict[str, torch.Tensor] = {}
    fields = mesh.cell_data if data_source == "cells" else mesh.point_data
    for name, values in fields.items():
        values = _floating(values, mesh.points)
        if data_source == "cells":
            per_pair = values[ci]
        else:
            dtype = torch.promote_types(values.dtype, mesh.points.dtype)
            w = bary.to(dtype).reshape(bary.shape + (1,) * (values.ndim - 1))
            per_pair = (values[mesh.cells[ci]].to(dtype) * w).sum(dim=1)
        total = per_pair.new_zeros((n,) + tuple(per_pair.shape[1:])).index_add_(0, qi, per_pair)
        count = hits.reshape((n,) + (1,) * (per_pair.ndim - 1))
        result = total / count.clamp_min(1).to(total.dtype if not total.is_complex() else total.real.dtype)
        bad = hits == 0 if multiple_cells_strategy == "mean" else hits != 1
        result[bad] = float("nan")
        out[name] = result
    return out
