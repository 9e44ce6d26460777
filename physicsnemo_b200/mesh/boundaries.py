"""Boundary detection and topological checks of simplicial meshes.

Parity: ``physicsnemo/mesh/boundaries/_detection.py`` (``get_boundary_vertices`` ``:83``,
``get_boundary_cells`` ``:132``, ``get_boundary_edges`` ``:202``) and ``_topology.py``
(``is_watertight`` ``:34``, ``is_manifold`` ``:91``).  Everything is derived from one table: the
sub-simplices of a given codimension of every cell, made unique, with the number of cells sharing
each.  A codimension-1 facet shared by exactly one cell lies on the boundary.
"""
from __future__ import annotations

import itertools

import torch

from .mesh import Mesh


def facet_table(cells: torch.Tensor, codimension: int = 1):
    """``(unique facets (F, k), multiplicity (F,), facet id of each candidate (C·m,), parent cell of each candidate)``.

    Candidates are enumerated cell-major over all ``k``-subsets of the (sorted) cell vertices,
    ``k = vertices_per_cell - codimension``.
    """
    n_cells, width = cells.shape
    k = width - codimension
    if not 1 <= k <= width:
        raise ValueError(f"codimension {codimension} is invalid for cells with {width} vertices")
    combos = torch.tensor(list(itertools.combinations(range(width), k)), device=cells.device)
    cand = cells.sort(dim=1).values[:, combos].reshape(-1, k)
    parent = torch.arange(n_cells, device=cells.device).repeat_interleave(combos.shape[0])
    if cand.shape[0] == 0:
        z = torch.zeros(0, dtype=torch.long, device=cells.device)
        return cand, z, z, parent
    facets, inverse, counts = torch.unique(cand, dim=0, return_inverse=True, return_counts=True)
    return facets, counts, inverse, parent


def get_boundary_facets(mesh: Mesh) -> torch.Tensor:
    facets, counts, _, _ = facet_table(mesh.cells, 1)
    return facets[counts == 1]


def get_boundary_vertices(mesh: Mesh) -> torch.Tensor:
    """Boolean ``(n_points,)``: the point belongs to a facet with a single adjacent cell."""
    flag = torch.zeros(mesh.n_points, dtype=torch.bool, device=mesh.points.device)
    if mesh.n_cells:
        flag[get_boundary_facets(mesh).reshape(-1)] = True
    return flag


def get_boundary_cells(mesh: Mesh, boundary_codimension: int = 1) -> torch.Tensor:
    """Boolean ``(n_cells,)``: the cell owns a sub-simplex of that codimension which no other cell shares."""
    flag = torch.zeros(mesh.n_cells, dtype=torch.bool, device=mesh.points.device)
    if mesh.n_cells == 0:
        return flag
    if not 1 <= boundary_codimension <= mesh.n_manifold_dims:
        raise ValueError(f"Invalid boundary_codimension={boundary_codimension!r}. Must be in range "
                         f"[1, {mesh.n_manifold_dims}] for mesh.n_manifold_dims={mesh.n_manifold_dims!r}")
    _, counts, inverse, parent = facet_table(mesh.cells, boundary_codimension)
    flag[parent[counts[inverse] == 1]] = True
    return flag


def get_boundary_edges(mesh: Mesh) -> torch.Tensor:
    """``(E, 2)`` sorted vertex pairs: the boundary curve of a surface, or the edges of a volume's boundary faces."""
    empty = torch.zeros(0, 2, dtype=torch.long, device=mesh.points.device)
    if mesh.n_cells == 0 or mesh.n_manifold_dims < 2:
        return empty
    faces = get_boundary_facets(mesh)
    if mesh.n_manifold_dims == 2 or faces.shape[0] == 0:
        return faces if faces.shape[0] else empty
    return facet_table(faces, faces.shape[1] - 2)[0]


def is_watertight(mesh: Mesh) -> bool:
    """Every codimension-1 facet is shared by exactly two cells (an empty mesh is not watertight; points are)."""
    if mesh.n_manifold_dims == 0:
        return True
    if mesh.n_cells == 0:
        return False
    return bool((facet_table(mesh.cells, 1)[1] == 2).all())


def _links_connected(cells: torch.Tensor, n_points: int) -> bool:
    """The cells around every vertex form one fan: facet-adjacent cells at the vertex are a single component."""
    n_cells, width = cells.shape
    if n_cells == 0:
        return True
    facets, counts, inverse, parent = facet_table(cells, 1)
    # corner = (cell, vertex); union corners of two cells that share a facet containing the vertex
    corner = torch.arange(n_cells * width, device=cells.device).reshape(n_cells, width)
    label = corner.reshape(-1).clone()
    shared = (counts == 2).nonzero().squeeze(1)
    if shared.numel():
        order = torch.argsort(inverse, stable=True)
        first = torch.searchsorted(inverse[order], shared)
        ca, cb = parent[order[first]], parent[order[first + 1]]
        pairs_a, pairs_b = [], []
        for j in range(facets.shape[1]):
            v = facets[shared, j]
            pairs_a.append(corner[ca, (cells[ca] == v[:, None]).float().argmax(1)])
            pairs_b.append(corner[cb, (cells[cb] == v[:, None]).float().argmax(1)])
        a, b = torch.cat(pairs_a), torch.cat(pairs_b)
        for _ in range(n_cells * width):
            low = torch.minimum(label[a], label[b])
            new = label.clone()
            new.scatter_reduce_(0, a, low, "amin")
            new.scatter_reduce_(0, b, low, "amin")
            new = new[new]                                    # pointer jumping
            if torch.equal(new, label):
                break
            label = new
    key = cells.reshape(-1) * (n_cells * width) + label          # (vertex, component) pairs
    per_vertex = torch.bincount(torch.unique(key) // (n_cells * width), minlength=n_points)
    return bool((per_vertex <= 1).all())


def is_manifold(mesh: Mesh, check_level: str = "full") -> bool:
    """``"facets"``: no facet has more than two cells; ``"edges"`` / ``"full"`` also require one cell fan per vertex."""
    if check_level not in ("facets", "edges", "full"):
        raise ValueError(f"check_level must be 'facets', 'edges' or 'full', got {check_level!r}")
    if mesh.n_cells == 0 or mesh.n_manifold_dims == 0:
        return True
    if bool((facet_table(mesh.cells, 1)[1] > 2).any()):
        return False
    if check_level == "facets" or mesh.n_manifold_dims < 2:
        return True
    return _links_connected(mesh.cells, mesh.n_points)
