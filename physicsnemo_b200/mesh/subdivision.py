"""Subdivision of triangle meshes: linear (midpoint) and Loop.

Parity: ``physicsnemo/mesh/subdivision/{linear,loop}.py``.  One level splits every triangle into four through the
midpoints of its edges; new vertices are shared between the two triangles of an edge (found by sorting the edge keys,
no Python loop over cells).  ``loop`` then moves the vertices to the positions of Loop's scheme: an edge vertex is
``3/8 (a + b) + 1/8 (c + d)`` with c, d the vertices opposite the edge (``1/2 (a + b)`` on the boundary), an old vertex
of valence n becomes ``(1 − n β) v + β Σ neighbours`` with Warren's ``β`` (3/16 for n = 3, 3/(8n) otherwise), boundary
vertices use the ``1/8, 3/4, 1/8`` curve rule.  Point data follows the same weights; cell data is copied to the children.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from .mesh import Mesh


def _edge_table(cells: torch.Tensor, n_points: int):
    """Unique undirected edges ``[n_edges, 2]``, the edge id of each of the 3 edges of every cell ``[n_cells, 3]`` (edge k
    is opposite corner k), and how many cells use each edge."""
    a = cells[:, [1, 2, 0]]
    b = cells[:, [2, 0, 1]]
    lo, hi = torch.minimum(a, b), torch.maximum(a, b)
    key = (lo * n_points + hi).reshape(-1)
    uniq, inverse, counts = torch.unique(key, return_inverse=True, return_counts=True)
    edges = torch.stack([uniq // n_points, uniq % n_points], dim=1)
    return edges, inverse.reshape(-1, 3), counts


def _split_cells(cells: torch.Tensor, edge_of: torch.Tensor, n_points: int) -> torch.Tensor:
    m = edge_of + n_points                                    # midpoint vertex ids; m[:, k] is opposite corner k
    v0, v1, v2 = cells[:, 0], cells[:, 1], cells[:, 2]
    m0, m1, m2 = m[:, 0], m[:, 1], m[:, 2]
    return torch.stack([torch.stack([v0, m2, m1], 1), torch.stack([v1, m0, m2], 1), torch.stack([v2, m1, m0], 1),
                        torch.stack([m0, m1, m2], 1)], dim=1).reshape(-1, 3)


def _children_data(data: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    return {k: v.repeat_interleave(4, dim=0) for k, v in data.items()}


def subdivide_linear(mesh: Mesh, levels: int = 1) -> Mesh:
    """Midpoint subdivision: the surface is unchanged, every triangle becomes four."""
    for _ in range(levels):
        if mesh.n_manifold_dims != 2:
            raise ValueError("subdivision is implemented for triangle meshes")
        edges, edge_of, _ = _edge_table(mesh.cells, mesh.n_points)
        mid = lambda t: 0.5 * (t[edges[:, 0]] + t[edges[:, 1]])          # noqa: E731
        points = torch.cat([mesh.points, mid(mesh.points)])
        pdata = {k: torch.cat([v, mid(v.to(mesh.points.dtype)).to(v.dtype)]) for k, v in mesh.point_data.items()}
        mesh = Mesh(points, _split_cells(mesh.cells, edge_of, mesh.n_points), pdata, _children_data(mesh.cell_data),
                    dict(mesh.global_data))
    return mesh


def _loop_positions(values: torch.Tensor, cells: torch.Tensor, edges: torch.Tensor, edge_of: torch.Tensor,
                    counts: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    n = values.shape[0]
    flat = values.reshape(n, -1)
    interior = counts == 2
    # ---- edge vertices
    opposite_sum = torch.zeros(edges.shape[0], flat.shape[1], dtype=flat.dtype, device=flat.device)
    for k in range(3):
        opposite_sum.index_add_(0, edge_of[:, k], flat[cells[:, k]])
    ends = flat[edges[:, 0]] + flat[edges[:, 1]]
    edge_pts = torch.where(interior[:, None], 0.375 * ends + 0.125 * opposite_sum, 0.5 * ends)
    # ---- old vertices
    on_boundary = torch.zeros(n, dtype=torch.bool, device=flat.device)
    bedges = edges[~interior]
    on_boundary[bedges.reshape(-1)] = True
    valence = torch.zeros(n, dtype=flat.dtype, device=flat.device)
    nb_sum = torch.zeros_like(flat)
    for s, d in ((0, 1), (1, 0)):
        valence.index_add_(0, edges[:, s], torch.ones(edges.shape[0], dtype=flat.dtype, device=flat.device))
        nb_sum.index_add_(0, edges[:, s], flat[edges[:, d]])
    beta = torch.where(valence == 3, torch.full_like(valence, 3.0 / 16.0), 3.0 / (8.0 * valence.clamp_min(1)))
    inner = (1 - valence * beta)[:, None] * flat + beta[:, None] * nb_sum
    b_sum = torch.zeros_like(flat)
    for s, d in ((0, 1), (1, 0)):
        b_sum.index_add_(0, bedges[:, s], flat[bedges[:, d]])
    border = 0.75 * flat + 0.125 * b_sum
    old = torch.where(on_boundary[:, None], border, inner)
    shape = values.shape[1:]
    return old.reshape(n, *shape), edge_pts.reshape(edges.shape[0], *shape)


def subdivide_loop(mesh: Mesh, levels: int = 1) -> Mesh:
    """Loop subdivision (approximating, C² away from extraordinary vertices)."""
    for _ in range(levels):
        if mesh.n_manifold_dims != 2:
            raise ValueError("subdivision is implemented for triangle meshes")
        edges, edge_of, counts = _edge_table(mesh.cells, mesh.n_points)
        if int(counts.max()) > 2:
            raise ValueError("Loop subdivision needs a manifold mesh (an edge is shared by more than two triangles)")
        old, new = _loop_positions(mesh.points, mesh.cells, edges, edge_of, counts)
        pdata = {}
        for k, v in mesh.point_data.items():
            o, e = _loop_positions(v.to(mesh.points.dtype), mesh.cells, edges, edge_of, counts)
            pdata[k] = torch.cat([o, e]).to(v.dtype)
        mesh = Mesh(torch.cat([old, new]), _split_cells(mesh.cells, edge_of, mesh.n_points), pdata,
                    _children_data(mesh.cell_data), dict(mesh.global_data))
    return mesh
