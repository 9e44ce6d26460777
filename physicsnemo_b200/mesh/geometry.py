"""Differential-geometric quantities of simplicial meshes: angles, circumcentres, dual volumes, FEM cotangent weights,
gradients of the barycentric coordinate functions.

Parity: ``physicsnemo/mesh/geometry/_angles.py`` (``stable_angle_between_vectors`` ``:61``,
``compute_triangle_angles`` ``:97``, ``compute_vertex_angle_sums`` ``:267``), ``dual_meshes.py``
(``compute_dual_volumes_0`` ``:240``, ``compute_circumcenters`` ``:427``,
``compute_cotan_weights_fem`` ``:509``) and ``interpolation.py`` (``compute_barycentric_gradients``
``:57``).  Everything is batched over cells; per-vertex results are index-added from the cells.
"""
from __future__ import annotations

import itertools

import torch

from .mesh import Mesh, simplex_measure


def stable_angle_between_vectors(v1: torch.Tensor, v2: torch.Tensor) -> torch.Tensor:
    """Angle in ``[0, π]`` via ``2 · atan2(|a − b|, |a + b|)`` of the unit vectors (accurate near 0 and π, any dimension)."""
    a = v1 / torch.linalg.norm(v1, dim=-1, keepdim=True).clamp_min(1e-30)
    b = v2 / torch.linalg.norm(v2, dim=-1, keepdim=True).clamp_min(1e-30)
    return 2 * torch.atan2(torch.linalg.norm(a - b, dim=-1), torch.linalg.norm(a + b, dim=-1))


def compute_triangle_angles(p0: torch.Tensor, p1: torch.Tensor, p2: torch.Tensor) -> torch.Tensor:
    """Interior angle at ``p0`` of the triangles ``(p0, p1, p2)``."""
    return stable_angle_between_vectors(p1 - p0, p2 - p0)


def corner_angles(mesh: Mesh) -> torch.Tensor:
    """``(n_cells, 3)`` interior angles of a triangle mesh, one per cell corner."""
    if mesh.n_manifold_dims != 2:
        raise ValueError(f"corner angles need a triangle mesh, got manifold dimension {mesh.n_manifold_dims}")
    p = mesh.points[mesh.cells]
    return torch.stack([compute_triangle_angles(p[:, i], p[:, (i + 1) % 3], p[:, (i + 2) % 3]) for i in range(3)], dim=1)


def compute_vertex_angle_sums(mesh: Mesh) -> torch.Tensor:
    """Sum of the incident corner angles at every vertex (2π at a flat interior vertex; curves: angle between the two edges)."""
    out = mesh.points.new_zeros(mesh.n_points)
    if mesh.n_cells == 0:
        return out
    if mesh.n_manifold_dims == 2:
        return out.index_add_(0, mesh.cells.reshape(-1), corner_angles(mesh).reshape(-1))
    if mesh.n_manifold_dims == 1:
        # interior vertices of a curve: angle between the two incident edges, seen from the vertex
        a, b = mesh.cells[:, 0], mesh.cells[:, 1]
        direction = mesh.points[b] - mesh.points[a]
        away = mesh.points.new_zeros(mesh.n_points, 2, mesh.n_spatial_dims)
        count = torch.zeros(mesh.n_points, dtype=torch.long, device=mesh.points.device)
        for vertex, vec in ((a, direction), (b, -direction)):
            order = torch.argsort(vertex, stable=True)
            v, d = vertex[order], vec[order]
            slot = count[v] + (torch.arange(v.numel(), device=v.device) - torch.searchsorted(v, v))
            ok = slot < 2
            away[v[ok], slot[ok]] = d[ok]
            count.index_add_(0, v, torch.ones_like(v))
        both = count >= 2
        out[both] = stable_angle_between_vectors(away[both, 0], away[both, 1])
        return out
    raise NotImplementedError("vertex angle sums are defined here for curves and triangle surfaces")


def compute_circumcenters(vertices: torch.Tensor) -> torch.Tensor:
    """Circumcentres of simplices ``(n, k + 1, d)`` embedded in ``d ≥ k`` dimensions.

    With edge vectors ``e_i = v_i − v_0`` the centre is ``v_0 + Σ c_i e_i`` where ``2 G c = diag(G)``,
    ``G = E Eᵀ`` the Gram matrix; this stays inside the simplex's affine hull for any codimension.
    """
    e = vertices[:, 1:] - vertices[:, :1]
    if e.shape[1] == 0:
        return vertices[:, 0]
    gram = e @ e.transpose(1, 2)
    rhs = 0.5 * torch.diagonal(gram, dim1=1, dim2=2).unsqueeze(-1)
    coeff = torch.linalg.lstsq(gram, rhs).solution if gram.shape[0] else rhs
    return vertices[:, 0] + (coeff * e).sum(dim=1)


def compute_dual_volumes_0(mesh: Mesh) -> torch.Tensor:
    """Measure of the dual cell of every vertex; the values sum to the total measure of the mesh.

    Curves: half of each incident edge.  Triangles: the mixed Voronoi areas of Meyer et al. — the
    circumcentric share ``(|e_1|² cot α_1 + |e_2|² cot α_2) / 8`` in non-obtuse triangles, and in an
    obtuse one half of the area at the obtuse corner and a quarter at the others.  Higher dimensions:
    an equal share ``|σ| / (n + 1)`` of every incident cell.
    """
    out = mesh.points.new_zeros(mesh.n_points)
    n = mesh.n_manifold_dims
    if mesh.n_cells == 0 or n == 0:
        return out
    areas = mesh.cell_areas
    if n != 2:
        share = (areas / (n + 1))[:, None].expand(-1, n + 1)
        return out.index_add_(0, mesh.cells.reshape(-1), share.reshape(-1))
    p = mesh.points[mesh.cells]
    angle = corner_angles(mesh)
    cot = torch.cos(angle) / torch.sin(angle).clamp_min(1e-30)
    obtuse = angle > torch.pi / 2
    any_obtuse = obtuse.any(dim=1, keepdim=True)
    voronoi = []
    for i in range(3):
        j, k = (i + 1) % 3, (i + 2) % 3
        len_ij = (p[:, j] - p[:, i]).square().sum(-1)            # edge i–j is opposite corner k
        len_ik = (p[:, k] - p[:, i]).square().sum(-1)
        voronoi.append((len_ij * cot[:, k] + len_ik * cot[:, j]) / 8)
    voronoi = torch.stack(voronoi, dim=1)
    mixed = torch.where(obtuse, areas[:, None] / 2, areas[:, None] / 4)
    return out.index_add_(0, mesh.cells.reshape(-1), torch.where(any_obtuse, mixed, voronoi).reshape(-1))


def compute_barycentric_gradients(mesh: Mesh) -> torch.Tensor:
    """``(n_cells, n + 1, d)``: gradient of each barycentric coordinate function inside each cell (tangent to the cell)."""
    p = mesh.points[mesh.cells]
    e = p[:, 1:] - p[:, :1]                                      # (c, n, d)
    gram_inv = torch.linalg.pinv(e @ e.transpose(1, 2))
    rest = gram_inv @ e                                          # rows: ∇λ_1 … ∇λ_n
    return torch.cat([-rest.sum(dim=1, keepdim=True), rest], dim=1)


def compute_cotan_weights_fem(mesh: Mesh):
    """``(weights (E,), edges (E, 2))`` with ``w_ij = −Σ_σ |σ| ∇λ_i · ∇λ_j`` over the cells sharing edge ``(i, j)``.

    For triangles this is ``(cot α + cot β) / 2``; for a curve ``1 / |e|``; the same formula covers tetrahedra.
    """
    width = mesh.cells.shape[1]
    if mesh.n_cells == 0 or width < 2:
        return mesh.points.new_zeros(0), torch.zeros(0, 2, dtype=torch.long, device=mesh.points.device)
    grads = compute_barycentric_gradients(mesh)
    stiffness = mesh.cell_areas[:, None, None] * (grads @ grads.transpose(1, 2))
    pairs = torch.tensor(list(itertools.combinations(range(width), 2)), device=mesh.points.device)
    ends = torch.stack([mesh.cells[:, pairs[:, 0]], mesh.cells[:, pairs[:, 1]]], dim=-1).reshape(-1, 2).sort(dim=1).values
    local = -stiffness[:, pairs[:, 0], pairs[:, 1]].reshape(-1)
    edges, which = torch.unique(ends, dim=0, return_inverse=True)
    return local.new_zeros(edges.shape[0]).index_add_(0, which, local), edges


def compute_dual_volumes_1(mesh: Mesh):
    """Dual measure of every edge, ``|⋆e| = w_e · |e|`` with the FEM cotangent weight: ``(volumes (E,), edges (E, 2))``."""
    w, edges = compute_cotan_weights_fem(mesh)
    length = torch.linalg.norm(mesh.points[edges[:, 1]] - mesh.points[edges[:, 0]], dim=1)
    return w * length, edges
