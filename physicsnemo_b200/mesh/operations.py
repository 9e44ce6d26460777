"""Differential-geometry operators, smoothing, projection and simple remeshing on ``Mesh``.

Parity: ``physicsnemo/mesh/{calculus,curvature,smoothing,remeshing,projections,repair,validation}`` — cotangent
Laplace–Beltrami, angle-defect Gaussian curvature, mean curvature from the Laplacian of the embedding, Laplacian /
Taubin smoothing, vertex-clustering decimation, orientation repair and manifold / watertightness checks.
"""
from __future__ import annotations

import math
from typing import Dict

import torch

from .mesh import Mesh, _angle


def _tri(mesh: Mesh):
    if mesh.n_manifold_dims != 2:
        raise ValueError("this operator needs a triangle mesh")
    return mesh.points[mesh.cells]


def cotangent_weights(mesh: Mesh):
    """``(i, j, w)``: for every triangle corner k the weight ``½ cot θ_k`` of the opposite edge (i, j)."""
    p = _tri(mesh)
    c = mesh.cells
    I, J, W = [], [], []
    for k in range(3):
        a, b = (k + 1) % 3, (k + 2) % 3
        u, v = p[:, a] - p[:, k], p[:, b] - p[:, k]
        cot = (u * v).sum(-1) / torch.linalg.cross(_pad3(u), _pad3(v)).norm(dim=-1).clamp_min(1e-30)
        I.append(c[:, a]), J.append(c[:, b]), W.append(0.5 * cot)
    return torch.cat(I), torch.cat(J), torch.cat(W)


def _pad3(v):
    return v if v.shape[-1] == 3 else torch.nn.functional.pad(v, (0, 3 - v.shape[-1]))


def vertex_areas(mesh: Mesh) -> torch.Tensor:
    """Barycentric dual area: a third (1/(M+1)) of every incident cell's measure."""
    V = mesh.cells.shape[1]
    a = torch.zeros(mesh.n_points, dtype=mesh.points.dtype, device=mesh.device)
    return a.index_add_(0, mesh.cells.reshape(-1), (mesh.cell_areas / V).repeat_interleave(V))


def cotangent_laplacian(mesh: Mesh, values: torch.Tensor, normalize: bool = True) -> torch.Tensor:
    """``(Δf)_i = (1/A_i) Σ_j w_ij (f_j − f_i)`` (area-normalised unless ``normalize=False``)."""
    i, j, w = cotangent_weights(mesh)
    f = values.reshape(mesh.n_points, -1)
    diff = w[:, None] * (f[j] - f[i])
    out = torch.zeros_like(f).index_add_(0, i, diff).index_add_(0, j, -diff)
    if normalize:
        out = out / vertex_areas(mesh).clamp_min(1e-30)[:, None]
    return out.reshape(values.shape)


def gaussian_curvature(mesh: Mesh) -> torch.Tensor:
    p = _tri(mesh)
    ang = torch.stack([_angle(p[:, (k + 1) % 3] - p[:, k], p[:, (k + 2) % 3] - p[:, k]) for k in range(3)], dim=1)
    total = torch.zeros(mesh.n_points, dtype=p.dtype, device=mesh.device).index_add_(0, mesh.cells.reshape(-1), ang.reshape(-1))
    boundary = torch.zeros(mesh.n_points, dtype=torch.bool, device=mesh.device)
    b = mesh.get_boundary_mesh(data_source="none").cells
    boundary[b.reshape(-1)] = True
    defect = torch.where(boundary, math.pi - total, 2 * math.pi - total)
    return defect / vertex_areas(mesh).clamp_min(1e-30)


def mean_curvature(mesh: Mesh) -> torch.Tensor:
    """``H = ½ |Δx|`` signed by the vertex normal where normals exist."""
    lap = cotangent_laplacian(mesh, mesh.points)
    h = 0.5 * lap.norm(dim=-1)
    if mesh.codimension == 1:
        h = h * torch.sign(-(lap * mesh.point_normals).sum(-1)).where(h > 0, torch.ones_like(h))
    return h


def laplacian_smooth(mesh: Mesh, iterations: int = 10, relaxation: float = 0.5, fix_boundary: bool = True,
                     taubin_mu: float | None = None) -> Mesh:
    """Umbrella-operator smoothing; with ``taubin_mu`` (< 0) every step is followed by an inflating step (no shrink)."""
    adj = mesh.get_point_to_points_adjacency()
    src, dst, cnt = adj.sources(), adj.indices, adj.counts().clamp_min(1)
    fixed = torch.zeros(mesh.n_points, dtype=torch.bool, device=mesh.device)
    if fix_boundary and mesh.n_manifold_dims >= 1 and mesh.n_cells:
        fixed[mesh.get_boundary_mesh(data_source="none").cells.reshape(-1)] = True
    pts = mesh.points
    for _ in range(iterations):
        for lam in ([relaxation] if taubin_mu is None else [relaxation, taubin_mu]):
            mean = torch.zeros_like(pts).index_add_(0, src, pts[dst]) / cnt[:, None]
            pts = torch.where(fixed[:, None], pts, pts + lam * (mean - pts))
    return Mesh(pts, mesh.cells, mesh.point_data, mesh.cell_data, mesh.global_data)


def cluster_decimate(mesh: Mesh, cell_size: float) -> Mesh:
    """Vertex clustering on a uniform lattice: points of a lattice cell collapse to their mean."""
    q = torch.floor((mesh.points - mesh.points.amin(0)) / cell_size).long()
    _, inv = torch.unique(q, dim=0, return_inverse=True)
    n = int(inv.max()) + 1
    cnt = torch.bincount(inv, minlength=n).clamp_min(1)
    pts = torch.zeros(n, mesh.n_spatial_dims, dtype=mesh.points.dtype, device=mesh.device).index_add_(0, inv, mesh.points) / cnt[:, None]
    pd = {k: torch.zeros(n, *v.shape[1:], dtype=v.dtype, device=v.device).index_add_(0, inv, v) / cnt.reshape(-1, *[1] * (v.ndim - 1))
          for k, v in mesh.point_data.items() if v.is_floating_point()}
    return Mesh(pts, inv[mesh.cells], pd, mesh.cell_data, mesh.global_data).clean(merge_points=False)


def project_to_plane(mesh: Mesh, origin, normal) -> Mesh:
    n = torch.as_tensor(normal, dtype=mesh.points.dtype, device=mesh.device)
    n = n / n.norm()
    o = torch.as_tensor(origin, dtype=mesh.points.dtype, device=mesh.device)
    d = ((mesh.points - o) * n).sum(-1, keepdim=True)
    return mesh._with_points(mesh.points - d * n)


def orient_consistently(mesh: Mesh) -> Mesh:
    """Flip triangles so that neighbours traverse their shared edge in opposite directions (breadth-first)."""
    if mesh.n_manifold_dims != 2 or mesh.n_cells == 0:
        return mesh
    cells = mesh.cells.clone().cpu()
    nbrs = mesh.facet_neighbors().cpu()
    seen = torch.zeros(mesh.n_cells, dtype=torch.bool)
    for seed in range(mesh.n_cells):
        if seen[seed]:
            continue
        seen[seed] = True
        queue = [seed]
        while queue:
            c = queue.pop()
            tri = cells[c].tolist()
            for k in range(3):
                nb = int(nbrs[c, k])
                if nb < 0 or seen[nb]:
                    continue
                a, b = tri[(k + 1) % 3], tri[(k + 2) % 3]
                t2 = cells[nb].tolist()
                ia, ib = t2.index(a), t2.index(b)
                if (ia + 1) % 3 == ib:                      # same direction on the shared edge: flip the neighbour
                    cells[nb] = cells[nb].flip(0)
                    nbrs[nb] = nbrs[nb].flip(0)
                seen[nb] = True
                queue.append(nb)
    return Mesh(mesh.points, cells.to(mesh.device), mesh.point_data, mesh.cell_data, mesh.global_data)


def validate(mesh: Mesh) -> Dict[str, object]:
    """Topological health report: facet multiplicities, watertightness, manifoldness, degenerate cells, Euler number."""
    rep: Dict[str, object] = {"n_points": mesh.n_points, "n_cells": mesh.n_cells}
    if mesh.n_cells == 0 or mesh.n_manifold_dims == 0:
        return rep
    facets = mesh.get_facet_mesh(1, data_source="none")
    mult = facets._cache["facet_parent_count"]
    rep["n_boundary_facets"] = int((mult == 1).sum())
    rep["n_nonmanifold_facets"] = int((mult > 2).sum())
    rep["is_watertight"] = bool((mult == 2).all())
    rep["is_manifold"] = bool((mult <= 2).all())
    rep["n_degenerate_cells"] = int((mesh.cell_areas <= 0).sum())
    used = torch.zeros(mesh.n_points, dtype=torch.bool, device=mesh.device)
    used[mesh.cells.reshape(-1)] = True
    rep["n_unused_points"] = int((~used).sum())
    if mesh.n_manifold_dims == 2:
        rep["euler_characteristic"] = int(used.sum()) - facets.n_cells + mesh.n_cells
    return rep


def total_measure(mesh: Mesh) -> torch.Tensor:
    return mesh.cell_areas.sum()


def enclosed_volume(mesh: Mesh) -> torch.Tensor:
    """Signed volume (area in 2-D) enclosed by a closed, consistently oriented codimension-1 mesh (divergence theorem)."""
    if mesh.codimension != 1:
        raise ValueError("enclosed_volume needs a codimension-1 mesh")
    p = mesh.points[mesh.cells]
    D = mesh.n_spatial_dims
    return torch.linalg.det(p).sum() / math.factorial(D)
