"""Triangulation of polygons and planar point sets.

Parity: ``physicsnemo/mesh/tessellation/{triangulate,_ear_clipping,delaunay,fill_interior}.py`` (``triangulate`` of polygon
meshes by fan / ear clipping, ``delaunay_mesh_2d``, ``fill_interior`` of closed boundary loops).  Polygons are projected
onto their best-fit plane before clipping; Delaunay triangulations come from ``scipy.spatial`` (a CPU library call —
tessellation is set-up work, not a training hot path).
"""
from __future__ import annotations

from typing import Sequence

import numpy as np
import torch

from .mesh import Mesh


def _to_plane(pts: np.ndarray) -> np.ndarray:
    if pts.shape[1] == 2:
        return pts
    c = pts - pts.mean(0)
    _, _, vt = np.linalg.svd(c, full_matrices=False)
    return c @ vt[:2].T


def ear_clip(polygon: np.ndarray) -> list[tuple[int, int, int]]:
    """Triangles (index triples into ``polygon``) of a simple polygon ``[n, 2 or 3]``, any winding."""
    p = _to_plane(np.asarray(polygon, dtype=np.float64))
    n = len(p)
    if n < 3:
        return []
    area2 = np.sum(p[:, 0] * np.roll(p[:, 1], -1) - np.roll(p[:, 0], -1) * p[:, 1])
    idx = list(range(n)) if area2 > 0 else list(range(n - 1, -1, -1))         # counter-clockwise walk
    cross = lambda o, a, b: (a[0] - o[0]) * (b[1] - o[1]) - (a[1] - o[1]) * (b[0] - o[0])  # noqa: E731
    tris = []
    guard = 0
    while len(idx) > 3 and guard < 10 * n:
        guard += 1
        clipped = False
        for k in range(len(idx)):
            i0, i1, i2 = idx[k - 1], idx[k], idx[(k + 1) % len(idx)]
            a, b, c = p[i0], p[i1], p[i2]
            if cross(a, b, c) <= 1e-14:
                continue                                                      # reflex or flat corner
            others = [q for q in idx if q not in (i0, i1, i2)]
            if any(cross(a, b, p[q]) >= 0 and cross(b, c, p[q]) >= 0 and cross(c, a, p[q]) >= 0 for q in others):
                continue                                                      # another vertex inside the ear
            tris.append((i0, i1, i2))
            idx.pop(k)
            clipped = True
            break
        if not clipped:                                                       # degenerate input: fall back to a fan
            break
    tris += [(idx[0], idx[k], idx[k + 1]) for k in range(1, len(idx) - 1)]
    return tris


def triangulate(points: torch.Tensor, polygons: Sequence[Sequence[int]]) -> Mesh:
    """Triangle mesh of arbitrary simple polygons; ``cell_data['polygon_index']`` records the source polygon."""
    P = points.detach().cpu().numpy()
    cells, owner = [], []
    for pi, poly in enumerate(polygons):
        poly = list(poly)
        for t in ear_clip(P[poly]):
            cells.append([poly[t[0]], poly[t[1]], poly[t[2]]])
            owner.append(pi)
    c = torch.tensor(cells, dtype=torch.long, device=points.device).reshape(-1, 3)
    return Mesh(points, c, cell_data={"polygon_index": torch.tensor(owner, dtype=torch.long, device=points.device)})


def _inside_polygon(q: np.ndarray, poly: np.ndarray) -> np.ndarray:
    x, y = q[:, 0:1], q[:, 1:2]
    x0, y0, x1, y1 = poly[:, 0], poly[:, 1], np.roll(poly[:, 0], -1), np.roll(poly[:, 1], -1)
    cond = ((y0 <= y) & (y1 > y)) | ((y1 <= y) & (y0 > y))
    with np.errstate(divide="ignore", invalid="ignore"):
        xi = x0 + (y - y0) * (x1 - x0) / (y1 - y0)
    return (np.sum(cond & (x < xi), axis=1) % 2) == 1


def delaunay_mesh_2d(points: torch.Tensor, boundary: Sequence[int] | None = None, holes: Sequence[Sequence[int]] = ()) -> Mesh:
    """Delaunay triangulation of planar points; with ``boundary`` (and ``holes``) given as vertex loops, triangles whose
    centroid lies outside the boundary or inside a hole are removed."""
    from scipy.spatial import Delaunay

    P = points.detach().cpu().numpy().astype(np.float64)[:, :2]
    tri = Delaunay(P).simplices
    if boundary is not None:
        cen = P[tri].mean(1)
        keep = _inside_polygon(cen, P[list(boundary)])
        for h in holes:
            keep &= ~_inside_polygon(cen, P[list(h)])
        tri = tri[keep]
    a, b, c = P[tri[:, 0]], P[tri[:, 1]], P[tri[:, 2]]
    ccw = ((b[:, 0] - a[:, 0]) * (c[:, 1] - a[:, 1]) - (b[:, 1] - a[:, 1]) * (c[:, 0] - a[:, 0])) > 0
    tri = np.where(ccw[:, None], tri, tri[:, [0, 2, 1]])
    return Mesh(points, torch.as_tensor(tri, dtype=torch.long, device=points.device))


def fill_interior(points: torch.Tensor, loops: Sequence[Sequence[int]], spacing: float | None = None) -> Mesh:
    """Triangulate the region bounded by ``loops[0]`` (outer) minus ``loops[1:]`` (holes), optionally seeding interior points
    on a lattice of the given spacing so the triangles stay well shaped."""
    P = points.detach().cpu().numpy().astype(np.float64)[:, :2]
    pts = [P]
    if spacing is not None:
        # boundary edges are split into pieces of at most spacing / 2 and interior seeds stay 0.6 spacing away from them,
        # so every boundary piece is a Gabriel edge and therefore part of the Delaunay triangulation (conforming boundary)
        extra = []
        for loop in loops:
            lp = P[list(loop)]
            for a, b in zip(lp, np.roll(lp, -1, axis=0)):
                k = int(np.ceil(np.linalg.norm(b - a) / (0.5 * spacing)))
                extra += [a + (b - a) * t / k for t in range(1, k)]
        edge_pts = np.concatenate([np.concatenate([P[list(l)] for l in loops]), np.array(extra).reshape(-1, 2)])
        pts.append(np.array(extra).reshape(-1, 2))
        outer = P[list(loops[0])]
        gx, gy = np.arange(outer[:, 0].min(), outer[:, 0].max(), spacing), np.arange(outer[:, 1].min(), outer[:, 1].max(), spacing)
        grid = np.stack(np.meshgrid(gx, gy, indexing="ij"), -1).reshape(-1, 2) + 0.5 * spacing * np.array([0.37, 0.61])
        ok = _inside_polygon(grid, outer)
        for h in loops[1:]:
            ok &= ~_inside_polygon(grid, P[list(h)])
        far = np.linalg.norm(grid[:, None] - edge_pts[None], axis=-1).min(1) > 0.6 * spacing
        pts.append(grid[ok & far])
    allp = torch.as_tensor(np.concatenate(pts), dtype=points.dtype, device=points.device)
    if points.shape[1] == 3:
        allp = torch.cat([allp, allp.new_zeros(allp.shape[0], 1)], dim=1)
        allp[: points.shape[0]] = points
    return delaunay_mesh_2d(allp, boundary=loops[0], holes=loops[1:])
