"""Mesh repair: degenerate-cell removal and hole filling.

Parity: ``physicsnemo/mesh/repair/{degenerate_removal,hole_filling}.py`` (``remove_degenerate_cells``,
``fill_holes(mesh, max_hole_edges) -> (mesh, stats)``): boundary edges (edges with one incident triangle) are chained into
closed loops; every loop of at most ``max_hole_edges`` edges is closed by a fan around a new vertex at the loop centroid,
wound against the boundary direction so the patch agrees with the surrounding orientation.
"""
from __future__ import annotations

import torch

from .mesh import Mesh


def remove_degenerate_cells(mesh: Mesh, area_tolerance: float = 0.0) -> tuple[Mesh, dict]:
    """Drop cells with repeated vertices or measure ``<= area_tolerance``."""
    c = mesh.cells
    s = c.sort(dim=1).values
    repeated = (s[:, 1:] == s[:, :-1]).any(dim=1)
    keep = ~repeated & (mesh.cell_areas > area_tolerance)
    return mesh.slice_cells(keep.nonzero().squeeze(1)), {"n_cells_removed": int((~keep).sum())}


def _boundary_loops(cells: torch.Tensor) -> list[list[int]]:
    e = torch.cat([cells[:, [0, 1]], cells[:, [1, 2]], cells[:, [2, 0]]])
    und = e.sort(dim=1).values
    uniq, inv, cnt = torch.unique(und, dim=0, return_inverse=True, return_counts=True)
    boundary = e[cnt[inv] == 1]                                            # directed as in their (single) triangle
    nxt = {}
    for a, b in boundary.tolist():
        nxt.setdefault(a, []).append(b)
    loops, used = [], set()
    for start in list(nxt):
        if start in used:
            continue
        loop, cur = [start], start
        used.add(start)
        while True:
            cands = [b for b in nxt.get(cur, []) if b == start or b not in used]
            if not cands:
                loop = []
                break
            cur = cands[0]
            if cur == start:
                break
            loop.append(cur)
            used.add(cur)
        if len(loop) >= 3:
            loops.append(loop)
    return loops


def fill_holes(mesh: Mesh, max_hole_edges: int = 10) -> tuple[Mesh, dict]:
    if mesh.n_manifold_dims != 2:
        raise ValueError("fill_holes needs a triangle mesh (2-D manifold)")
    loops = _boundary_loops(mesh.cells.cpu())
    stats = {"n_holes_detected": len(loops), "n_holes_filled": 0, "n_holes_skipped": 0, "n_faces_added": 0, "n_points_added": 0}
    new_pts, new_cells = [], []
    n = mesh.n_points
    for loop in loops:
        if len(loop) > max_hole_edges:
            stats["n_holes_skipped"] += 1
            continue
        idx = torch.tensor(loop, device=mesh.points.device)
        new_pts.append(mesh.points[idx].mean(0))
        centre = n + len(new_pts) - 1
        for a, b in zip(loop, loop[1:] + loop[:1]):
            new_cells.append([b, a, centre])                               # against the boundary edge direction
        stats["n_holes_filled"] += 1
        stats["n_faces_added"] += len(loop)
        stats["n_points_added"] += 1
    if not new_pts:
        return mesh, stats
    points = torch.cat([mesh.points, torch.stack(new_pts)])
    cells = torch.cat([mesh.cells, torch.tensor(new_cells, dtype=mesh.cells.dtype, device=mesh.cells.device)])
    pad = lambda v, k: torch.cat([v, v.new_zeros(k, *v.shape[1:])])  # noqa: E731
    return Mesh(points, cells, {k: pad(v, len(new_pts)) for k, v in mesh.point_data.items()},
                {k: pad(v, len(new_cells)) for k, v in mesh.cell_data.items()}, dict(mesh.global_data)), stats
