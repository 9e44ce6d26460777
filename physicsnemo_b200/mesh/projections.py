"""Changing the ambient or the manifold dimension of a mesh: ``embed``, ``project``, ``extrude``.

Parity: ``physicsnemo/mesh/projections/_embed.py:24``, ``_project.py:27``, ``_extrude.py:29``.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .mesh import Mesh


def _rebuild(mesh: Mesh, points: torch.Tensor, **over) -> Mesh:
    args = dict(points=points, cells=mesh.cells, point_data=mesh.point_data, cell_data=mesh.cell_data,
                global_data=mesh.global_data)
    args.update(over)
    return Mesh(**args)


def embed(mesh: Mesh, target_n_spatial_dims: int, insert_at: Optional[int] = None) -> Mesh:
    """Add zero coordinates until the points have ``target_n_spatial_dims`` components (appended, or inserted before column ``insert_at``)."""
    d = mesh.n_spatial_dims
    if target_n_spatial_dims < 1:
        raise ValueError(f"target_n_spatial_dims must be >= 1, got {target_n_spatial_dims=!r}")
    if target_n_spatial_dims < d:
        raise ValueError(f"Cannot embed: {target_n_spatial_dims=!r} < current n_spatial_dims={d!r}. Use project() to reduce "
                         "spatial dimensions.")
    if target_n_spatial_dims == d:
        return mesh
    at = d if insert_at is None else insert_at
    if not 0 <= at <= d:
        raise ValueError(f"insert_at must be in [0, {d}], got {insert_at=!r}")
    zeros = mesh.points.new_zeros(mesh.n_points, target_n_spatial_dims - d)
    return _rebuild(mesh, torch.cat([mesh.points[:, :at], zeros, mesh.points[:, at:]], dim=1))


def project(mesh: Mesh, target_n_spatial_dims: Optional[int] = None, *, keep_dims: Optional[Sequence[int]] = None,
            transform_point_data: bool = False, transform_cell_data: bool = False, transform_global_data: bool = False) -> Mesh:
    """Keep the first ``target_n_spatial_dims`` coordinates, or the listed ``keep_dims``; vector fields follow on request."""
    if (target_n_spatial_dims is None) == (keep_dims is None):
        raise ValueError("Specify exactly one of target_n_spatial_dims or keep_dims.")
    d = mesh.n_spatial_dims
    if keep_dims is None:
        if target_n_spatial_dims < 1:
            raise ValueError(f"target_n_spatial_dims must be >= 1, got {target_n_spatial_dims=!r}")
        if target_n_spatial_dims > d:
            raise ValueError(f"Cannot project: {target_n_spatial_dims=!r} > current n_spatial_dims={d!r}. Use embed() to add "
                             "spatial dimensions.")
        keep = list(range(target_n_spatial_dims))
    else:
        keep = [int(i) for i in keep_dims]
        bad = [i for i in keep if not 0 <= i < d]
        if bad:
            raise ValueError(f"keep_dims contains index {bad[0]}, but mesh has only {d} spatial dimensions")
    if len(keep) < mesh.n_manifold_dims:
        raise ValueError(f"Cannot project to {len(keep)} spatial dimensions: mesh has n_manifold_dims={mesh.n_manifold_dims}")
    if keep == list(range(d)):
        return mesh

    def fields(data, on):
        if not on:
            return data
        return {k: (v[..., keep] if v.ndim >= 2 and v.shape[-1] == d else v) for k, v in data.items()}

    glob = {k: (v[..., keep] if transform_global_data and v.ndim >= 1 and v.shape[-1] == d else v)
            for k, v in mesh.global_data.items()}
    return _rebuild(mesh, mesh.points[:, keep], point_data=fields(mesh.point_data, transform_point_data),
                    cell_data=fields(mesh.cell_data, transform_cell_data), global_data=glob)


def extrude(mesh: Mesh, vector=None, capping: bool = False, allow_new_spatial_dims: bool = False) -> Mesh:
    """Sweep every ``n``-simplex along ``vector`` and split the prism into ``n + 1`` simplices of dimension ``n + 1``.

    With sorted cell vertices ``v_0 … v_n`` and their translated copies ``w_i``, child ``j`` is
    ``(w_0 … w_j, v_j … v_n)``; neighbouring prisms split their shared side faces identically, so the
    result is conforming.  Point data are duplicated, cell data repeated per child.  The default
    vector is the last unit axis.
    """
    if capping:
        raise NotImplementedError("Capping is not yet implemented. Use capping=False.")
    n, d = mesh.n_manifold_dims, mesh.n_spatial_dims
    d_out = d
    if n + 1 > d:
        if not allow_new_spatial_dims:
            raise ValueError(f"Cannot extrude a {n}-dimensional manifold in {d}-dimensional space to dimension {n + 1} without "
                             "allow_new_spatial_dims=True.")
        d_out = n + 1
        mesh = embed(mesh, d_out)
    if vector is None:
        step = mesh.points.new_zeros(d_out)
        step[-1] = 1.0
    else:
        step = torch.as_tensor(vector, dtype=mesh.points.dtype, device=mesh.points.device)
        if step.ndim != 1:
            raise ValueError(f"Extrusion vector must be 1D, got shape {tuple(step.shape)}")
        if step.shape[0] > d_out:
            raise ValueError(f"Extrusion vector has {step.shape[0]} dimensions but target spatial dimensions are {d_out}")
        step = torch.nn.functional.pad(step, (0, d_out - step.shape[0]))
    points = torch.cat([mesh.points, mesh.points + step])
    base = mesh.cells.sort(dim=1).values
    lifted = base + mesh.n_points
    children = [torch.cat([lifted[:, :j + 1], base[:, j:]], dim=1) for j in range(n + 1)]
    cells = torch.cat(children) if mesh.n_cells else mesh.cells.new_zeros(0, n + 2)
    if cells.shape[0] and n + 1 == d_out:           # full-dimensional: make every child positively oriented
        edges = points[cells[:, 1:]] - points[cells[:, :1]]
        flip = torch.det(edges) < 0
        cells[flip, -2], cells[flip, -1] = cells[flip, -1].clone(), cells[flip, -2].clone()
    point_data = {k: torch.cat([v, v]) for k, v in mesh.point_data.items()}
    cell_data = {k: v.repeat((n + 1,) + (1,) * (v.ndim - 1)) for k, v in mesh.cell_data.items()}
    return Mesh(points=points, cells=cells, point_data=point_data, cell_data=cell_data, global_data=mesh.global_data)
