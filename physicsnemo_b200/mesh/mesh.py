"""``Mesh``: a simplicial mesh of any manifold dimension embedded in any spatial dimension, with tensor data.

Parity: ``physicsnemo/mesh/mesh.py`` — ``points [P, D]``, ``cells [C, M+1]`` (point clouds have ``M = 0`` cells or
none), ``point_data`` / ``cell_data`` / ``global_data`` dictionaries of tensors, cached geometry (centroids,
measures, normals), topology (facets, boundary, edge / dual graphs, adjacency in CSR form), data transfer between
points and cells, sampling, slicing, merging, cleaning, subdivision, discrete calculus and curvature.  All arrays
are ``torch`` tensors, so a mesh lives on any device and every geometric quantity is differentiable with respect
to ``points``.
"""
from __future__ import annotations

import math
from enum import Enum
from itertools import combinations
from typing import Any, Callable, Dict, Optional, Sequence

import torch


class MeshFieldAssociation(str, Enum):
    POINT = "point"
    CELL = "cell"
    GLOBAL = "global"


MESH_FIELD_ASSOCIATIONS = tuple(a.value for a in MeshFieldAssociation)


class Adjacency:
    """Ragged neighbour lists in CSR form: ``indices[offsets[i]:offsets[i+1]]`` are the neighbours of ``i``."""

    def __init__(self, offsets: torch.Tensor, indices: torch.Tensor):
        self.offsets, self.indices = offsets, indices

    @property
    def n_sources(self) -> int:
        return self.offsets.numel() - 1

    def counts(self) -> torch.Tensor:
        return self.offsets[1:] - self.offsets[:-1]

    def to_list(self) -> list[list[int]]:
        o, i = self.offsets.tolist(), self.indices.tolist()
        return [i[o[k]:o[k + 1]] for k in range(len(o) - 1)]

    def sources(self) -> torch.Tensor:
        return torch.repeat_interleave(torch.arange(self.n_sources, device=self.indices.device), self.counts())

    @staticmethod
    def from_pairs(src: torch.Tensor, dst: torch.Tensor, n_sources: int, unique: bool = True) -> "Adjacency":
        if unique and src.numel():
            key = torch.unique(src * (int(dst.max()) + 1 if dst.numel() else 1) + dst)
            width = int(dst.max()) + 1
            src, dst = key // width, key % width
        else:
            order = torch.argsort(src, stable=True)
            src, dst = src[order], dst[order]
        counts = torch.bincount(src, minlength=n_sources)
        offsets = torch.zeros(n_sources + 1, dtype=torch.long, device=src.device)
        offsets[1:] = torch.cumsum(counts, 0)
        return Adjacency(offsets, dst)


def simplex_measure(rel: torch.Tensor) -> torch.Tensor:
    """Measure of simplices given edge vectors from vertex 0, ``rel [C, M, D]``: ``sqrt(det(rel relᵀ)) / M!``."""
    M = rel.shape[1]
    if M == 0:
        return torch.ones(rel.shape[0], dtype=rel.dtype, device=rel.device)
    if M == 1:
        return rel[:, 0].norm(dim=-1)
    if M == 2 and rel.shape[2] == 3:
        return 0.5 * torch.linalg.cross(rel[:, 0], rel[:, 1]).norm(dim=-1)
    if M == rel.shape[2]:
        return torch.linalg.det(rel).abs() / math.factorial(M)
    gram = rel @ rel.transpose(1, 2)
    return torch.linalg.det(gram).clamp_min(0).sqrt() / math.factorial(M)


def simplex_normals(rel: torch.Tensor) -> torch.Tensor:
    """Unit normals of codimension-1 simplices (``rel [C, D-1, D]``): rotation in 2-D, cross product in 3-D,
    signed minors otherwise."""
    D = rel.shape[2]
    if D == 2:
        n = torch.stack([rel[:, 0, 1], -rel[:, 0, 0]], dim=-1)
    elif D == 3:
        n = torch.linalg.cross(rel[:, 0], rel[:, 1])
    else:
        comps = []
        for k in range(D):
            cols = [c for c in range(D) if c != k]
            comps.append((-1) ** k * torch.linalg.det(rel[:, :, cols]))
        n = torch.stack(comps, dim=-1)
    return n / n.norm(dim=-1, keepdim=True).clamp_min(torch.finfo(rel.dtype).tiny)


class Mesh:
    def __init__(self, points: torch.Tensor, cells: Optional[torch.Tensor] = None,
                 point_data: Optional[Dict[str, torch.Tensor]] = None, cell_data: Optional[Dict[str, torch.Tensor]] = None,
                 global_data: Optional[Dict[str, torch.Tensor]] = None, *, _cache: Optional[dict] = None) -> None:
        points = torch.as_tensor(points)
        if points.ndim != 2:
            raise ValueError(f"points must have shape (n_points, n_spatial_dims), got {tuple(points.shape)}")
        if not points.is_floating_point():
            points = points.float()
        if cells is None:
            cells = torch.empty(0, 1, dtype=torch.long, device=points.device)
        cells = torch.as_tensor(cells, device=points.device)
        if cells.ndim != 2:
            raise ValueError(f"cells must have shape (n_cells, n_vertices_per_cell), got {tuple(cells.shape)}")
        if cells.is_floating_point():
            raise TypeError("cells must be an integer tensor")
        cells = cells.long()
        if cells.numel() and (int(cells.min()) < 0 or int(cells.max()) >= points.shape[0]):
            raise ValueError(f"cell indices must satisfy 0 <= index < n_points ({points.shape[0]})")
        if cells.shape[1] - 1 > points.shape[1]:
            raise ValueError(f"manifold dimension {cells.shape[1] - 1} exceeds spatial dimension {points.shape[1]}")
        self.points, self.cells = points, cells
        self.point_data = self._coerce(point_data, points.shape[0], "point_data")
        self.cell_data = self._coerce(cell_data, cells.shape[0], "cell_data")
        self.global_data = {k: torch.as_tensor(v, device=points.device) for k, v in dict(global_data or {}).items()}
        self._cache: dict = _cache if _cache is not None else {}

    def _coerce(self, data, n, what):
        out = {}
        for k, v in dict(data or {}).items():
            t = torch.as_tensor(v, device=self.points.device)
            if t.shape[0] != n:
                raise ValueError(f"{what}['{k}'] must have leading dimension {n}, got {tuple(t.shape)}")
            out[k] = t
        return out

    # ------------------------------------------------------------------ basics
    @classmethod
    def from_polygons(cls, points: torch.Tensor, polygons: Sequence[Sequence[int]], **kw) -> "Mesh":
        """Fan-triangulate polygons (triangles, quads, …) into a triangle mesh; ``cell_data['polygon_index']`` keeps the origin."""
        tris, owner = [], []
        for pi, poly in enumerate(polygons):
            for k in range(1, len(poly) - 1):
                tris.append([poly[0], poly[k], poly[k + 1]])
                owner.append(pi)
        cd = dict(kw.pop("cell_data", None) or {})
        cd["polygon_index"] = torch.tensor(owner, dtype=torch.long)
        return cls(points, torch.tensor(tris, dtype=torch.long).reshape(-1, 3), cell_data=cd, **kw)

    @property
    def n_points(self) -> int:
        return self.points.shape[0]

    @property
    def n_spatial_dims(self) -> int:
        return self.points.shape[1]

    @property
    def n_cells(self) -> int:
        return self.cells.shape[0]

    @property
    def n_manifold_dims(self) -> int:
        return self.cells.shape[1] - 1

    @property
    def codimension(self) -> int:
        return self.n_spatial_dims - self.n_manifold_dims

    @property
    def device(self):
        return self.points.device

    def __repr__(self) -> str:
        return (f"Mesh(manifold_dim={self.n_manifold_dims}, spatial_dim={self.n_spatial_dims}, n_points={self.n_points}, "
                f"n_cells={self.n_cells}, point_data={list(self.point_data)}, cell_data={list(self.cell_data)}, "
                f"global_data={list(self.global_data)}, device={self.device})")

    def _map_tensors(self, fn) -> "Mesh":
        return Mesh(fn(self.points), self.cells.to(fn(self.points).device), {k: fn(v) for k, v in self.point_data.items()},
                    {k: fn(v) for k, v in self.cell_data.items()}, {k: fn(v) for k, v in self.global_data.items()})

    def to(self, *args, **kwargs) -> "Mesh":
        def move(t):
            if t.is_floating_point():
                return t.to(*args, **kwargs)
            dev = torch.empty(0).to(*args, **kwargs).device
            return t.to(dev)

        return self._map_tensors(move)

    def clone(self) -> "Mesh":
        return self._map_tensors(lambda t: t.clone())

    def strip_caches(self) -> "Mesh":
        self._cache.clear()
        return self

    def save(self, path: str) -> None:
        torch.save({"points": self.points.cpu(), "cells": self.cells.cpu(),
                    "point_data": {k: v.cpu() for k, v in self.point_data.items()},
                    "cell_data": {k: v.cpu() for k, v in self.cell_data.items()},
                    "global_data": {k: v.cpu() for k, v in self.global_data.items()}}, path)

    @classmethod
    def load(cls, path: str, device=None) -> "Mesh":
        d = torch.load(path, map_location=device or "cpu")
        return cls(d["points"], d["cells"], d["point_data"], d["cell_data"], d["global_data"])

    def _cached(self, key: str, fn: Callable[[], Any]):
        if key not in self._cache:
            self._cache[key] = fn()
        return self._cache[key]

    # ---------------------------------------------------------------- geometry
    def _relative(self) -> torch.Tensor:
        return self.points[self.cells[:, 1:]] - self.points[self.cells[:, :1]]

    @property
    def cell_centroids(self) -> torch.Tensor:
        return self._cached("cell_centroids", lambda: self.points[self.cells].mean(dim=1))

    @property
    def cell_areas(self) -> torch.Tensor:
        """Measure of each cell: length / area / volume according to the manifold dimension."""
        return self._cached("cell_areas", lambda: simplex_measure(self._relative()))

    @property
    def cell_normals(self) -> torch.Tensor:
        if self.codimension != 1:
            raise ValueError("cell normals are only defined for codimension-1 manifolds.\n"
                             f"Got {self.n_manifold_dims=} and {self.n_spatial_dims=}.\n"
                             "Required: n_manifold_dims = n_spatial_dims - 1 (codimension-1).\n"
                             f"Current codimension: {self.codimension}")
        return self._cached("cell_normals", lambda: simplex_normals(self._relative()))

    @property
    def point_normals(self) -> torch.Tensor:
        return self._cached("point_normals", lambda: self.compute_point_normals("area"))

    def compute_point_normals(self, weighting: str = "area") -> torch.Tensor:
        """Vertex normals as the normalised sum of incident cell normals weighted by ``"area" | "uniform" | "angle"``."""
        n = self.cell_normals
        V = self.cells.shape[1]
        if weighting == "area":
            w = self.cell_areas[:, None].expand(-1, V)
        elif weighting == "uniform":
            w = torch.ones(self.n_cells, V, dtype=n.dtype, device=n.device)
        elif weighting == "angle":
            if self.n_manifold_dims != 2:
                raise ValueError("angle weighting needs a triangle mesh")
            p = self.points[self.cells]
            w = torch.stack([_angle(p[:, (k + 1) % 3] - p[:, k], p[:, (k + 2) % 3] - p[:, k]) for k in range(3)], dim=1)
        else:
            raise ValueError(f"unknown weighting '{weighting}'")
        acc = torch.zeros(self.n_points, self.n_spatial_dims, dtype=n.dtype, device=n.device)
        acc.index_add_(0, self.cells.reshape(-1), (w[:, :, None] * n[:, None, :]).reshape(-1, self.n_spatial_dims))
        return acc / acc.norm(dim=-1, keepdim=True).clamp_min(torch.finfo(n.dtype).tiny)

    # ---------------------------------------------------------------- topology
    def get_facet_mesh(self, manifold_codimension: int = 1, data_source: str = "cells", data_aggregation: str = "mean") -> "Mesh":
        """Mesh of the unique (M − k)-dimensional faces; cell data is carried to the facets by averaging the
        parent cells (``data_source="cells"``) or point data by averaging the facet's vertices (``"points"``)."""
        M = self.n_manifold_dims
        m = M - manifold_codimension
        if m < 0:
            raise ValueError(f"cannot take codimension-{manifold_codimension} facets of a {M}-dimensional mesh")
        combos = list(combinations(range(M + 1), m + 1))
        cand = self.cells[:, combos].reshape(-1, m + 1)                                  # [C·K, m+1]
        parent = torch.arange(self.n_cells, device=self.device).repeat_interleave(len(combos))
        key = torch.sort(cand, dim=1).values
        uniq, inverse = torch.unique(key, dim=0, return_inverse=True)
        first = torch.full((uniq.shape[0],), cand.shape[0], dtype=torch.long, device=self.device)
        first.scatter_reduce_(0, inverse, torch.arange(cand.shape[0], device=self.device), reduce="amin")
        facets = cand[first]                                                              # keeps one parent's orientation
        cell_data = {}
        if data_source == "cells":
            cnt = torch.bincount(inverse, minlength=uniq.shape[0]).clamp_min(1)
            for k, v in self.cell_data.items():
                if not v.is_floating_point():
                    continue
                acc = torch.zeros(uniq.shape[0], *v.shape[1:], dtype=v.dtype, device=v.device).index_add_(0, inverse, v[parent])
                cell_data[k] = acc / cnt.reshape(-1, *[1] * (v.ndim - 1)) if data_aggregation == "mean" else acc
        elif data_source == "points":
            for k, v in self.point_data.items():
                if v.is_floating_point():
                    cell_data[k] = v[facets].mean(dim=1)
        out = Mesh(self.points, facets, self.point_data, cell_data, self.global_data)
        out._cache["facet_parent_count"] = torch.bincount(inverse, minlength=uniq.shape[0])
        return out

    def get_boundary_mesh(self, data_source: str = "cells") -> "Mesh":
        """Facets that belong to exactly one cell."""
        f = self.get_facet_mesh(1, data_source=data_source)
        keep = f._cache["facet_parent_count"] == 1
        return f.slice_cells(keep)

    def to_edge_graph(self) -> "Mesh":
        return self if self.n_manifold_dims == 1 else self.get_facet_mesh(self.n_manifold_dims - 1, data_source="none")

    def to_dual_graph(self) -> "Mesh":
        """Points = cell centroids, edges = pairs of cells sharing a facet."""
        adj = self.get_cell_to_cells_adjacency()
        src = adj.sources()
        keep = src < adj.indices
        return Mesh(self.cell_centroids, torch.stack([src[keep], adj.indices[keep]], dim=1), point_data=self.cell_data,
                    global_data=self.global_data)

    def to_point_cloud(self, keep_cell_data_as_point_data: bool = False) -> "Mesh":
        return Mesh(self.points, None, self.point_data, None, self.global_data)

    def get_point_to_cells_adjacency(self) -> Adjacency:
        def build():
            V = self.cells.shape[1]
            return Adjacency.from_pairs(self.cells.reshape(-1), torch.arange(self.n_cells, device=self.device).repeat_interleave(V),
                                        self.n_points, unique=False)

        return self._cached("adj_point_cells", build)

    def get_cell_to_points_adjacency(self) -> Adjacency:
        V = self.cells.shape[1]
        return Adjacency(torch.arange(0, (self.n_cells + 1) * V, V, device=self.device), self.cells.reshape(-1))

    def get_point_to_points_adjacency(self) -> Adjacency:
        def build():
            e = self.to_edge_graph().cells
            both = torch.cat([e, e.flip(1)], dim=0)
            return Adjacency.from_pairs(both[:, 0], both[:, 1], self.n_points)

        return self._cached("adj_point_points", build)

    def get_cell_to_cells_adjacency(self, adjacency_codimension: int = 1) -> Adjacency:
        def build():
            M = self.n_manifold_dims
            combos = list(combinations(range(M + 1), M + 1 - adjacency_codimension))
            cand = torch.sort(self.cells[:, combos].reshape(-1, M + 1 - adjacency_codimension), dim=1).values
            parent = torch.arange(self.n_cells, device=self.device).repeat_interleave(len(combos))
            _, inverse = torch.unique(cand, dim=0, return_inverse=True)
            order = torch.argsort(inverse)
            inv_s, par_s = inverse[order], parent[order]
            same = inv_s[1:] == inv_s[:-1]                      # consecutive entries of one shared facet (pairs for manifolds)
            a, b = par_s[:-1][same], par_s[1:][same]
            return Adjacency.from_pairs(torch.cat([a, b]), torch.cat([b, a]), self.n_cells)

        return self._cached(f"adj_cell_cells_{adjacency_codimension}", build)

    def facet_neighbors(self) -> torch.Tensor:
        """``[C, M+1]`` index of the cell across the facet opposite each vertex (−1 on the boundary)."""
        M = self.n_manifold_dims
        combos = [tuple(v for v in range(M + 1) if v != k) for k in range(M + 1)]
        cand = torch.sort(self.cells[:, combos].reshape(-1, M), dim=1).values
        parent = torch.arange(self.n_cells, device=self.device).repeat_interleave(M + 1)
        _, inverse = torch.unique(cand, dim=0, return_inverse=True)
        order = torch.argsort(inverse)
        inv_s = inverse[order]
        nb = torch.full((cand.shape[0],), -1, dtype=torch.long, device=self.device)
        same = inv_s[1:] == inv_s[:-1]
        a, b = order[:-1][same], order[1:][same]
        nb[a], nb[b] = parent[b], parent[a]
        return nb.reshape(self.n_cells, M + 1)

    # --------------------------------------------------------------- data moves
    def with_data(self, point_data=None, cell_data=None, global_data=None) -> "Mesh":
        return Mesh(self.points, self.cells, {**self.point_data, **dict(point_data or {})},
                    {**self.cell_data, **dict(cell_data or {})}, {**self.global_data, **dict(global_data or {})})

    def cell_data_to_point_data(self, overwrite_keys: bool = False) -> "Mesh":
        """Measure-weighted average of the incident cells' values at every point."""
        w = self.cell_areas
        V = self.cells.shape[1]
        idx = self.cells.reshape(-1)
        denom = torch.zeros(self.n_points, dtype=w.dtype, device=self.device).index_add_(0, idx, w.repeat_interleave(V)).clamp_min(1e-30)
        new = {}
        for k, v in self.cell_data.items():
            if not v.is_floating_point():
                continue
            if k in self.point_data and not overwrite_keys:
                raise ValueError(f"point_data already has key '{k}'; pass overwrite_keys=True to replace it")
            wv = (v * w.reshape(-1, *[1] * (v.ndim - 1))).repeat_interleave(V, dim=0)
            acc = torch.zeros(self.n_points, *v.shape[1:], dtype=v.dtype, device=self.device).index_add_(0, idx, wv)
            new[k] = acc / denom.reshape(-1, *[1] * (v.ndim - 1))
        return self.with_data(point_data=new)

    def point_data_to_cell_data(self, overwrite_keys: bool = False) -> "Mesh":
        new = {}
        for k, v in self.point_data.items():
            if not v.is_floating_point():
                continue
            if k in self.cell_data and not overwrite_keys:
                raise ValueError(f"cell_data already has key '{k}'; pass overwrite_keys=True to replace it")
            new[k] = v[self.cells].mean(dim=1)
        return self.with_data(cell_data=new)

    # ------------------------------------------------------------ slicing etc.
    def slice_cells(self, index) -> "Mesh":
        index = torch.as_tensor(index, device=self.device)
        return Mesh(self.points, self.cells[index], self.point_data, {k: v[index] for k, v in self.cell_data.items()},
                    self.global_data)

    def slice_points(self, index) -> "Mesh":
        """Keep the given points; cells with a dropped vertex are removed and the rest re-indexed."""
        index = torch.as_tensor(index, device=self.device)
        keep = torch.zeros(self.n_points, dtype=torch.bool, device=self.device)
        keep[index] = True
        new_id = torch.cumsum(keep, 0) - 1
        cell_ok = keep[self.cells].all(dim=1) if self.n_cells else torch.zeros(0, dtype=torch.bool, device=self.device)
        return Mesh(self.points[keep], new_id[self.cells[cell_ok]], {k: v[keep] for k, v in self.point_data.items()},
                    {k: v[cell_ok] for k, v in self.cell_data.items()}, self.global_data)

    @staticmethod
    def merge(meshes: Sequence["Mesh"], global_data_strategy: str = "first") -> "Mesh":
        if not meshes:
            raise ValueError("need at least one mesh to merge")
        first = meshes[0]
        for m in meshes[1:]:
            if m.n_spatial_dims != first.n_spatial_dims or m.n_manifold_dims != first.n_manifold_dims:
                raise ValueError("all meshes must share spatial and manifold dimensions")
        offs = [0]
        for m in meshes[:-1]:
            offs.append(offs[-1] + m.n_points)
        pk = set.intersection(*[set(m.point_data) for m in meshes])
        ck = set.intersection(*[set(m.cell_data) for m in meshes])
        return Mesh(torch.cat([m.points for m in meshes]), torch.cat([m.cells + o for m, o in zip(meshes, offs)]),
                    {k: torch.cat([m.point_data[k] for m in meshes]) for k in pk},
                    {k: torch.cat([m.cell_data[k] for m in meshes]) for k in ck}, first.global_data)

    def clean(self, tolerance: float = 1e-12, merge_points: bool = True, remove_degenerate_cells: bool = True,
              remove_unused_points: bool = True, remove_duplicate_cells: bool = True) -> "Mesh":
        """Weld coincident points, drop zero-measure / repeated-vertex / duplicate cells and unreferenced points."""
        m = self
        if merge_points and m.n_points:
            scale = max(tolerance, 1e-300)
            q = torch.round(m.points.double() / scale).long() if tolerance > 0 else m.points
            _, inverse = torch.unique(q, dim=0, return_inverse=True)
            first = torch.full((int(inverse.max()) + 1,), m.n_points, dtype=torch.long, device=m.device)
            first.scatter_reduce_(0, inverse, torch.arange(m.n_points, device=m.device), reduce="amin")
            order = torch.argsort(first)
            rank = torch.empty_like(order)
            rank[order] = torch.arange(order.numel(), device=m.device)
            keep = first[order]
            m = Mesh(m.points[keep], rank[inverse][m.cells], {k: v[keep] for k, v in m.point_data.items()}, m.cell_data, m.global_data)
        if m.n_cells:
            ok = torch.ones(m.n_cells, dtype=torch.bool, device=m.device)
            if remove_degenerate_cells:
                s = torch.sort(m.cells, dim=1).values
                ok &= (s[:, 1:] != s[:, :-1]).all(dim=1) if m.cells.shape[1] > 1 else ok
                ok &= m.cell_areas > 0
            if remove_duplicate_cells:
                s = torch.sort(m.cells, dim=1).values
                _, inv = torch.unique(s, dim=0, return_inverse=True)
                first = torch.full((int(inv.max()) + 1,), m.n_cells, dtype=torch.long, device=m.device)
                first.scatter_reduce_(0, inv, torch.arange(m.n_cells, device=m.device), reduce="amin")
                dup = torch.ones(m.n_cells, dtype=torch.bool, device=m.device)
                dup[first] = False
                ok &= ~dup
            m = m.slice_cells(ok)
        if remove_unused_points and m.n_cells:
            used = torch.zeros(m.n_points, dtype=torch.bool, device=m.device)
            used[m.cells.reshape(-1)] = True
            m = m.slice_points(torch.nonzero(used).squeeze(1))
        return m

    # ------------------------------------------------------------------ sampling
    def sample_random_points_on_cells(self, cell_indices=None, alpha: float = 1.0, generator=None) -> torch.Tensor:
        """One Dirichlet(α)-distributed point per listed cell (``α = 1``: uniform over the simplex)."""
        idx = torch.arange(self.n_cells, device=self.device) if cell_indices is None else torch.as_tensor(cell_indices, device=self.device)
        V = self.cells.shape[1]
        g = torch.empty(idx.numel(), V, dtype=self.points.dtype, device=self.device)
        if alpha == 1.0:
            g.exponential_(generator=generator)
        else:
            g = torch.distributions.Gamma(torch.full_like(g, alpha), torch.ones_like(g)).sample()
        bary = g / g.sum(dim=1, keepdim=True)
        return (bary[:, :, None] * self.points[self.cells[idx]]).sum(dim=1)

    def sample_points(self, n: int, generator=None) -> tuple[torch.Tensor, torch.Tensor]:
        """``n`` points distributed uniformly over the mesh (cells drawn ∝ measure); returns (points, cell index)."""
        cell = torch.multinomial(self.cell_areas.float().clamp_min(0), n, replacement=True, generator=generator)
        return self.sample_random_points_on_cells(cell, generator=generator), cell

    def sample_data_at_points(self, query_points: torch.Tensor, data_source: str = "cells") -> Dict[str, torch.Tensor]:
        """Values at arbitrary points: of the nearest cell (by centroid), or barycentric-free inverse-distance
        interpolation of that cell's vertices for ``data_source="points"``."""
        from ..nn.functional.neighbors import knn

        cell = knn(self.cell_centroids.float(), query_points.float(), k=1)[0][:, 0]
        if data_source == "cells":
            return {k: v[cell] for k, v in self.cell_data.items()}
        verts = self.cells[cell]
        d = (self.points[verts] - query_points[:, None]).norm(dim=-1).clamp_min(1e-12)
        w = (1 / d) / (1 / d).sum(dim=1, keepdim=True)
        return {k: (w.reshape(*w.shape, *[1] * (v.ndim - 1)) * v[verts]).sum(dim=1) for k, v in self.point_data.items()
                if v.is_floating_point()}

    # ------------------------------------------------------------ transformation
    def translate(self, offset) -> "Mesh":
        return self._with_points(self.points + torch.as_tensor(offset, dtype=self.points.dtype, device=self.device))

    def scale(self, factor, center=None) -> "Mesh":
        c = torch.zeros(self.n_spatial_dims, dtype=self.points.dtype, device=self.device) if center is None else torch.as_tensor(center, dtype=self.points.dtype, device=self.device)
        return self._with_points((self.points - c) * torch.as_tensor(factor, dtype=self.points.dtype, device=self.device) + c)

    def transform(self, matrix: torch.Tensor, transform_vectors: Sequence[str] = ()) -> "Mesh":
        """Apply a ``D×D`` linear or ``(D+1)×(D+1)`` homogeneous matrix; listed vector fields are rotated too."""
        A = torch.as_tensor(matrix, dtype=self.points.dtype, device=self.device)
        D = self.n_spatial_dims
        lin, shift = (A[:D, :D], A[:D, D]) if A.shape == (D + 1, D + 1) else (A, None)
        p = self.points @ lin.T
        out = self._with_points(p + shift if shift is not None else p)
        for k in transform_vectors:
            for store in (out.point_data, out.cell_data):
                if k in store:
                    store[k] = store[k] @ lin.T
        return out

    def rotate(self, angle: float, axis=None, center=None) -> "Mesh":
        D = self.n_spatial_dims
        c, s = math.cos(angle), math.sin(angle)
        if D == 2:
            R = torch.tensor([[c, -s], [s, c]])
        elif D == 3:
            a = torch.as_tensor([0.0, 0.0, 1.0] if axis is None else axis, dtype=torch.float64)
            a = a / a.norm()
            K = torch.tensor([[0, -a[2], a[1]], [a[2], 0, -a[0]], [-a[1], a[0], 0]], dtype=torch.float64)
            R = torch.eye(3, dtype=torch.float64) + s * K + (1 - c) * (K @ K)
        else:
            raise ValueError("rotate supports 2-D and 3-D meshes")
        R = R.to(self.points.dtype).to(self.device)
        ctr = torch.zeros(D, dtype=self.points.dtype, device=self.device) if center is None else torch.as_tensor(center, dtype=self.points.dtype, device=self.device)
        return self._with_points((self.points - ctr) @ R.T + ctr)

    def _with_points(self, points) -> "Mesh":
        return Mesh(points, self.cells, self.point_data, self.cell_data, self.global_data)

    # ---------------------------------------------------------------- refinement
    def subdivide(self, levels: int = 1, filter: str = "linear") -> "Mesh":
        """Midpoint subdivision of edges (→2), triangles (→4) or tetrahedra (→8); ``"loop"``-style smoothing is
        approximated by one Laplacian pass on the new vertices for ``filter != "linear"``."""
        m = self
        for _ in range(levels):
            m = _subdivide_once(m)
            if filter != "linear" and m.n_manifold_dims == 2:
                from .operations import laplacian_smooth

                m = laplacian_smooth(m, iterations=1, relaxation=0.25)
        return m

    # ------------------------------------------------------------------ calculus
    def _lsq(self, values: torch.Tensor, at: str) -> torch.Tensor:
        from ..nn.functional.derivatives import mesh_lsq_gradient

        if at == "points":
            adj = self.get_point_to_points_adjacency()
            return mesh_lsq_gradient(self.points, values, adj.offsets, adj.indices)
        adj = self.get_cell_to_cells_adjacency()
        return mesh_lsq_gradient(self.cell_centroids, values, adj.offsets, adj.indices)

    def gradient(self, key: str, data_source: str = "points", method: str = "lsq") -> torch.Tensor:
        """Gradient ``[n, D, ...]`` of a point or cell field (weighted least squares over the 1-ring; Green-Gauss for
        cell fields of full-dimensional meshes with ``method="green_gauss"``)."""
        if data_source == "points":
            return self._lsq(self.point_data[key], "points")
        if method == "green_gauss" and self.codimension == 0:
            from ..nn.functional.derivatives import mesh_green_gauss_gradient

            return mesh_green_gauss_gradient(self.points, self.cells, self.facet_neighbors(), self.cell_data[key])
        return self._lsq(self.cell_data[key], "cells")

    def divergence(self, key: str, data_source: str = "points") -> torch.Tensor:
        g = self.gradient(key, data_source)                               # [n, D, D]: d(component j)/d(x_i)
        return torch.diagonal(g, dim1=1, dim2=2).sum(-1)

    def curl(self, key: str, data_source: str = "points") -> torch.Tensor:
        g = self.gradient(key, data_source)
        if self.n_spatial_dims == 2:
            return g[:, 0, 1] - g[:, 1, 0]
        if self.n_spatial_dims != 3:
            raise ValueError("curl needs 2 or 3 spatial dimensions")
        return torch.stack([g[:, 1, 2] - g[:, 2, 1], g[:, 2, 0] - g[:, 0, 2], g[:, 0, 1] - g[:, 1, 0]], dim=-1)

    def laplacian(self, key: str, data_source: str = "points") -> torch.Tensor:
        """Cotangent Laplace–Beltrami on triangle meshes (point data), divergence of the LSQ gradient otherwise."""
        if data_source == "points" and self.n_manifold_dims == 2:
            from .operations import cotangent_laplacian

            return cotangent_laplacian(self, self.point_data[key])
        g = self._lsq(self.point_data[key] if data_source == "points" else self.cell_data[key], data_source)
        gg = self._lsq(g.reshape(g.shape[0], -1), data_source).reshape(g.shape[0], self.n_spatial_dims, *g.shape[1:])
        return torch.diagonal(gg, dim1=1, dim2=2).movedim(-1, 1).sum(1) if gg.ndim > 3 else torch.diagonal(gg, dim1=1, dim2=2).sum(-1)

    # ----------------------------------------------------------------- curvature
    @property
    def gaussian_curvature_vertices(self) -> torch.Tensor:
        """Angle defect divided by the barycentric vertex area (triangle meshes)."""
        from .operations import gaussian_curvature

        return self._cached("gauss_curv", lambda: gaussian_curvature(self))

    @property
    def mean_curvature_vertices(self) -> torch.Tensor:
        from .operations import mean_curvature

        return self._cached("mean_curv", lambda: mean_curvature(self))

    @property
    def gaussian_curvature_cells(self) -> torch.Tensor:
        return self.gaussian_curvature_vertices[self.cells].mean(dim=1)

    # ------------------------------------------------------------------- quality
    @property
    def quality_metrics(self) -> Dict[str, torch.Tensor]:
        p = self.points[self.cells]
        V = self.cells.shape[1]
        edges = torch.stack([(p[:, a] - p[:, b]).norm(dim=-1) for a, b in combinations(range(V), 2)], dim=1) if V > 1 else p.new_zeros(self.n_cells, 1)
        M = self.n_manifold_dims
        ideal = math.sqrt(M + 1) / (math.factorial(M) * 2 ** (M / 2)) if M else 1.0     # regular simplex measure at unit edge
        rms = edges.pow(2).mean(dim=1).sqrt().clamp_min(1e-30)
        return {"min_edge": edges.min(dim=1).values, "max_edge": edges.max(dim=1).values,
                "aspect_ratio": edges.max(dim=1).values / edges.min(dim=1).values.clamp_min(1e-30),
                "measure": self.cell_areas, "shape_quality": self.cell_areas / (ideal * rms ** M)}

    @property
    def statistics(self) -> Dict[str, Any]:
        q = self.quality_metrics
        return {"n_points": self.n_points, "n_cells": self.n_cells, "manifold_dim": self.n_manifold_dims,
                "spatial_dim": self.n_spatial_dims, "total_measure": float(self.cell_areas.sum()) if self.n_cells else 0.0,
                "bounds": (self.points.amin(0).tolist(), self.points.amax(0).tolist()) if self.n_points else None,
                "min_shape_quality": float(q["shape_quality"].min()) if self.n_cells else None,
                "mean_aspect_ratio": float(q["aspect_ratio"].mean()) if self.n_cells else None}

    def pad(self, target_n_points: int, target_n_cells: int, data_padding_value: float = 0.0) -> "Mesh":
        """Pad to fixed sizes (degenerate cells on the last point) so shapes stay static across samples."""
        if target_n_points < self.n_points or target_n_cells < self.n_cells:
            raise ValueError("targets must not be smaller than the current sizes")
        dp, dc = target_n_points - self.n_points, target_n_cells - self.n_cells
        padt = lambda t, n: torch.cat([t, t.new_full((n, *t.shape[1:]), data_padding_value)]) if n else t  # noqa: E731
        pts = torch.cat([self.points, self.points[-1:].expand(dp, -1)]) if dp else self.points
        cells = torch.cat([self.cells, self.cells.new_full((dc, self.cells.shape[1]), max(target_n_points - 1, 0))]) if dc else self.cells
        return Mesh(pts, cells, {k: padt(v, dp) for k, v in self.point_data.items()}, {k: padt(v, dc) for k, v in self.cell_data.items()},
                    self.global_data)

    def pad_to_next_power(self, power: float = 1.5, data_padding_value: float = 0.0) -> "Mesh":
        nxt = lambda n: n if n <= 1 else int(math.ceil(power ** math.ceil(math.log(n) / math.log(power))))  # noqa: E731
        return self.pad(nxt(self.n_points), nxt(self.n_cells), data_padding_value)


def _angle(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    cosv = (a * b).sum(-1) / (a.norm(dim=-1) * b.norm(dim=-1)).clamp_min(1e-30)
    return torch.acos(cosv.clamp(-1, 1))


def _subdivide_once(m: Mesh) -> Mesh:
    M = m.n_manifold_dims
    if M == 0 or m.n_cells == 0:
        return m
    edges = m.to_edge_graph().cells
    key = torch.sort(edges, dim=1).values
    P = m.n_points
    mid = 0.5 * (m.points[key[:, 0]] + m.points[key[:, 1]])
    codes = key[:, 0] * P + key[:, 1]
    order = torch.argsort(codes)
    codes_sorted = codes[order]

    def mid_id(a, b):
        lo, hi = torch.minimum(a, b), torch.maximum(a, b)
        return P + order[torch.searchsorted(codes_sorted, lo * P + hi)]

    c = m.cells
    if M == 1:
        ab = mid_id(c[:, 0], c[:, 1])
        new = torch.cat([torch.stack([c[:, 0], ab], 1), torch.stack([ab, c[:, 1]], 1)])
        reps = 2
    elif M == 2:
        a, b, d = c[:, 0], c[:, 1], c[:, 2]
        ab, bd, da = mid_id(a, b), mid_id(b, d), mid_id(d, a)
        new = torch.cat([torch.stack([a, ab, da], 1), torch.stack([ab, b, bd], 1), torch.stack([da, bd, d], 1), torch.stack([ab, bd, da], 1)])
        reps = 4
    elif M == 3:
        v = [c[:, i] for i in range(4)]
        e = {(i, j): mid_id(v[i], v[j]) for i, j in combinations(range(4), 2)}
        t = lambda *ids: torch.stack(ids, 1)  # noqa: E731
        new = torch.cat([t(v[0], e[0, 1], e[0, 2], e[0, 3]), t(e[0, 1], v[1], e[1, 2], e[1, 3]), t(e[0, 2], e[1, 2], v[2], e[2, 3]),
                         t(e[0, 3], e[1, 3], e[2, 3], v[3]), t(e[0, 1], e[0, 2], e[0, 3], e[1, 3]), t(e[0, 1], e[0, 2], e[1, 2], e[1, 3]),
                         t(e[0, 2], e[0, 3], e[1, 3], e[2, 3]), t(e[0, 2], e[1, 2], e[1, 3], e[2, 3])])
        reps = 8
    else:
        raise NotImplementedError("subdivision is implemented for manifold dimensions 1-3")
    pd = {k: torch.cat([v, 0.5 * (v[key[:, 0]] + v[key[:, 1]])]) for k, v in m.point_data.items() if v.is_floating_point()}
    cd = {k: v.repeat(reps, *[1] * (v.ndim - 1)) for k, v in m.cell_data.items()}
    return Mesh(torch.cat([m.points, mid]), new, pd, cd, m.global_data)
