"""Transforms and augmentations that act on ``Mesh`` objects inside a datapipe.

Parity: ``physicsnemo/datapipes/transforms/mesh/{base,transforms,augmentations}.py``: deterministic geometry transforms
(scale, translate, rotate, centre, subsample), field bookkeeping (drop, rename, set global, normalise from statistics),
derived fields (surface normals, cell centroids), conversion to a plain nested dict of tensors, and random augmentations
whose generator is re-seeded per epoch.  Vector-valued fields (trailing dimension = spatial dimension) follow the geometry
when the corresponding ``transform_*_data`` flag is set: rotations rotate them, scalings leave directions alone.
"""
from __future__ import annotations

import json
import math
from abc import ABC, abstractmethod
from typing import Literal, Optional

import torch

from ..._rng import derive_seed  # noqa: F401  (re-exported for subclasses)
from ....mesh import Mesh


class MeshTransform(ABC):
    def __init__(self) -> None:
        self._device: Optional[torch.device] = None

    @abstractmethod
    def __call__(self, mesh: Mesh) -> Mesh: ...

    def apply_to_domain(self, domain):
        return domain.apply_to_meshes(self)

    @property
    def stochastic(self) -> bool:
        return hasattr(self, "_generator")

    def set_generator(self, generator: torch.Generator) -> None:
        if self.stochastic:
            self._generator, self._seed_base = generator, generator.initial_seed()

    def set_epoch(self, epoch: int) -> None:
        if self.stochastic and self._generator is not None:
            if getattr(self, "_seed_base", None) is None:
                self._seed_base = self._generator.initial_seed()
            self._generator.manual_seed(derive_seed(self._seed_base, epoch))

    def to(self, device) -> "MeshTransform":
        self._device = torch.device(device)
        for name, value in list(self.__dict__.items()):
            if isinstance(value, torch.Tensor):
                setattr(self, name, value.to(self._device))
            elif isinstance(value, torch.Generator):
                gen = torch.Generator(device=self._device)
                gen.manual_seed(value.initial_seed())
                setattr(self, name, gen)
        return self

    @property
    def device(self):
        return self._device

    def extra_repr(self) -> str:
        return ""

    def __repr__(self) -> str:
        return f"{type(self).__name__}({self.extra_repr()})"


def _map_vectors(mesh: Mesh, fn, point: bool, cell: bool, glob: bool) -> Mesh:
    D = mesh.points.shape[-1]
    for store, on in ((mesh.point_data, point), (mesh.cell_data, cell), (mesh.global_data, glob)):
        if on:
            for k, v in list(store.items()):
                if v.is_floating_point() and v.ndim >= 1 and v.shape[-1] == D:
                    store[k] = fn(v)
    return mesh


def _rotation_matrix(angle, axis, D: int, dtype, device) -> torch.Tensor:
    c, s = math.cos(float(angle)), math.sin(float(angle))
    if D == 2:
        return torch.tensor([[c, -s], [s, c]], dtype=dtype, device=device)
    if isinstance(axis, str):
        axis = {"x": [1.0, 0, 0], "y": [0, 1.0, 0], "z": [0, 0, 1.0]}[axis]
    a = torch.as_tensor([0.0, 0.0, 1.0] if axis is None else axis, dtype=torch.float64)
    a = a / a.norm()
    K = torch.tensor([[0, -a[2], a[1]], [a[2], 0, -a[0]], [-a[1], a[0], 0]], dtype=torch.float64)
    return (torch.eye(3, dtype=torch.float64) + s * K + (1 - c) * (K @ K)).to(dtype=dtype, device=device)   # Rodrigues


class ScaleMesh(MeshTransform):
    def __init__(self, factor, transform_point_data=False, transform_cell_data=False, transform_global_data=False) -> None:
        super().__init__()
        self.factor, self.flags = factor, (transform_point_data, transform_cell_data, transform_global_data)

    def __call__(self, mesh: Mesh) -> Mesh:
        f = torch.as_tensor(self.factor, dtype=mesh.points.dtype, device=mesh.points.device)
        return _map_vectors(mesh.scale(f), lambda v: v * f.to(v.dtype), *self.flags)


class TranslateMesh(MeshTransform):
    def __init__(self, vector) -> None:
        super().__init__()
        self.vector = torch.as_tensor(vector, dtype=torch.float32)

    def __call__(self, mesh: Mesh) -> Mesh:
        return mesh.translate(self.vector.to(mesh.points))


class RotateMesh(MeshTransform):
    def __init__(self, angle: float, axis=None, center=None, transform_point_data=False, transform_cell_data=False,
                 transform_global_data=False) -> None:
        super().__init__()
        self.angle, self.axis, self.center = angle, axis, center
        self.flags = (transform_point_data, transform_cell_data, transform_global_data)

    def __call__(self, mesh: Mesh) -> Mesh:
        p = mesh.points
        R = _rotation_matrix(self.angle, self.axis, p.shape[-1], p.dtype, p.device)
        c = torch.zeros(p.shape[-1], dtype=p.dtype, device=p.device) if self.center is None else torch.as_tensor(self.center, dtype=p.dtype, device=p.device)
        out = mesh.translate(-c).transform(R).translate(c)
        return _map_vectors(out, lambda v: v @ R.to(v.dtype).T, *self.flags)


class CenterMesh(MeshTransform):
    """Move the (area-weighted) centroid to the origin."""

    def __init__(self, use_area_weighting: bool = True) -> None:
        super().__init__()
        self.use_area_weighting = use_area_weighting

    def __call__(self, mesh: Mesh) -> Mesh:
        if self.use_area_weighting and mesh.n_cells > 0:
            w = mesh.cell_areas.unsqueeze(-1) if hasattr(mesh, "cell_areas") else None
            cen = mesh.cell_centroids
            centre = (cen * w).sum(0) / w.sum().clamp_min(1e-30) if w is not None else cen.mean(0)
        else:
            centre = mesh.points.mean(0)
        return mesh.translate(-centre)


class SubsampleMesh(MeshTransform):
    """Keep ``n_cells`` random cells (optionally dropping unused points) or ``n_points`` random points of a point cloud."""

    def __init__(self, n_cells: int | None = None, n_points: int | None = None, compact: bool = True, seed: int = 0) -> None:
        super().__init__()
        if (n_cells is None) == (n_points is None):
            raise ValueError("exactly one of n_cells and n_points must be given")
        self.n_cells, self.n_points, self.compact = n_cells, n_points, compact
        self._generator = torch.Generator().manual_seed(seed)

    def __call__(self, mesh: Mesh) -> Mesh:
        gen = self._generator
        if self.n_cells is not None:
            if mesh.n_cells <= self.n_cells:
                return mesh
            idx = torch.randperm(mesh.n_cells, generator=gen, device=gen.device)[:self.n_cells].to(mesh.points.device)
            out = mesh.slice_cells(idx)
            if self.compact:
                used, inv = torch.unique(out.cells, return_inverse=True)
                out = Mesh(out.points[used], inv.reshape(out.cells.shape), {k: v[used] for k, v in out.point_data.items()}, dict(out.cell_data),
                           dict(out.global_data))
            return out
        if mesh.n_points <= self.n_points:
            return mesh
        idx = torch.randperm(mesh.n_points, generator=gen, device=gen.device)[:self.n_points].to(mesh.points.device)
        return mesh.slice_points(idx)


class DropMeshFields(MeshTransform):
    def __init__(self, point_data=None, cell_data=None, global_data=None) -> None:
        super().__init__()
        self.names = {"point_data": list(point_data or []), "cell_data": list(cell_data or []), "global_data": list(global_data or [])}

    def __call__(self, mesh: Mesh) -> Mesh:
        for store, names in self.names.items():
            for n in names:
                getattr(mesh, store).pop(n, None)
        return mesh


class RenameMeshFields(MeshTransform):
    def __init__(self, point_data=None, cell_data=None, global_data=None) -> None:
        super().__init__()
        self.maps = {"point_data": dict(point_data or {}), "cell_data": dict(cell_data or {}), "global_data": dict(global_data or {})}

    def __call__(self, mesh: Mesh) -> Mesh:
        for store, mapping in self.maps.items():
            d = getattr(mesh, store)
            for old, new in mapping.items():
                if old in d:
                    d[new] = d.pop(old)
        return mesh


class SetGlobalField(MeshTransform):
    def __init__(self, fields: dict) -> None:
        super().__init__()
        self.fields = {k: torch.as_tensor(v, dtype=torch.float32) if not isinstance(v, torch.Tensor) else v for k, v in fields.items()}

    def __call__(self, mesh: Mesh) -> Mesh:
        for k, v in self.fields.items():
            mesh.global_data[k] = v.to(mesh.points.device)
        return mesh


class NormalizeMeshFields(MeshTransform):
    """``(x − mean) / (std + eps)`` (or min-max to ``[-1, 1]``) per named field; statistics inline or from a JSON file."""

    def __init__(self, association: str = "point_data", fields: dict | None = None, stats_file: str | None = None, eps: float = 1e-8) -> None:
        super().__init__()
        association = getattr(association, "value", association)
        if association not in ("point_data", "cell_data", "global_data"):
            raise ValueError(f"unknown association {association!r}")
        if (fields is None) == (stats_file is None):
            raise ValueError("give exactly one of fields and stats_file")
        if stats_file is not None:
            with open(stats_file) as f:
                fields = json.load(f)
        self.association, self.eps = association, eps
        self.fields = {k: {s: torch.as_tensor(v, dtype=torch.float32) for s, v in st.items()} for k, st in fields.items()}

    def _apply(self, mesh: Mesh, inverse: bool) -> Mesh:
        store = getattr(mesh, self.association)
        for name, st in self.fields.items():
            if name not in store:
                continue
            x = store[name]
            st = {k: v.to(x) for k, v in st.items()}
            if "mean" in st:
                store[name] = x * (st["std"] + self.eps) + st["mean"] if inverse else (x - st["mean"]) / (st["std"] + self.eps)
            elif "min" in st:
                span = st["max"] - st["min"] + self.eps
                store[name] = (x + 1) * 0.5 * span + st["min"] if inverse else 2 * (x - st["min"]) / span - 1
            else:
                raise ValueError(f"statistics of {name!r} need mean/std or min/max")
        return mesh

    def __call__(self, mesh: Mesh) -> Mesh:
        return self._apply(mesh, False)

    def inverse(self, mesh: Mesh) -> Mesh:
        return self._apply(mesh, True)


class ComputeSurfaceNormals(MeshTransform):
    def __init__(self, store_as: Literal["cell_data", "point_data"] = "cell_data", field_name: str = "normals") -> None:
        super().__init__()
        if store_as not in ("cell_data", "point_data"):
            raise ValueError("store_as must be 'cell_data' or 'point_data'")
        self.store_as, self.field_name = store_as, field_name

    def __call__(self, mesh: Mesh) -> Mesh:
        getattr(mesh, self.store_as)[self.field_name] = mesh.cell_normals if self.store_as == "cell_data" else mesh.point_normals
        return mesh


class ComputeCellCentroids(MeshTransform):
    def __init__(self, field_name: str = "centroids") -> None:
        super().__init__()
        self.field_name = field_name

    def __call__(self, mesh: Mesh) -> Mesh:
        mesh.cell_data[self.field_name] = mesh.cell_centroids
        return mesh


class MeshToTensorDict(MeshTransform):
    """Plain nested dict ``{"points", "cells", "point_data": {...}, "cell_data": {...}, "global_data": {...}}``."""

    def __call__(self, mesh: Mesh) -> dict:
        return {"points": mesh.points, "cells": mesh.cells, "point_data": dict(mesh.point_data), "cell_data": dict(mesh.cell_data),
                "global_data": dict(mesh.global_data)}


class RestructureTensorDict(MeshTransform):
    """Regroup a nested dict: ``groups = {"inputs": {"pos": "points", "p": "point_data.pressure"}, ...}``."""

    def __init__(self, groups: dict) -> None:
        super().__init__()
        self.groups = groups

    def __call__(self, td: dict) -> dict:
        def resolve(path):
            node = td
            for part in path.split("."):
                node = node[part]
            return node

        return {g: {new: resolve(path) for new, path in mapping.items()} for g, mapping in self.groups.items()}


# ---- augmentations -----------------------------------------------------------------------------------------------------
def _sample(dist, shape, generator) -> torch.Tensor:
    """Sample a ``torch.distributions`` object reproducibly from ``generator`` via the inverse CDF."""
    u = torch.rand(shape, generator=generator, device=generator.device).clamp(1e-6, 1 - 1e-6)
    try:
        return dist.icdf(u.to(dist.mean.device if hasattr(dist.mean, "device") else u.device))
    except NotImplementedError as e:
        raise ValueError(f"{type(dist).__name__} has no inverse CDF; use Uniform, Normal, LogNormal, …") from e


class RandomScaleMesh(MeshTransform):
    def __init__(self, distribution=None, transform_point_data=False, transform_cell_data=False, transform_global_data=False, seed: int = 0) -> None:
        super().__init__()
        self.distribution = distribution if distribution is not None else torch.distributions.Uniform(0.9, 1.1)
        self.flags = (transform_point_data, transform_cell_data, transform_global_data)
        self._generator = torch.Generator().manual_seed(seed)

    def __call__(self, mesh: Mesh) -> Mesh:
        f = _sample(self.distribution, (), self._generator).to(mesh.points)
        return _map_vectors(mesh.scale(f), lambda v: v * f.to(v.dtype), *self.flags)


class RandomTranslateMesh(MeshTransform):
    def __init__(self, distribution=None, seed: int = 0) -> None:
        super().__init__()
        self.distribution = distribution if distribution is not None else torch.distributions.Uniform(-0.1, 0.1)
        self._generator = torch.Generator().manual_seed(seed)

    def __call__(self, mesh: Mesh) -> Mesh:
        return mesh.translate(_sample(self.distribution, (mesh.points.shape[-1],), self._generator).to(mesh.points))


class RandomRotateMesh(MeshTransform):
    """``uniform``: a rotation drawn uniformly from SO(3) (angle-distribution ignored); ``axis_aligned``: an angle from
    ``distribution`` (default uniform in [−π, π)) about one of ``axes`` chosen at random."""

    def __init__(self, axes=None, distribution=None, mode: Literal["axis_aligned", "uniform"] = "uniform", transform_point_data=False,
                 transform_cell_data=False, transform_global_data=False, seed: int = 0) -> None:
        super().__init__()
        if mode not in ("axis_aligned", "uniform"):
            raise ValueError("mode must be 'axis_aligned' or 'uniform'")
        self.axes, self.mode = list(axes) if axes is not None else ["x", "y", "z"], mode
        self.distribution = distribution if distribution is not None else torch.distributions.Uniform(-math.pi, math.pi)
        self.flags = (transform_point_data, transform_cell_data, transform_global_data)
        self._generator = torch.Generator().manual_seed(seed)

    def __call__(self, mesh: Mesh) -> Mesh:
        p, gen = mesh.points, self._generator
        D = p.shape[-1]
        if D == 3 and self.mode == "uniform":
            q = torch.randn(4, generator=gen, device=gen.device, dtype=torch.float64)
            w, x, y, z = (q / q.norm()).tolist()                      # a normalised Gaussian quaternion is uniform on SO(3)
            R = torch.tensor([[1 - 2 * (y * y + z * z), 2 * (x * y - z * w), 2 * (x * z + y * w)],
                              [2 * (x * y + z * w), 1 - 2 * (x * x + z * z), 2 * (y * z - x * w)],
                              [2 * (x * z - y * w), 2 * (y * z + x * w), 1 - 2 * (x * x + y * y)]], dtype=p.dtype, device=p.device)
        else:
            angle = float(_sample(self.distribution, (), gen))
            axis = self.axes[int(torch.randint(len(self.axes), (1,), generator=gen, device=gen.device))] if D == 3 else None
            R = _rotation_matrix(angle, axis, D, p.dtype, p.device)
        return _map_vectors(mesh.transform(R), lambda v: v @ R.to(v.dtype).T, *self.flags)
