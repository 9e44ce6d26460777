"""The standard transform set.

Parity: ``physicsnemo/datapipes/transforms/{normalize,subsample,concat_fields,field_slice,field_processing,geometric,
spatial,utility}.py`` — every transform maps a ``TensorDict`` to a ``TensorDict`` (updated in place and returned),
keeps its constants on the dataset's device, and — when stochastic — draws from a generator seeded per
(epoch, position in the pipeline).
"""
from __future__ import annotations

import warnings
from pathlib import Path
from typing import Any, Literal, Optional

import numpy as np
import torch

from ...nn.functional.neighbors import knn
from ...nn.functional.weighted_multinomial import weighted_multinomial
from ..registry import register
from ..tensordict import TensorDict
from .base import Transform


def _need(data, key, what="Field"):
    if key not in data.keys():
        raise KeyError(f"{what} '{key}' not found in data. Available: {list(data.keys())}")
    return data[key]


# ------------------------------------------------------------------- normalisation
@register()
class Normalize(Transform):
    """``(x − mean) / (std + eps)`` or ``(x − centre) / (half range + eps)`` per field; ``inverse`` undoes it."""

    def __init__(self, input_keys: list[str], means=None, stds=None, *, method: Optional[Literal["mean_std", "min_max"]] = None,
                 mins=None, maxs=None, stats_file: Optional[str | Path] = None, eps: float = 1e-8) -> None:
        super().__init__()
        if not input_keys:
            raise ValueError("input_keys cannot be empty")
        self.input_keys, self.eps = list(input_keys), eps
        if means is not None and stds is not None and method is None:
            warnings.warn("Providing 'means' and 'stds' without 'method' parameter is deprecated. Please specify "
                          "method='mean_std' explicitly. This will become an error in a future version.",
                          DeprecationWarning, stacklevel=2)
            method = "mean_std"
        if method not in ("mean_std", "min_max"):
            raise ValueError(f"method must be 'mean_std' or 'min_max', got: {method}")
        self.method = method
        if stats_file is not None:
            stats = self._load_stats_from_npz(stats_file)
            means = stats["means"] if means is None else means
            stds = stats["stds"] if stds is None else stds
            mins = stats["mins"] if mins is None else mins
            maxs = stats["maxs"] if maxs is None else maxs
        self._means = self._stds = self._mins = self._maxs = None
        if method == "mean_std":
            if means is None or stds is None:
                raise ValueError("For method='mean_std', both 'means' and 'stds' must be provided either directly or via stats_file")
            self._means, self._stds = self._per_key(means, "mean"), self._per_key(stds, "std")
        else:
            if mins is None or maxs is None:
                raise ValueError("For method='min_max', both 'mins' and 'maxs' must be provided either directly or via stats_file")
            self._mins, self._maxs = self._per_key(mins, "min"), self._per_key(maxs, "max")

    def _per_key(self, stats, name) -> dict[str, torch.Tensor]:
        if isinstance(stats, dict):
            for k in self.input_keys:
                if k not in stats:
                    raise ValueError(f"{name.capitalize()} not provided for field '{k}'")
            return {k: torch.as_tensor(stats[k]) for k in self.input_keys}
        t = torch.as_tensor(stats)
        return {k: t.clone() for k in self.input_keys}

    def _load_stats_from_npz(self, stats_file) -> dict[str, dict]:
        path = Path(stats_file)
        if not path.exists():
            raise FileNotFoundError(f"Statistics file not found: {stats_file}")
        raw = np.load(str(path), allow_pickle=True)
        out = {"means": {}, "stds": {}, "mins": {}, "maxs": {}}
        for k in self.input_keys:
            if k not in raw:
                raise ValueError(f"Field '{k}' not found in stats file. Available fields: {list(raw.keys())}")
            entry = raw[k]
            if isinstance(entry, np.ndarray) and entry.dtype == object:
                entry = entry.item()
            for short, long in (("mean", "means"), ("std", "stds"), ("min", "mins"), ("max", "maxs")):
                if short in entry:
                    out[long][k] = torch.as_tensor(entry[short])
        return out

    def _affine(self, key):
        if self.method == "mean_std":
            return self._means[key], self._stds[key] + self.eps
        lo, hi = self._mins[key], self._maxs[key]
        return (hi + lo) / 2.0, (hi - lo) / 2.0 + self.eps

    def __call__(self, data: TensorDict) -> TensorDict:
        upd = {}
        for k in self.input_keys:
            shift, scale = self._affine(k)
            upd[k] = (_need(data, k) - shift) / scale
        return data.update(upd)

    def inverse(self, data: TensorDict) -> TensorDict:
        upd = {}
        for k in self.input_keys:
            shift, scale = self._affine(k)
            upd[k] = _need(data, k) * scale + shift
        return data.update(upd)

    def state_dict(self) -> dict[str, Any]:
        sd = {"input_keys": self.input_keys, "method": self.method, "eps": self.eps}
        pairs = (("means", self._means), ("stds", self._stds)) if self.method == "mean_std" else (("mins", self._mins), ("maxs", self._maxs))
        for name, table in pairs:
            sd[name] = {k: v.cpu() for k, v in table.items()}
        return sd

    def load_state_dict(self, sd: dict[str, Any]) -> None:
        self.input_keys, self.method, self.eps = sd["input_keys"], sd.get("method", "mean_std"), sd["eps"]
        get = lambda n: {k: v.clone() for k, v in sd[n].items()} if n in sd else None  # noqa: E731
        self._means, self._stds, self._mins, self._maxs = get("means"), get("stds"), get("mins"), get("maxs")

    def extra_repr(self) -> str:
        return f"keys={self.input_keys}, method={self.method}"


# --------------------------------------------------------------------- sub-sampling
def shuffle_array(points: torch.Tensor, n_points: int, weights: Optional[torch.Tensor] = None, generator=None):
    """``(points[idx], idx)`` for ``n_points`` indices drawn without replacement (all points when fewer exist)."""
    N = points.shape[0]
    if N < n_points:
        return points, torch.arange(N, device=points.device)
    strategy = "poisson_gap" if weights is None and N > 2 ** 24 and n_points < N else "exact"
    idx = weighted_multinomial(weights if weights is not None else N, n_points, strategy=strategy, device=points.device,
                               generator=generator)
    return points[idx], idx


@register()
class SubsamplePoints(Transform):
    def __init__(self, input_keys: list[str], n_points: int, *, algorithm: Literal["poisson_fixed", "uniform"] = "poisson_fixed",
                 weights_key: Optional[str] = None) -> None:
        super().__init__()
        self.input_keys, self.n_points, self.algorithm, self.weights_key = input_keys, n_points, algorithm, weights_key
        self._generator: torch.Generator | None = None

    def __call__(self, data: TensorDict) -> TensorDict:
        if not self.input_keys:
            return data
        first = _need(data, self.input_keys[0], "Key")
        N = first.shape[0]
        for k in self.input_keys[1:]:
            if _need(data, k, "Key").shape[0] != N:
                raise ValueError(f"All keys must have the same first dimension. Key '{self.input_keys[0]}' has {N}, but '{k}' has {data[k].shape[0]}")
        if N <= self.n_points:
            return data
        if self.weights_key is not None:
            _, idx = shuffle_array(first, self.n_points, weights=_need(data, self.weights_key, "Weights key"), generator=self._generator)
        else:
            strategy = "poisson_gap" if (self.algorithm == "poisson_fixed" and N > 2 ** 24) else "exact"
            idx = weighted_multinomial(N, self.n_points, strategy=strategy, device=first.device, generator=self._generator)
        return data.update({k: data[k][idx] for k in self.input_keys})

    def extra_repr(self) -> str:
        w = f", weights_key={self.weights_key}" if self.weights_key else ""
        return f"input_keys={self.input_keys}, n_points={self.n_points}, algorithm={self.algorithm}{w}"


# ------------------------------------------------------------------ field utilities
@register()
class ConcatFields(Transform):
    def __init__(self, input_keys: list[str], output_key: str, *, dim: int = -1, skip_missing: bool = False) -> None:
        super().__init__()
        self.input_keys, self.output_key, self.dim, self.skip_missing = input_keys, output_key, dim, skip_missing

    def __call__(self, data: TensorDict) -> TensorDict:
        parts = []
        for k in self.input_keys:
            if k not in data.keys():
                if self.skip_missing:
                    continue
                raise KeyError(f"Field '{k}' not found in data. Available: {list(data.keys())}")
            t = data[k]
            parts.append(t.unsqueeze(-1) if t.ndim == 1 else t)
        if not parts:
            raise ValueError("No fields to concatenate")
        return data.update({self.output_key: torch.cat(parts, dim=self.dim)})


@register()
class FieldSlice(Transform):
    """``slicing = {field: {dim: [indices] | {"start", "stop", "step"}}}``."""

    def __init__(self, slicing: dict) -> None:
        super().__init__()
        self.slicing = slicing

    def __call__(self, data: TensorDict) -> TensorDict:
        upd = {}
        for name, dims in self.slicing.items():
            t = _need(data, name)
            for dim_key, spec in dims.items():
                d = int(dim_key) % t.ndim
                if isinstance(spec, (list, tuple)):
                    t = torch.index_select(t, d, torch.tensor(list(spec), dtype=torch.long, device=t.device))
                elif isinstance(spec, dict):
                    idx = [slice(None)] * t.ndim
                    idx[d] = slice(spec.get("start"), spec.get("stop"), spec.get("step"))
                    t = t[tuple(idx)]
                else:
                    raise TypeError(f"Invalid slice spec type: {type(spec)}. Expected list of indices or dict with start/stop/step.")
            upd[name] = t
        return data.update(upd)

    def extra_repr(self) -> str:
        return f"slicing={self.slicing}"


@register()
class BroadcastGlobalFeatures(Transform):
    """Tile per-sample scalars / vectors to every point: ``[n_points, Σ dims]``."""

    def __init__(self, input_keys: list[str], n_points_key: str, output_key: str) -> None:
        super().__init__()
        self.input_keys, self.n_points_key, self.output_key = input_keys, n_points_key, output_key

    def __call__(self, data: TensorDict) -> TensorDict:
        n = _need(data, self.n_points_key).shape[0]
        feats = torch.cat([_need(data, k).reshape(-1) for k in self.input_keys])
        return data.update({self.output_key: feats.unsqueeze(0).expand(n, -1).contiguous()})


@register()
class Rename(Transform):
    def __init__(self, mapping: dict[str, str], *, strict: bool = True) -> None:
        super().__init__()
        self.mapping, self.strict = mapping, strict

    def __call__(self, data: TensorDict) -> TensorDict:
        for old, new in self.mapping.items():
            if old not in data.keys():
                if self.strict:
                    raise KeyError(f"Key '{old}' not found in data. Available: {list(data.keys())}")
                continue
            data.rename_key_(old, new)
        return data


@register()
class Purge(Transform):
    def __init__(self, *, keep_only: Optional[list[str]] = None, drop_only: Optional[list[str]] = None, strict: bool = True) -> None:
        super().__init__()
        if (keep_only is None) == (drop_only is None):
            raise ValueError("Exactly one of keep_only / drop_only must be given")
        self.keep_only, self.drop_only, self.strict = keep_only, drop_only, strict

    def __call__(self, data: TensorDict) -> TensorDict:
        names = self.keep_only if self.keep_only is not None else self.drop_only
        missing = [k for k in names if k not in data.keys()]
        if missing and self.strict:
            raise KeyError(f"Keys {missing} not found in data. Available: {list(data.keys())}")
        if self.keep_only is not None:
            return data.select(*[k for k in self.keep_only if k in data.keys()])
        return data.exclude(*self.drop_only)


@register()
class ConstantField(Transform):
    def __init__(self, reference_key: str, output_key: str, *, fill_value: float = 0.0, output_dim: int = 1) -> None:
        super().__init__()
        self.reference_key, self.output_key, self.fill_value, self.output_dim = reference_key, output_key, fill_value, output_dim

    def __call__(self, data: TensorDict) -> TensorDict:
        ref = _need(data, self.reference_key)
        return data.update({self.output_key: torch.full((ref.shape[0], self.output_dim), self.fill_value, dtype=ref.dtype, device=ref.device)})


# ----------------------------------------------------------------------- geometry
@register()
class Translate(Transform):
    def __init__(self, input_keys: list[str], center_key_or_value, *, subtract: bool = False) -> None:
        super().__init__()
        self.input_keys, self.subtract = input_keys, subtract
        self.center_key = center_key_or_value if isinstance(center_key_or_value, str) else None
        self.center_value = None if self.center_key else torch.as_tensor(center_key_or_value)

    def __call__(self, data: TensorDict) -> TensorDict:
        c = _need(data, self.center_key) if self.center_key else self.center_value
        return data.update({k: (_need(data, k) - c if self.subtract else data[k] + c) for k in self.input_keys})


@register()
class Scale(Transform):
    def __init__(self, input_keys: list[str], scale: torch.Tensor, *, divide: bool = False) -> None:
        super().__init__()
        self.input_keys, self.scale, self.divide = input_keys, torch.as_tensor(scale), divide

    def __call__(self, data: TensorDict) -> TensorDict:
        return data.update({k: (_need(data, k) / self.scale if self.divide else data[k] * self.scale) for k in self.input_keys})


@register()
class BoundingBoxFilter(Transform):
    """Keep the points inside ``[bbox_min, bbox_max]`` for ``input_keys`` and, with the same mask, ``dependent_keys``."""

    def __init__(self, input_keys: list[str], bbox_min, bbox_max, *, dependent_keys: Optional[list[str]] = None) -> None:
        super().__init__()
        self.input_keys, self.dependent_keys = input_keys, dependent_keys or []
        self.bbox_min, self.bbox_max = torch.as_tensor(bbox_min), torch.as_tensor(bbox_max)

    def __call__(self, data: TensorDict) -> TensorDict:
        upd = {}
        for k in self.input_keys:
            p = _need(data, k)
            keep = ((p >= self.bbox_min) & (p <= self.bbox_max)).all(dim=-1)
            upd[k] = p[keep]
            for d in self.dependent_keys:
                if d in data.keys() and data[d].shape[0] == p.shape[0]:
                    upd[d] = data[d][keep]
        return data.update(upd)


@register()
class CreateGrid(Transform):
    def __init__(self, output_key: str, resolution: tuple[int, int, int], bbox_min, bbox_max) -> None:
        super().__init__()
        self.output_key, self.resolution = output_key, tuple(resolution)
        self.bbox_min, self.bbox_max = torch.as_tensor(bbox_min, dtype=torch.float32), torch.as_tensor(bbox_max, dtype=torch.float32)

    def __call__(self, data: TensorDict) -> TensorDict:
        axes = [torch.linspace(float(lo), float(hi), n, device=self.bbox_min.device)
                for lo, hi, n in zip(self.bbox_min, self.bbox_max, self.resolution)]
        return data.update({self.output_key: torch.stack(torch.meshgrid(*axes, indexing="ij"), dim=-1)})


@register()
class KNearestNeighbors(Transform):
    """Adds ``{prefix}_indices``, ``{prefix}_distances`` and, for each ``extract_keys`` field, ``{prefix}_{key}``."""

    def __init__(self, points_key: str, queries_key: str, k: int, *, output_prefix: str = "neighbors",
                 extract_keys: Optional[list[str]] = None, drop_first_neighbor: bool = False) -> None:
        super().__init__()
        self.points_key, self.queries_key, self.k = points_key, queries_key, k
        self.output_prefix, self.extract_keys, self.drop_first_neighbor = output_prefix, extract_keys or [], drop_first_neighbor

    def __call__(self, data: TensorDict) -> TensorDict:
        pts, qs = _need(data, self.points_key), _need(data, self.queries_key)
        k = self.k + 1 if self.drop_first_neighbor else self.k
        idx, dist = knn(pts.float(), qs.float(), k=k)
        if self.drop_first_neighbor:
            idx, dist = idx[:, 1:], dist[:, 1:]
        upd = {f"{self.output_prefix}_indices": idx, f"{self.output_prefix}_distances": dist}
        for key in self.extract_keys:
            upd[f"{self.output_prefix}_{key}"] = _need(data, key)[idx]
        return data.update(upd)


@register()
class CenterOfMass(Transform):
    def __init__(self, coords_key: str, output_key: str, *, areas_key: str | None = None) -> None:
        super().__init__()
        self.coords_key, self.output_key, self.areas_key = coords_key, output_key, areas_key

    def __call__(self, data: TensorDict) -> TensorDict:
        x = _need(data, self.coords_key)
        if self.areas_key is None:
            com = x.mean(dim=0, keepdim=True)
        else:
            a = _need(data, self.areas_key).reshape(-1, 1)
            com = (x * a).sum(dim=0, keepdim=True) / a.sum()
        return data.update({self.output_key: com})


@register()
class ComputeSDF(Transform):
    """Signed distance (and optionally closest points) of query fields to a triangle mesh held in the sample."""

    def __init__(self, input_keys: list[str], output_key: str, mesh_coords_key: str, mesh_faces_key: str, *,
                 use_winding_number: bool = True, closest_points_key: Optional[str] = None) -> None:
        super().__init__()
        self.input_keys, self.output_key = input_keys, output_key
        self.mesh_coords_key, self.mesh_faces_key = mesh_coords_key, mesh_faces_key
        self.use_winding_number, self.closest_points_key = use_winding_number, closest_points_key

    def __call__(self, data: TensorDict) -> TensorDict:
        from ...nn.functional.geometry.sdf import signed_distance_field

        verts, faces = _need(data, self.mesh_coords_key), _need(data, self.mesh_faces_key)
        upd = {}
        for i, k in enumerate(self.input_keys):
            sdf, closest, _ = signed_distance_field(verts, faces, _need(data, k), use_sign_winding_number=self.use_winding_number)
            suffix = "" if len(self.input_keys) == 1 else f"_{k}"
            upd[self.output_key + suffix] = sdf.reshape(-1, 1)
            if self.closest_points_key:
                upd[self.closest_points_key + suffix] = closest
        return data.update(upd)


@register()
class ComputeNormals(Transform):
    """Unit vectors from each position's closest surface point to the position (centre-of-mass direction where the
    distance vanishes)."""

    def __init__(self, positions_key: str, closest_points_key: str, center_of_mass_key: str, output_key: str, *,
                 handle_zero_distance: bool = True) -> None:
        super().__init__()
        self.positions_key, self.closest_points_key = positions_key, closest_points_key
        self.center_of_mass_key, self.output_key, self.handle_zero_distance = center_of_mass_key, output_key, handle_zero_distance

    def __call__(self, data: TensorDict) -> TensorDict:
        pos, close = _need(data, self.positions_key), _need(data, self.closest_points_key)
        vec = pos - close
        norm = vec.norm(dim=-1, keepdim=True)
        if self.handle_zero_distance:
            fallback = pos - _need(data, self.center_of_mass_key)
            zero = norm < 1e-6
            vec = torch.where(zero, fallback, vec)
            norm = torch.where(zero, fallback.norm(dim=-1, keepdim=True), norm)
        return data.update({self.output_key: vec / norm.clamp_min(1e-12)})
