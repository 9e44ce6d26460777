"""Pre-processing pipeline that turns raw CFD samples into Transolver / GeoTransolver inputs.

Parity: ``physicsnemo/datapipes/cae/transolver_datapipe.py`` (``TransolverDataConfig``, ``TransolverDataPipe``): from a
sample with surface (``surface_mesh_centers``, ``surface_normals``, ``surface_fields`` …) and / or volume data
(``volume_mesh_centers``, ``volume_fields``, the STL for signed distances) it draws ``resolution`` points, builds the
position(+normal / SDF) ``embeddings``, the broadcast global features ``fx`` (air density, stream velocity), the scaled target
``fields``, optionally a sub-sampled ``geometry`` point cloud, and applies translation / scale invariance.  Sampling uses the
``weighted_multinomial`` functional (without replacement: exact for surfaces, Poisson-gap stream for the very large volume
sets); signed distances come from the BVH kernel.  Everything stays on the device of the incoming tensors; ``__call__`` adds
the batch dimension.
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Iterable, Literal, Optional

import torch

from ...nn.functional import signed_distance_field, weighted_multinomial
from .domino_datapipe import normalize, standardize, unnormalize, unstandardize


@dataclass
class TransolverDataConfig:
    data_path: Path | None = None
    model_type: Literal["surface", "volume", "combined"] = "surface"
    resolution: int | None = 200_000
    include_normals: bool = True
    include_sdf: bool = True
    include_geometry: bool = False
    geometry_sampling: int | None = 300_000
    scaling_type: Optional[Literal["min_max_scaling", "mean_std_scaling"]] = None
    surface_factors: Optional[dict] = None
    volume_factors: Optional[dict] = None
    translational_invariance: bool = False
    reference_origin: torch.Tensor | None = None
    scale_invariance: bool = False
    reference_scale: list | torch.Tensor | None = None
    broadcast_global_features: bool = True
    volume_sample_from_disk: bool = True
    return_mesh_features: bool = False

    def __post_init__(self):
        if self.data_path is not None:
            self.data_path = Path(self.data_path).expanduser()
            if not self.data_path.exists():
                raise ValueError(f"Path {self.data_path} does not exist")
            if not self.data_path.is_dir():
                raise ValueError(f"Path {self.data_path} is not a directory")
        if self.model_type not in ("surface", "volume", "combined"):
            raise ValueError(f"model_type must be 'surface', 'volume' or 'combined', got {self.model_type}")
        if self.scaling_type not in (None, "min_max_scaling", "mean_std_scaling"):
            raise ValueError(f"scaling_type should be one of ['min_max_scaling', 'mean_std_scaling'], got {self.scaling_type}")
        if self.scale_invariance:
            if self.reference_scale is None:
                raise ValueError("reference_scale must be set if scale invariance is enabled")
            ref = torch.as_tensor(self.reference_scale, dtype=torch.float32).reshape(-1)
            if ref.numel() != 3:
                raise ValueError("reference_scale must be a list of 3 floats")
            self.reference_scale = ref.reshape(1, 3)


def _draw(n: int, k: int | None, strategy: str, device) -> torch.Tensor | None:
    if k is None or k >= n:
        return None
    return weighted_multinomial(n, k, strategy=strategy, device=device)


class TransolverDataPipe(torch.utils.data.Dataset):
    def __init__(self, input_path=None, model_type: Literal["surface", "volume", "combined"] = "surface", pin_memory: bool = False,
                 dataset: Iterable | None = None, **data_config_overrides):
        self.config = TransolverDataConfig(data_path=input_path, model_type=model_type, **data_config_overrides)
        self.dataset, self.pin_memory = dataset, pin_memory

    # ---- scaling
    def _factors(self, which: str) -> dict:
        f = self.config.surface_factors if which == "surface" else self.config.volume_factors
        if f is None:
            raise ValueError(f"{which}_factors are needed when scaling_type is set")
        return f

    def scale_model_targets(self, fields: torch.Tensor, factors: dict) -> torch.Tensor:
        f = {k: torch.as_tensor(v).to(fields) for k, v in factors.items()}
        if self.config.scaling_type == "mean_std_scaling":
            return standardize(fields, f["mean"], f["std"])
        if self.config.scaling_type == "min_max_scaling":
            return normalize(fields, f["max"], f["min"])
        return fields

    def unscale_model_targets(self, fields: torch.Tensor, air_density=None, stream_velocity=None,
                              factor_type: Literal["surface", "volume", "auto"] = "auto") -> torch.Tensor:
        if factor_type == "auto":
            if self.config.model_type == "combined":
                raise ValueError("factor_type must be 'surface' or 'volume' for a combined pipeline")
            factor_type = self.config.model_type
        f = {k: torch.as_tensor(v).to(fields) for k, v in self._factors(factor_type).items()}
        if self.config.scaling_type == "mean_std_scaling":
            return unstandardize(fields, f["mean"], f["std"])
        if self.config.scaling_type == "min_max_scaling":
            return unnormalize(fields, f["max"], f["min"])
        return fields

    def _global_features(self, d: dict, n: int):
        if "air_density" not in d or "stream_velocity" not in d:
            return None
        fx = torch.stack([torch.as_tensor(d["air_density"]).reshape(()), torch.as_tensor(d["stream_velocity"]).reshape(())], dim=-1).float()
        fx = fx.to(d["stl_centers"].device)
        return fx.broadcast_to(n, -1) if self.config.broadcast_global_features else fx.unsqueeze(0)

    def _invariant(self, xyz, com, scale):
        if self.config.translational_invariance:
            xyz = xyz - com
        if self.config.scale_invariance:
            xyz = xyz / scale.to(xyz)
        return xyz

    # ---- branches
    def preprocess_surface_data(self, d: dict, com=None, scale=None) -> dict:
        c = self.config
        pos = d["surface_mesh_centers"]
        idx = _draw(pos.shape[0], c.resolution, "exact", pos.device)
        take = (lambda t: t[idx]) if idx is not None else (lambda t: t)
        parts = [self._invariant(take(pos), com, scale)]
        if c.include_normals:
            nrm = take(d["surface_normals"])
            parts.append(nrm / nrm.norm(dim=-1, keepdim=True))
        emb = torch.cat(parts, dim=-1)
        fields = take(d["surface_fields"])
        if c.scaling_type is not None:
            fields = self.scale_model_targets(fields, self._factors("surface"))
        out = {"embeddings": emb, "fields": fields}
        fx = self._global_features(d, emb.shape[0])
        if fx is not None:
            out["fx"] = fx
        if "surface_areas" in d and "surface_normals" in d:
            out["surface_areas_sub"], out["surface_normals_sub"] = take(d["surface_areas"]), take(d["surface_normals"])
        return out

    def preprocess_volume_data(self, d: dict, com=None, scale=None) -> dict:
        c = self.config
        pos = d["volume_mesh_centers"]
        idx = _draw(pos.shape[0], c.resolution, "poisson_gap", pos.device)
        take = (lambda t: t[idx]) if idx is not None else (lambda t: t)
        centre = com if com is not None else d["stl_centers"].mean(0, keepdim=True)
        pos = self._invariant(take(pos), centre, scale)
        parts = [pos]
        if c.include_sdf:
            verts = self._invariant(d["stl_coordinates"], centre, scale)
            sdf, closest, _ = signed_distance_field(verts, d["stl_faces"].reshape(-1, 3), pos, use_sign_winding_number=True)
            parts.append(sdf.reshape(-1, 1))
        else:
            closest = centre / scale.to(centre) if c.scale_invariance else centre
        if c.include_normals:
            nrm = pos - closest
            null = nrm.norm(dim=-1) < 1e-6
            nrm = torch.where(null.unsqueeze(-1), pos - centre, nrm)
            parts.append(nrm / (nrm.norm(dim=-1, keepdim=True) + 1e-6))
        emb = torch.cat(parts, dim=-1)
        fields = take(d["volume_fields"])
        if c.scaling_type is not None:
            fields = self.scale_model_targets(fields, self._factors("volume"))
        out = {"embeddings": emb, "fields": fields}
        fx = self._global_features(d, emb.shape[0])
        if fx is not None:
            out["fx"] = fx
        return out

    def process_geometry(self, d: dict, com=None, scale=None) -> torch.Tensor:
        g = d["stl_coordinates"]
        idx = _draw(g.shape[0], self.config.geometry_sampling, "poisson_gap", g.device)
        return self._invariant(g if idx is None else g[idx], com, scale)

    @torch.no_grad()
    def process_data(self, data_dict: dict) -> dict:
        c = self.config
        need = ["stl_centers"]
        if c.model_type in ("volume", "combined"):
            need += ["stl_coordinates", "stl_faces", "volume_fields", "volume_mesh_centers"]
        if c.model_type in ("surface", "combined"):
            need += ["surface_fields", "surface_mesh_centers"] + (["surface_normals"] if c.include_normals else [])
        missing = [k for k in need if k not in data_dict]
        if missing:
            raise ValueError(f"Missing required keys in data_dict: {missing}. Required keys are: {need}")
        d = data_dict
        com = None
        if c.translational_invariance:
            com = (c.reference_origin if c.reference_origin is not None else d["stl_centers"].mean(0)).reshape(1, -1).to(d["stl_centers"])
        scale = c.reference_scale if c.scale_invariance else None
        if c.model_type == "surface":
            out = self.preprocess_surface_data(d, com, scale)
        elif c.model_type == "volume":
            out = self.preprocess_volume_data(d, com, scale)
        else:
            s, v = self.preprocess_surface_data(d, com, scale), self.preprocess_volume_data(d, com, scale)
            out = {"embeddings": [s["embeddings"], v["embeddings"]], "fields": [s["fields"], v["fields"]]}
            if "fx" in s:
                out["fx"] = s["fx"]
        if c.include_geometry:
            out["geometry"] = self.process_geometry(d, com, scale)
        if c.return_mesh_features:
            for k in ("surface_areas", "surface_normals"):
                if k in d:
                    out[k] = d[k]
            if c.model_type in ("surface", "combined"):
                out["fields_full"] = (self.scale_model_targets(d["surface_fields"], self._factors("surface")) if c.scaling_type is not None
                                      else d["surface_fields"])
        for k in ("air_density", "stream_velocity"):
            if k in d:
                out[k] = d[k]
        return out

    # ---- dataset protocol
    def set_dataset(self, dataset: Iterable) -> None:
        self.dataset = dataset

    def __len__(self):
        return len(self.dataset) if self.dataset is not None else 0

    def __call__(self, data_dict: dict) -> dict:
        out = self.process_data(data_dict)
        batch = lambda v: [t.unsqueeze(0) for t in v] if isinstance(v, list) else (v.unsqueeze(0) if isinstance(v, torch.Tensor) else v)  # noqa: E731
        return {k: batch(v) for k, v in out.items()}

    def __getitem__(self, idx):
        if self.dataset is None:
            raise ValueError("Dataset is not present")
        return self(self.dataset[idx])

    def __iter__(self):
        if self.dataset is None:
            raise ValueError("Dataset is not present, can not be consumed as an iterator.")
        for sample in self.dataset:
            yield self(sample)
