"""Pre-processing pipeline that turns raw CFD samples into the input dictionary of the DoMINO model.

Parity: ``physicsnemo/datapipes/cae/domino_datapipe.py`` (``DoMINODataConfig``, ``DoMINODataPipe``,
``compute_scaling_factors``).  One sample is a dict with the geometry (``stl_coordinates``, ``stl_faces``, ``stl_centers``,
``stl_areas``), global parameters, the surface mesh (``surface_mesh_centers``, ``surface_normals``, ``surface_areas``,
``surface_fields``) and / or the volume mesh (``volume_mesh_centers``, ``volume_fields``).  The pipeline

* evaluates the signed distance of the geometry on the regular surface and volume grids and at the volume points
  (BVH closest-point kernel, winding-number sign),
* optionally samples points (area-weighted on the surface), finds ``num_surface_neighbors`` nearest surface neighbours
  (kNN kernel), and restricts to the bounding boxes,
* builds the position encodings relative to the centre of mass and to the closest surface point,
* normalises coordinates to ``[-1, 1]`` inside the bounding boxes and scales the target fields.

Everything runs on the device of the incoming tensors (pre-processing on the GPU is the default), so a training step
receives tensors that are already resident; ``__call__`` adds the batch dimension the model expects.
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Iterable, Literal, Optional, Sequence

import torch

from ...nn.functional import knn, signed_distance_field


def normalize(x: torch.Tensor, max_val: torch.Tensor, min_val: torch.Tensor) -> torch.Tensor:
    """Map ``[min, max]`` to ``[-1, 1]``."""
    return 2.0 * (x - min_val) / (max_val - min_val) - 1.0


def unnormalize(x, max_val, min_val):
    return (x + 1.0) * (max_val - min_val) * 0.5 + min_val


def standardize(x, mean, std):
    return (x - mean) / std


def unstandardize(x, mean, std):
    return x * std + mean


def create_grid(max_coords, min_coords, resolution: Sequence[int], device=None) -> torch.Tensor:
    """Regular grid ``[nx, ny, nz, 3]`` spanning the box, end points included."""
    axes = [torch.linspace(float(min_coords[i]), float(max_coords[i]), int(resolution[i]), device=device) for i in range(3)]
    return torch.stack(torch.meshgrid(*axes, indexing="ij"), dim=-1)


def calculate_center_of_mass(centers: torch.Tensor, sizes: torch.Tensor) -> torch.Tensor:
    w = sizes.reshape(-1, 1)
    return ((centers * w).sum(0) / w.sum()).reshape(1, 3)


def shuffle_array(x: torch.Tensor, n: int, weights: torch.Tensor | None = None, generator=None):
    """``n`` rows of ``x`` without replacement (all rows, shuffled, when there are fewer), uniformly or by weight."""
    total = x.shape[0]
    n = min(n, total)
    if weights is None:
        idx = torch.randperm(total, device=x.device, generator=generator)[:n]
    else:
        idx = torch.multinomial(weights.double().clamp_min(0), n, replacement=False, generator=generator)
    return x[idx], idx


@dataclass
class DoMINODataConfig:
    data_path: Path | None = None
    phase: Literal["train", "val", "test"] = "train"
    surface_variables: Optional[Sequence] = ("pMean", "wallShearStress")
    surface_points_sample: int = 1024
    num_surface_neighbors: int = 11
    surface_sampling_algorithm: str = "area_weighted"
    surface_factors: Optional[Sequence] = None
    bounding_box_dims_surf: Optional[Sequence] = None      # (max xyz, min xyz)
    volume_variables: Optional[Sequence] = ("UMean", "pMean")
    volume_points_sample: int = 1024
    volume_sample_from_disk: bool = False
    volume_factors: Optional[Sequence] = None
    bounding_box_dims: Optional[Sequence] = None            # (max xyz, min xyz)
    grid_resolution: Sequence = (256, 96, 64)
    normalize_coordinates: bool = False
    sample_in_bbox: bool = False
    sampling: bool = False
    geom_points_sample: int = 300000
    scaling_type: Optional[Literal["min_max_scaling", "mean_std_scaling"]] = None
    compute_scaling_factors: bool = False
    caching: bool = False
    deterministic: bool = False
    gpu_preprocessing: bool = True
    gpu_output: bool = True
    shard_grid: bool = False
    shard_points: bool = False

    def __post_init__(self):
        if self.data_path is not None:
            self.data_path = Path(self.data_path).expanduser()
            if not self.data_path.exists():
                raise ValueError(f"Path {self.data_path} does not exist")
            if not self.data_path.is_dir():
                raise ValueError(f"Path {self.data_path} is not a directory")
        if self.caching and self.sampling:
            raise ValueError("Sampling should be False for caching")
        if self.caching and self.compute_scaling_factors:
            raise ValueError("Compute scaling factors should be False for caching")
        if self.phase not in ("train", "val", "test"):
            raise ValueError(f"phase should be one of ['train', 'val', 'test'], got {self.phase}")
        if self.scaling_type not in (None, "min_max_scaling", "mean_std_scaling"):
            raise ValueError(f"scaling_type should be one of ['min_max_scaling', 'mean_std_scaling'], got {self.scaling_type}")
        if self.surface_sampling_algorithm not in ("area_weighted", "random"):
            raise ValueError("surface_sampling_algorithm should be 'area_weighted' or 'random'")


class DoMINODataPipe(torch.utils.data.Dataset):
    """``DoMINODataPipe(dataset, model_type="combined", **config)``; indexable (reads ``dataset[i]``) and callable on a dict."""

    def __init__(self, input_path=None, model_type: Literal["surface", "volume", "combined"] = "combined", dataset: Iterable | None = None,
                 device=None, **config_overrides):
        if model_type not in ("surface", "volume", "combined"):
            raise ValueError("model_type must be 'surface', 'volume' or 'combined'")
        self.config = DoMINODataConfig(data_path=input_path, **config_overrides)
        self.model_type, self.dataset = model_type, dataset
        self.device = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() and self.config.gpu_preprocessing else "cpu")
        c = self.config
        if c.bounding_box_dims_surf is None:
            raise ValueError("Bounding box dimensions are not set in config")
        if model_type != "surface" and c.bounding_box_dims is None:
            raise ValueError("Bounding box dimensions are not set in config")
        t = lambda v: torch.as_tensor(v, dtype=torch.float32, device=self.device)  # noqa: E731
        self.s_max, self.s_min = t(c.bounding_box_dims_surf[0]), t(c.bounding_box_dims_surf[1])
        self.default_surface_grid = create_grid(self.s_max, self.s_min, c.grid_resolution, self.device)
        if c.bounding_box_dims is not None:
            self.c_max, self.c_min = t(c.bounding_box_dims[0]), t(c.bounding_box_dims[1])
            self.default_volume_grid = create_grid(self.c_max, self.c_min, c.grid_resolution, self.device)
        else:
            self.c_max = self.c_min = self.default_volume_grid = None
        for name in ("surface_factors", "volume_factors"):
            if getattr(c, name) is not None:
                setattr(c, name, t(getattr(c, name)))
        self._gen = torch.Generator(device=self.device)
        if c.deterministic:
            self._gen.manual_seed(0)

    # ---- scaling of the targets
    def scale_model_targets(self, fields, factors):
        if self.config.scaling_type == "mean_std_scaling":
            return standardize(fields, factors[0], factors[1])
        if self.config.scaling_type == "min_max_scaling":
            return normalize(fields, factors[0], factors[1])
        return fields

    def unscale_model_outputs(self, volume_fields=None, surface_fields=None):
        def undo(f, factors):
            if f is None or self.config.scaling_type is None:
                return f
            if self.config.scaling_type == "mean_std_scaling":
                return unstandardize(f, factors[0], factors[1])
            return unnormalize(f, factors[0], factors[1])

        return undo(volume_fields, self.config.volume_factors), undo(surface_fields, self.config.surface_factors)

    # ---- the two branches
    def process_surface(self, center_of_mass, d):
        c = self.config
        xyz, normals, sizes = d["surface_mesh_centers"], d["surface_normals"], d["surface_areas"]
        fields = d.get("surface_fields")
        keep = sizes > 0
        if c.sample_in_bbox and self.c_min is not None:
            keep = keep & ((xyz > self.c_min) & (xyz < self.c_max)).all(dim=-1)
        xyz, normals, sizes = xyz[keep], normals[keep], sizes[keep]
        fields = fields[keep] if fields is not None else None
        full_xyz, full_normals, full_sizes = xyz, normals, sizes
        if c.sampling:
            w = sizes if c.surface_sampling_algorithm == "area_weighted" else None
            xyz, idx = shuffle_array(xyz, c.surface_points_sample, weights=w, generator=self._gen)
            if xyz.shape[0] < c.surface_points_sample:
                raise ValueError("Surface mesh has fewer points than requested sample size")
            normals, sizes = normals[idx], sizes[idx]
            fields = fields[idx] if fields is not None else None
        if c.num_surface_neighbors > 1:
            nbr = knn(full_xyz, xyz, c.num_surface_neighbors)[0].long()
            neighbors, nbr_normals, nbr_sizes = full_xyz[nbr][:, 1:], full_normals[nbr][:, 1:], full_sizes[nbr][:, 1:]
        else:
            neighbors, nbr_normals, nbr_sizes = xyz, normals, sizes
        com = center_of_mass
        if c.normalize_coordinates:
            xyz, neighbors, com = (normalize(v, self.s_max, self.s_min) for v in (xyz, neighbors, com))
        if c.scaling_type is not None and fields is not None:
            fields = self.scale_model_targets(fields, c.surface_factors)
        out = {"pos_surface_center_of_mass": xyz - com, "surface_mesh_centers": xyz, "surface_mesh_neighbors": neighbors,
               "surface_normals": normals, "surface_neighbors_normals": nbr_normals, "surface_areas": sizes,
               "surface_neighbors_areas": nbr_sizes}
        if fields is not None:
            out["surface_fields"] = fields
        return out

    def process_volume(self, center_of_mass, d, stl_vertices, stl_faces):
        c = self.config
        xyz, fields = d["volume_mesh_centers"], d.get("volume_fields")
        if c.sample_in_bbox:
            keep = ((xyz > self.c_min) & (xyz < self.c_max)).all(dim=1)
            xyz = xyz[keep]
            fields = fields[keep] if fields is not None else None
        if c.sampling:
            xyz, idx = shuffle_array(xyz, c.volume_points_sample, generator=self._gen)
            if xyz.shape[0] < c.volume_points_sample:
                raise ValueError("Volume mesh has fewer points than requested sample size")
            fields = fields[idx] if fields is not None else None
        grid, verts, com = self.default_volume_grid, stl_vertices, center_of_mass
        if c.normalize_coordinates:
            xyz, grid, verts, com = (normalize(v, self.c_max, self.c_min) for v in (xyz, grid, verts, com))
        if c.scaling_type is not None and fields is not None:
            fields = self.scale_model_targets(fields, c.volume_factors)
        sdf_grid, _, _ = signed_distance_field(verts, stl_faces, grid, use_sign_winding_number=True)
        sdf_nodes, closest, _ = signed_distance_field(verts, stl_faces, xyz, use_sign_winding_number=True)
        out = {"volume_mesh_centers": xyz, "sdf_nodes": sdf_nodes.reshape(-1, 1), "grid": grid, "sdf_grid": sdf_grid,
               "pos_volume_closest": xyz - closest, "pos_volume_center_of_mass": xyz - com}
        if fields is not None:
            out["volume_fields"] = fields
        return out

    @torch.no_grad()
    def process_data(self, data_dict: dict) -> dict:
        required = ["global_params_values", "global_params_reference", "stl_coordinates", "stl_faces", "stl_centers", "stl_areas"]
        missing = [k for k in required if k not in data_dict]
        if missing:
            raise ValueError(f"Missing required keys in data_dict: {missing}. Required keys are: {required}")
        d = {k: (v.to(self.device) if isinstance(v, torch.Tensor) else torch.as_tensor(v, device=self.device)) for k, v in data_dict.items()}
        d = {k: (v.float() if v.is_floating_point() else v) for k, v in d.items()}
        c = self.config
        out = {"global_params_values": d["global_params_values"], "global_params_reference": d["global_params_reference"]}
        verts, faces = d["stl_coordinates"], d["stl_faces"].reshape(-1, 3).long()
        surf_grid = self.default_surface_grid
        normed = verts
        if c.normalize_coordinates:
            normed, surf_grid = normalize(verts, self.s_max, self.s_min), normalize(surf_grid, self.s_max, self.s_min)
            out["surface_min_max"] = torch.stack([self.s_min, self.s_max])
        out["sdf_surf_grid"], _, _ = signed_distance_field(normed, faces, surf_grid, use_sign_winding_number=True)
        out["surf_grid"] = surf_grid
        com = calculate_center_of_mass(d["stl_centers"], d["stl_areas"])
        if c.sampling:
            geo, _ = shuffle_array(verts, c.geom_points_sample, generator=self._gen)
        else:
            geo = verts
        out["geometry_coordinates"] = geo
        if self.model_type in ("surface", "combined"):
            out.update(self.process_surface(com, d))
        if self.model_type in ("volume", "combined"):
            if c.normalize_coordinates:
                out["volume_min_max"] = torch.stack([self.c_min, self.c_max])
            out.update(self.process_volume(com, d, verts, faces))
        return out

    # ---- dataset protocol
    def set_dataset(self, dataset: Iterable) -> None:
        self.dataset = dataset

    def __len__(self):
        return len(self.dataset) if self.dataset is not None else 0

    def __call__(self, data_dict: dict) -> dict:
        out = self.process_data(data_dict)
        out = {k: v.unsqueeze(0) for k, v in out.items()}
        return out if self.config.gpu_output else {k: v.cpu() for k, v in out.items()}

    def __getitem__(self, idx):
        if self.dataset is None:
            raise ValueError("Dataset is not present")
        return self(self.dataset[idx])

    def __iter__(self):
        if self.dataset is None:
            raise ValueError("Dataset is not present, can not be consumed as an iterator.")
        for sample in self.dataset:
            yield self(sample)


def compute_scaling_factors(samples: Iterable[dict], keys: Sequence[str] = ("volume_fields", "surface_fields")) -> dict:
    """Per-channel mean / std / min / max of the given field keys over an iterable of samples (streaming, fp64)."""
    stats = {}
    for sample in samples:
        for k in keys:
            if k not in sample:
                continue
            f = torch.as_tensor(sample[k]).double().reshape(-1, sample[k].shape[-1])
            s = stats.setdefault(k, {"n": 0, "sum": 0.0, "sq": 0.0, "min": f.min(0).values, "max": f.max(0).values})
            s["n"] += f.shape[0]
            s["sum"] = s["sum"] + f.sum(0)
            s["sq"] = s["sq"] + (f * f).sum(0)
            s["min"], s["max"] = torch.minimum(s["min"], f.min(0).values), torch.maximum(s["max"], f.max(0).values)
    out = {}
    for k, s in stats.items():
        mean = s["sum"] / s["n"]
        out[k] = {"mean": mean.float(), "std": (s["sq"] / s["n"] - mean * mean).clamp_min(0).sqrt().float(), "min": s["min"].float(),
                  "max": s["max"].float()}
    return out
