"""Data-driven token centres ("prototype anchors") for the ``data_prototype_cluster`` tokenizer strategy.

Parity: ``physicsnemo/experimental/models/aerojepa/layers/prototype_anchors.py``
(``build_context_prototype_anchors`` ``:359``, ``build_target_prototype_anchors`` ``:415``,
``ensure_*`` ``:459`` / ``:511``, ``load_*`` ``:203`` / ``:231``).  Token positions produced by a
source tokenizer over the training cases are pooled, subsampled and clustered with k-means seeded by
farthest-point sampling; the sorted centres are stored as ``coords`` in an ``.npz`` with a JSON
record of the settings.
"""
from __future__ import annotations

import json
import logging
from pathlib import Path
from typing import Any, Callable, Mapping

import numpy as np
import torch

from ....nn.functional.neighbors import knn
from ...nn.point_tokenizer import PointCloudTokenizer
from .encoders import build_geometry_features

logger = logging.getLogger(__name__)


def seeded_farthest_points(points: torch.Tensor, count: int, seed: int) -> torch.Tensor:
    """Indices of ``count`` mutually distant points; the first one is drawn with ``seed``."""
    n = points.shape[0]
    if count >= n:
        return torch.arange(n, device=points.device)
    if count <= 0:
        raise ValueError("num_samples must be > 0")
    gen = torch.Generator(device=points.device).manual_seed(int(seed))
    picked = torch.empty(count, dtype=torch.long, device=points.device)
    nearest = points.new_full((n,), float("inf"))
    current = torch.randint(0, n, (1,), generator=gen, device=points.device)[0]
    for i in range(count):
        picked[i] = current
        nearest = torch.minimum(nearest, (points - points[current]).square().sum(-1))
        current = nearest.argmax()
    return picked


def kmeans_centres(points: torch.Tensor, *, num_clusters: int, num_iters: int, seed: int) -> torch.Tensor:
    """Lloyd iterations from farthest-point seeds; a centre that loses all its points is re-seeded from the data."""
    if points.shape[0] <= num_clusters:
        return points.clone()
    centres = points[seeded_farthest_points(points, num_clusters, seed)].clone()
    for _ in range(max(1, int(num_iters))):
        owner = knn(points=centres, queries=points, k=1)[0][:, 0].long()
        total = torch.zeros_like(centres).index_add_(0, owner, points)
        count = points.new_zeros(num_clusters).index_add_(0, owner, points.new_ones(points.shape[0]))
        alive = count > 0
        centres = torch.where(alive[:, None], total / count.clamp_min(1.0)[:, None], centres)
        if not bool(alive.all()):
            centres[~alive] = points[seeded_farthest_points(points, int((~alive).sum()), seed + 17)]
    return centres


def load_prototype_anchors(path) -> torch.Tensor:
    coords = np.asarray(np.load(str(path), allow_pickle=False)["coords"], dtype=np.float32)
    if coords.ndim != 2 or coords.shape[1] != 3:
        raise ValueError(f"Prototype anchor file {path} must contain coords with shape [P, 3].")
    return torch.from_numpy(coords)


load_target_prototype_anchors = load_context_prototype_anchors = load_prototype_anchors


def _target_points(sample: Mapping[str, Any]):
    surf_feat = sample.get("target_surface_main_feat", sample.get("surface_main_feat", sample.get("surface_feat")))
    surf_pos = sample.get("target_surface_pos", sample.get("surface_pos"))
    vol_pos = sample.get("target_volume_pos", sample.get("volume_pos"))
    vol_feat = sample.get("target_volume_feat", sample.get("volume_feat"))
    if surf_feat.shape[-1] != vol_feat.shape[-1]:
        raise ValueError("surface_main_feat and volume_feat must have matching feature dimensions.")
    return (torch.cat([surf_pos, vol_pos]).detach().cpu().float(), torch.cat([surf_feat, vol_feat]).detach().cpu().float())


def _context_points(sample: Mapping[str, Any], cfg: Mapping[str, Any]):
    feats = build_geometry_features(context_pos=sample["surface_pos"], context_feat=sample["surface_feat"],
                                    use_sdf=bool(cfg.get("use_sdf", False)), use_solid_normals=bool(cfg.get("use_solid_normals", False)),
                                    use_solid_n_dot_uinf=bool(cfg.get("use_solid_n_dot_uinf", False)))
    return sample["surface_pos"].detach().cpu().float(), feats.detach().cpu().float()


def build_prototype_anchors(*, train_dataset, cfg: Mapping[str, Any], output_path, seed: int, source_name: str,
                            point_loader: Callable) -> torch.Tensor:
    """Collect source-tokenizer positions over ``train_dataset``, cluster them, save and return the centres."""
    out = Path(output_path)
    out.parent.mkdir(parents=True, exist_ok=True)
    get = cfg.get
    settings = dict(
        prototype_anchor_count=int(get("prototype_anchor_count", 3072)), prototype_num_passes=int(get("prototype_num_passes", 1)),
        max_candidate_coords=int(get("prototype_max_candidate_coords", 65536)), kmeans_iters=int(get("prototype_kmeans_iters", 12)),
        source_strategy=str(get("prototype_source_strategy", "voxel_fps_cluster")).lower(),
        source_max_point_tokens=int(get("prototype_source_max_point_tokens", get("max_point_tokens", get("prototype_anchor_count", 3072)))),
        source_cluster_size=get("prototype_source_cluster_size", get("tokenizer_cluster_size")),
        source_voxel_size=get("prototype_source_voxel_size", get("tokenizer_voxel_size")),
        source_knn_chunk_size=int(get("prototype_source_knn_chunk_size", get("tokenizer_knn_chunk_size", 128))))
    tokenizer = PointCloudTokenizer(max_point_tokens=settings["source_max_point_tokens"], strategy=settings["source_strategy"],
                                    deterministic_eval=False, cluster_size=settings["source_cluster_size"],
                                    knn_chunk_size=settings["source_knn_chunk_size"], voxel_size=settings["source_voxel_size"]).train(True)
    pool = []
    for _ in range(settings["prototype_num_passes"]):
        for i in range(len(train_dataset)):
            pos, feat = point_loader(train_dataset[i])
            pool.append(tokenizer.tokenize_with_clusters(point_positions=pos, point_features=feat)[0].detach().cpu())
    if not pool:
        raise ValueError(f"No {source_name} token coordinates were collected for prototype anchors.")
    coords = torch.cat(pool).float()
    if coords.shape[0] > settings["max_candidate_coords"]:
        gen = torch.Generator().manual_seed(int(seed))
        coords = coords[torch.randperm(coords.shape[0], generator=gen)[:settings["max_candidate_coords"]]]
    centres = kmeans_centres(coords, num_clusters=settings["prototype_anchor_count"], num_iters=settings["kmeans_iters"],
                             seed=seed).cpu().numpy()
    centres = centres[np.lexsort((centres[:, 2], centres[:, 1], centres[:, 0]))].astype(np.float32, copy=False)
    record = dict(settings, prototype_anchor_count=int(centres.shape[0]), source_name=source_name, seed=int(seed),
                  n_cases=len(train_dataset))
    np.savez_compressed(out, coords=centres, metadata_json=np.asarray(json.dumps(record, default=str)))
    logger.info("saved %d %s prototype anchors to %s", centres.shape[0], source_name, out)
    return torch.from_numpy(centres)


def build_context_prototype_anchors(*, train_dataset, context_cfg, output_path, seed: int = 42) -> torch.Tensor:
    return build_prototype_anchors(train_dataset=train_dataset, cfg=context_cfg, output_path=output_path, seed=seed,
                                   source_name="context", point_loader=lambda s: _context_points(s, context_cfg))


def build_target_prototype_anchors(*, train_dataset, target_cfg, output_path, seed: int = 42) -> torch.Tensor:
    return build_prototype_anchors(train_dataset=train_dataset, cfg=target_cfg, output_path=output_path, seed=seed,
                                   source_name="target", point_loader=_target_points)


def _ensure(which: str, builder, train_dataset, cfg, seed):
    path = cfg.get("prototype_anchor_path")
    if not path:
        raise ValueError(f"{which}_encoder.prototype_anchor_path is required when tokenizer_strategy='data_prototype_cluster'.")
    if Path(path).exists() and not bool(cfg.get("prototype_rebuild", False)):
        return load_prototype_anchors(path)
    return builder(train_dataset, cfg, Path(path), seed)


def ensure_context_prototype_anchors(*, train_dataset, context_cfg, seed: int = 42) -> torch.Tensor:
    """Load the anchors named by ``prototype_anchor_path`` or build them when missing / ``prototype_rebuild``."""
    return _ensure("context", lambda d, c, p, s: build_context_prototype_anchors(train_dataset=d, context_cfg=c, output_path=p, seed=s),
                   train_dataset, context_cfg, seed)


def ensure_target_prototype_anchors(*, train_dataset, target_cfg, seed: int = 42) -> torch.Tensor:
    return _ensure("target", lambda d, c, p, s: build_target_prototype_anchors(train_dataset=d, target_cfg=c, output_path=p, seed=s),
                   train_dataset, target_cfg, seed)
