"""Reduction of a raw point cloud to a bounded set of tokens.

Parity: ``physicsnemo/experimental/nn/point_tokenizer.py`` (``PointCloudTokenizer`` ``:101``).  A
strategy has two independent parts, which is how this file is organised: *where the token centres
come from* (all points, a random subset, farthest-point samples, farthest-point samples of voxel
means, fixed prototype coordinates) and *what a token carries* (the feature of its centre point, or
the mean feature of the ``cluster_size`` points nearest to the centre).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
from torch import nn

from ...nn.functional.geometry import farthest_point_sampling
from .point_utils import chunked_knn_indices

#: strategy → (centre source, pools a neighbourhood)
_STRATEGIES = {
    "identity": ("all", False),
    "random": ("random", False),
    "fps": ("fps", False),
    "random_cluster": ("random", True),
    "fps_cluster": ("fps", True),
    "voxel_fps_cluster": ("voxel_fps", True),
    "data_prototype_cluster": ("prototype", True),
}


def voxel_mean_positions(points: torch.Tensor, voxel_size) -> torch.Tensor:
    """Mean position of the points of every occupied voxel of an axis-aligned grid anchored at the cloud's minimum."""
    if points.ndim != 2:
        raise ValueError("voxel_mean_positions expects rank-2 point positions.")
    d = points.shape[1]
    edge = [float(voxel_size)] * d if isinstance(voxel_size, (int, float)) else [float(v) for v in voxel_size]
    if len(edge) != d:
        raise ValueError(f"voxel_size must have length {d}, got {len(edge)}")
    if min(edge) <= 0:
        raise ValueError("voxel_size values must be > 0.")
    edge_t = torch.tensor(edge, device=points.device, dtype=points.dtype)
    cell = torch.floor((points - points.amin(0)) / edge_t).long()
    _, member = torch.unique(cell, dim=0, return_inverse=True)
    n_voxels = int(member.max()) + 1
    total = points.new_zeros(n_voxels, d).index_add_(0, member, points)
    count = points.new_zeros(n_voxels).index_add_(0, member, points.new_ones(points.shape[0]))
    return total / count.clamp_min(1.0).unsqueeze(1)


class PointCloudTokenizer(nn.Module):
    """Turn ``(N, D)`` positions and ``(N, F)`` features into at most ``max_point_tokens`` tokens.

    Strategies: ``identity``, ``random``, ``fps``, ``random_cluster``, ``fps_cluster``,
    ``voxel_fps_cluster`` (needs ``voxel_size``) and ``data_prototype_cluster`` (needs
    ``prototype_coords``; the token count is the prototype count, each pooling ``prototype_knn_k``
    or ``cluster_size`` or 16 points).  The ``*_cluster`` strategies need ``cluster_size``.  In eval
    mode with ``deterministic_eval`` the random subset becomes an even stride and farthest-point
    sampling starts from the first point.  Clouds that already fit the budget pass through unchanged.
    """

    def __init__(self, *, max_point_tokens: Optional[int] = None, strategy: str = "identity", deterministic_eval: bool = True,
                 cluster_size: Optional[int] = None, knn_chunk_size: int = 128, voxel_size=None,
                 prototype_coords: Optional[torch.Tensor] = None, prototype_knn_k: Optional[int] = None):
        super().__init__()
        for label, value in (("max_point_tokens", max_point_tokens), ("cluster_size", cluster_size),
                             ("prototype_knn_k", prototype_knn_k)):
            if value is not None and int(value) <= 0:
                raise ValueError(f"{label} must be > 0 when provided.")
        if int(knn_chunk_size) <= 0:
            raise ValueError("knn_chunk_size must be > 0.")
        self.strategy = str(strategy).lower()
        if self.strategy not in _STRATEGIES:
            raise ValueError("PointCloudTokenizer.strategy must be one of: " + ", ".join(f"'{s}'" for s in _STRATEGIES))
        self._centres, self._pools = _STRATEGIES[self.strategy]
        self.max_point_tokens = None if max_point_tokens is None else int(max_point_tokens)
        self.cluster_size = None if cluster_size is None else int(cluster_size)
        self.prototype_knn_k = None if prototype_knn_k is None else int(prototype_knn_k)
        self.deterministic_eval, self.knn_chunk_size, self.voxel_size = bool(deterministic_eval), int(knn_chunk_size), voxel_size
        proto = torch.empty(0, 3) if prototype_coords is None else prototype_coords.detach().float().clone()
        if proto.ndim != 2 or proto.shape[-1] != 3:
            raise ValueError("prototype_coords must have shape [P, 3].")
        self.register_buffer("prototype_coords", proto, persistent=False)
        if self._centres == "prototype":
            if proto.shape[0] == 0:
                raise ValueError("prototype_coords must be provided for tokenizer_strategy='data_prototype_cluster'.")
        elif self._pools and self.cluster_size is None:
            raise ValueError(f"cluster_size must be provided for tokenizer_strategy='{self.strategy}'.")

    @property
    def uses_cluster_pooling(self) -> bool:
        return self._pools

    @property
    def requires_per_sample_loop(self) -> bool:
        """Whether a batched caller has to tokenise one sample at a time (fixed prototype centres)."""
        return self._centres == "prototype"

    # ---------------------------------------------------------------- centres
    def _random_start(self) -> bool:
        return bool(self.training or not self.deterministic_eval)

    def _subset(self, positions: torch.Tensor, budget: int) -> torch.Tensor:
        """Indices of ``budget`` points chosen by the strategy's sampler."""
        n, dev = positions.shape[0], positions.device
        if self._centres == "random":
            if self._random_start():
                return torch.randperm(n, device=dev)[:budget]
            return torch.linspace(0, n - 1, steps=budget, device=dev).long()
        if budget >= n:
            return torch.arange(n, device=dev)
        return farthest_point_sampling(positions, budget, random_start=self._random_start())

    def _centre_positions(self, positions: torch.Tensor, budget: int) -> torch.Tensor:
        if self._centres != "voxel_fps":
            return positions[self._subset(positions, budget)]
        if self.voxel_size is None:
            raise ValueError("voxel_size must be provided for tokenizer_strategy='voxel_fps_cluster'.")
        candidates = voxel_mean_positions(positions, self.voxel_size)
        if candidates.shape[0] <= budget:
            return candidates
        return candidates[farthest_point_sampling(candidates, budget, random_start=self._random_start())]

    # --------------------------------------------------------------- tokenise
    def tokenize_with_clusters(self, *, point_positions: torch.Tensor, point_features: torch.Tensor):
        """``(token_positions, token_features, cluster_idx)``; ``cluster_idx`` ``(T, k)`` lists the pooled points or is ``None``."""
        if point_positions.ndim != 2 or point_features.ndim != 2:
            raise ValueError("PointCloudTokenizer expects rank-2 point_positions and point_features.")
        n = point_positions.shape[0]
        if n != point_features.shape[0]:
            raise ValueError(f"point_positions and point_features must agree on point count, got {n} and {point_features.shape[0]}")
        if self._centres == "prototype":
            centres = self.prototype_coords.to(device=point_positions.device, dtype=point_positions.dtype)
            if n == 0:
                return (centres, point_features.new_zeros(centres.shape[0], point_features.shape[-1]),
                        torch.zeros(centres.shape[0], 0, dtype=torch.long, device=point_positions.device))
            k = self.prototype_knn_k or self.cluster_size or 16
        else:
            if self._centres == "all" or self.max_point_tokens is None or n <= self.max_point_tokens:
                return point_positions, point_features, None
            if not self._pools:
                keep = self._subset(point_positions, self.max_point_tokens)
                return point_positions[keep], point_features[keep], None
            centres = self._centre_positions(point_positions, self.max_point_tokens)
            k = self.cluster_size
        members = chunked_knn_indices(query_coords=centres, key_coords=point_positions, k=max(1, min(int(k), n)),
                                      chunk_size=self.knn_chunk_size)
        return centres, point_features[members].mean(dim=1), members

    def forward(self, *, point_positions: torch.Tensor, point_features: torch.Tensor):
        return self.tokenize_with_clusters(point_positions=point_positions, point_features=point_features)[:2]

    def forward_batched(self, *, point_positions: torch.Tensor, point_features: torch.Tensor,
                        point_counts: Optional[torch.Tensor] = None):
        """Padded batch in, padded tokens out: ``(positions (B, T, D), features (B, T, F), mask (B, T), counts (B,))``."""
        if point_positions.ndim != 3 or point_features.ndim != 3:
            raise ValueError("PointCloudTokenizer.forward_batched expects rank-3 point_positions and point_features.")
        if point_positions.shape[:2] != point_features.shape[:2]:
            raise ValueError("point_positions and point_features must agree on batch/point dims, "
                             f"got {tuple(point_positions.shape[:2])} and {tuple(point_features.shape[:2])}")
        B, n_max = point_positions.shape[:2]
        if point_counts is None:
            sizes = [n_max] * B
        elif point_counts.ndim != 1 or point_counts.shape[0] != B:
            raise ValueError("point_counts must have shape [B].")
        else:
            sizes = [int(c) for c in point_counts.tolist()]
        tokens = [self(point_positions=point_positions[b, :m], point_features=point_features[b, :m]) for b, m in enumerate(sizes)]
        counts = [t[0].shape[0] for t in tokens]
        T = max(counts, default=0)
        pos = point_positions.new_zeros(B, T, point_positions.shape[-1])
        feat = point_features.new_zeros(B, T, point_features.shape[-1])
        for b, (p, f) in enumerate(tokens):
            pos[b, :p.shape[0]], feat[b, :f.shape[0]] = p, f
        counts_t = torch.tensor(counts, device=point_positions.device, dtype=torch.long)
        mask = torch.arange(T, device=counts_t.device)[None, :] < counts_t[:, None]
        return pos, feat, mask, counts_t
