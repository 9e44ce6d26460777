"""Out-of-distribution guards on model embeddings.

Parity: ``physicsnemo/experimental/guardrails/embedded/ood_guard.py`` (``OODGuard``, ``OODGuardConfig``): during training
``collect`` records per-channel min / max of the global-parameter embedding and a ring buffer of (unit-normalised)
geometry latents; at inference ``check`` warns when a global value leaves the recorded bounds or when the mean cosine-space
distance to the ``k`` nearest stored latents exceeds ``sensitivity ×`` the 99th percentile of that statistic inside the
buffer.  Distances come from the kNN functional (CUDA kernel on GPU).  State lives in buffers, so it is saved with the model.
"""
from __future__ import annotations

import logging
from dataclasses import dataclass

import torch
import torch.nn as nn

from ...nn.functional import knn

logger = logging.getLogger(__name__)


@dataclass
class OODGuardConfig:
    buffer_size: int
    knn_k: int = 10
    sensitivity: float = 1.5


def _unit(x: torch.Tensor) -> torch.Tensor:
    return x / (x.norm(dim=-1, keepdim=True) + 1e-8)


class OODGuard(nn.Module):
    def __init__(self, buffer_size: int, global_dim: int | None = None, geometry_embed_dim: int | None = None, knn_k: int = 10,
                 sensitivity: float = 1.5) -> None:
        super().__init__()
        self.buffer_size, self.sensitivity, self.knn_k = buffer_size, sensitivity, knn_k
        self.register_buffer("global_min", torch.full((global_dim,), float("inf")) if global_dim is not None else None)
        self.register_buffer("global_max", torch.full((global_dim,), float("-inf")) if global_dim is not None else None)
        has_geo = geometry_embed_dim is not None
        self.register_buffer("geo_embeddings", torch.zeros(buffer_size, geometry_embed_dim) if has_geo else None)
        self.register_buffer("geo_ptr", torch.zeros(1, dtype=torch.long) if has_geo else None)
        self.register_buffer("geo_full", torch.zeros(1, dtype=torch.bool) if has_geo else None)
        self.register_buffer("knn_threshold", torch.tensor(float("inf")) if has_geo else None)
        self._threshold_stale = True
        self.last_flags: dict = {}

    def _n_valid(self) -> int:
        return self.buffer_size if bool(self.geo_full) else int(self.geo_ptr)

    def _validate(self, g, z) -> None:
        if g is not None and self.global_min is not None:
            if g.ndim < 2:
                raise ValueError(f"global_embedding must have at least 2 dims (batch + channel); got shape {tuple(g.shape)}")
            if g.shape[-1] != self.global_min.shape[0]:
                raise ValueError(f"global_embedding last-dim mismatch: expected {self.global_min.shape[0]}, got {g.shape[-1]}")
        if z is not None and self.geo_embeddings is not None:
            if z.ndim != 2:
                raise ValueError(f"geometry_latent must be rank-2 (B, D); got shape {tuple(z.shape)}. Pool higher-rank latents first.")
            if z.shape[1] != self.geo_embeddings.shape[1]:
                raise ValueError(f"geometry_latent channel dim mismatch: expected {self.geo_embeddings.shape[1]}, got {z.shape[1]}")

    @torch.no_grad()
    def collect(self, global_embedding: torch.Tensor | None = None, geometry_latent: torch.Tensor | None = None) -> None:
        self._validate(global_embedding, geometry_latent)
        if global_embedding is not None and self.global_min is not None:
            v = global_embedding.detach().to(self.global_min.dtype).reshape(-1, global_embedding.shape[-1])
            self.global_min.copy_(torch.minimum(self.global_min, v.amin(0)))
            self.global_max.copy_(torch.maximum(self.global_max, v.amax(0)))
        if geometry_latent is not None and self.geo_embeddings is not None:
            z = geometry_latent.detach().to(self.geo_embeddings.dtype)[-self.buffer_size:]
            start = int(self.geo_ptr)
            idx = (start + torch.arange(z.shape[0], device=z.device)) % self.buffer_size
            self.geo_embeddings[idx] = z
            if start + z.shape[0] >= self.buffer_size:
                self.geo_full.fill_(True)
            self.geo_ptr.fill_((start + z.shape[0]) % self.buffer_size)
            self._threshold_stale = True

    @torch.no_grad()
    def score_geometry(self, geometry_latent: torch.Tensor) -> torch.Tensor:
        """Mean distance of every latent to its ``k`` nearest stored latents (both unit-normalised)."""
        self._validate(None, geometry_latent)
        if self.geo_embeddings is None:
            raise ValueError("OODGuard.score_geometry requires geometry_embed_dim to be set at construction time.")
        n = self._n_valid()
        if n == 0:
            raise RuntimeError("OODGuard.score_geometry called with an empty calibration buffer; call collect(geometry_latent=...) first.")
        store = _unit(self.geo_embeddings[:n])
        _, d = knn(store, _unit(geometry_latent.detach().to(store.dtype)), min(self.knn_k, n))
        return d.mean(dim=-1)

    @torch.no_grad()
    def compute_threshold(self) -> None:
        if self.geo_embeddings is None:
            return
        n = self._n_valid()
        k = min(self.knn_k, n - 1)
        if k <= 0:
            return
        store = _unit(self.geo_embeddings[:n])
        _, d = knn(store, store, k + 1)
        base = torch.quantile(d[:, 1:].mean(dim=-1), 0.99)                   # leave-one-out statistic inside the buffer
        self.knn_threshold.copy_(base * self.sensitivity)

    @torch.no_grad()
    def check(self, global_embedding: torch.Tensor | None = None, geometry_latent: torch.Tensor | None = None) -> dict:
        """Log a warning per violation and return ``{"global": bool mask | None, "geometry": bool mask | None}``."""
        self._validate(global_embedding, geometry_latent)
        flags = {"global": None, "geometry": None}
        if global_embedding is not None and self.global_min is not None:
            v = global_embedding.detach().to(self.global_min.dtype).reshape(-1, global_embedding.shape[-1])
            out = (v < self.global_min) | (v > self.global_max)
            flags["global"] = out.any(dim=-1)
            for ch in out.any(dim=0).nonzero().flatten().tolist():
                logger.warning("OOD Guard: global parameter channel %d outside the training range [%.4g, %.4g]", ch,
                               float(self.global_min[ch]), float(self.global_max[ch]))
        if geometry_latent is not None and self.geo_embeddings is not None and self._n_valid() > 0:
            if self._threshold_stale:
                self.compute_threshold()
                self._threshold_stale = False
            score = self.score_geometry(geometry_latent)
            flags["geometry"] = score > self.knn_threshold
            for i in flags["geometry"].nonzero().flatten().tolist():
                logger.warning("OOD Guard: geometry sample %d has kNN distance %.4g above the threshold %.4g", i, float(score[i]),
                               float(self.knn_threshold))
        self.last_flags = flags
        return flags
