"""Embedding of multi-sensor point observations onto the model grid.

Counterpart of ``physicsnemo/experimental/models/healda/point_embed.py`` (``ObsTokenizer`` :158, ``UniformFusion`` :240,
``SensorEmbedder`` :304, ``MultiSensorObsEmbedder`` :533); parameter names are the same.  Observations arrive as flat
arrays grouped by sensor, then by ``(batch, time)`` window: ``offsets[s, b, t]`` is the end of window ``(b, t)`` of
sensor ``s`` in the flat arrays.  Every sensor tokenises its observations, averages them per
``(window, pixel, platform x channel)`` cell, mixes the cells of a pixel with an MLP, and the sensors are fused by a
normalised sum.
"""

from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch
from torch.utils.checkpoint import checkpoint

from .scatter_aggregator import ScatterAggregator

__all__ = ["ObsTokenizer", "UniformFusion", "SensorEmbedder", "MultiSensorObsEmbedder"]


def _offsets_to_batch_idx(offsets: torch.Tensor) -> torch.Tensor:
    """Window index of every observation from the cumulative window ends ``[B, T]``."""
    ends = offsets.flatten()
    counts = torch.diff(ends, prepend=ends.new_zeros(1))
    return torch.arange(ends.numel(), dtype=torch.long, device=offsets.device).repeat_interleave(counts)


def _check_obs(obs, float_metadata, named) -> int:
    if obs.ndim != 1:
        raise ValueError(f"Expected obs of shape (nobs,), got {obs.ndim}D tensor with shape {tuple(obs.shape)}")
    n = obs.shape[0]
    if float_metadata.ndim != 2:
        raise ValueError(f"Expected float_metadata of shape (nobs, meta_dim), got {float_metadata.ndim}D tensor with shape "
                         f"{tuple(float_metadata.shape)}")
    if float_metadata.shape[0] != n:
        raise ValueError(f"Expected float_metadata with {n} rows (matching obs), got tensor with shape {tuple(float_metadata.shape)}")
    for name, t in named:
        if t.ndim != 1 or t.shape[0] != n:
            raise ValueError(f"Expected {name} of shape ({n},) matching obs, got tensor with shape {tuple(t.shape)}")
    return n


@torch.compiler.disable
def _split_by_sensor(arrays: Tuple[torch.Tensor, ...], offsets: torch.Tensor) -> List[Tuple[torch.Tensor, ...]]:
    """Views of the flat arrays per sensor plus that sensor's window ends relative to its own start."""
    if offsets.ndim != 3:
        raise ValueError(f"offsets must have shape (S, B, T), got {offsets.shape}")
    total = arrays[0].shape[0]
    ends = offsets[:, -1, -1].tolist()                       # one host read for all sensors
    out, start = [], 0
    for s, end in enumerate(ends):
        if not (0 <= start <= end <= total):
            raise ValueError(f"Invalid offsets for sensor index {s}: start={start}, end={end}, total_obs={total}.")
        out.append(tuple(a.narrow(0, start, end - start) for a in arrays) + (offsets[s] - start,))
        start = end
    return out


class ObsTokenizer(torch.nn.Module):
    """``[obs, MLP(obs, metadata, type embedding)]``: the raw value stays the first feature of the token."""

    def __init__(self, meta_dim: int, out_dim: int, n_embed: int = 1024, embed_dim: int = 4):
        super().__init__()
        self.embed_table = torch.nn.Embedding(n_embed, embed_dim)
        hidden = out_dim * 2 if out_dim <= 32 else out_dim
        self.meta_mlp = torch.nn.Sequential(torch.nn.Linear(1 + meta_dim + embed_dim, hidden), torch.nn.LayerNorm(hidden), torch.nn.SiLU(),
                                            torch.nn.Linear(hidden, out_dim - 1))

    def forward(self, obs: torch.Tensor, float_metadata: torch.Tensor, obs_type: torch.Tensor) -> torch.Tensor:
        if not torch.compiler.is_compiling():
            _check_obs(obs, float_metadata, (("obs_type", obs_type),))
        value = obs.unsqueeze(-1)
        return torch.cat([value, self.meta_mlp(torch.cat([value, float_metadata, self.embed_table(obs_type)], dim=-1))], dim=-1)


class UniformFusion(torch.nn.Module):
    """Layer-normalised sum of the sensor embeddings divided by ``sqrt(num_sensors)``."""

    def __init__(self, fusion_dim: int):
        super().__init__()
        self.fusion_dim = fusion_dim
        self.norm = torch.nn.LayerNorm(fusion_dim)

    def forward(self, sensor_embeddings: torch.Tensor) -> torch.Tensor:
        if not torch.compiler.is_compiling():
            if sensor_embeddings.ndim != 5:
                raise ValueError(f"Expected sensor_embeddings of shape (num_sensors, batch, time, npix, fusion_dim), got "
                                 f"{sensor_embeddings.ndim}D tensor with shape {tuple(sensor_embeddings.shape)}")
            if sensor_embeddings.shape[-1] != self.fusion_dim:
                raise ValueError(f"Expected fusion_dim={self.fusion_dim} in last dimension, got {sensor_embeddings.shape[-1]} in tensor "
                                 f"with shape {tuple(sensor_embeddings.shape)}")
        return self.norm(sensor_embeddings).sum(dim=0) / math.sqrt(sensor_embeddings.shape[0])


class SensorEmbedder(torch.nn.Module):
    """Tokenise one sensor's observations and aggregate them to ``[B, T, npix, output_dim]``."""

    def __init__(self, *, nplatform: int, nchannel: int, sensor_embed_dim: int = 32, output_dim: int = 512, meta_dim: int = 28,
                 n_embed: int = 1024, embed_dim: int = 4, gradient_checkpointing: bool = False):
        super().__init__()
        self.sensor_embed_dim, self.output_dim, self.gradient_checkpointing = sensor_embed_dim, output_dim, gradient_checkpointing
        self.nchannel, self.nplatform = nchannel, nplatform
        self.obs_tokenizer = ObsTokenizer(meta_dim=meta_dim, out_dim=sensor_embed_dim, n_embed=n_embed, embed_dim=embed_dim)
        self.scatter_infill_aggregator = ScatterAggregator(in_dim=sensor_embed_dim, out_dim=output_dim, nbuckets=nchannel * nplatform)

    def aggregate(self, embedded_obs, pix, local_channel, local_platform, batch_idx, nbatch: int, npix: int) -> torch.Tensor:
        if not torch.compiler.is_compiling():
            if embedded_obs.ndim != 2:
                raise ValueError(f"Expected embedded_obs of shape (nobs, embed_dim), got {embedded_obs.ndim}D tensor with shape "
                                 f"{tuple(embedded_obs.shape)}")
            if embedded_obs.shape[1] != self.sensor_embed_dim:
                raise ValueError(f"Expected embed_dim={self.sensor_embed_dim} in embedded_obs, got {embedded_obs.shape[1]} in tensor with "
                                 f"shape {tuple(embedded_obs.shape)}")
            for name, t in (("pix", pix), ("local_channel", local_channel), ("local_platform", local_platform), ("batch_idx", batch_idx)):
                if t.ndim != 1 or t.shape[0] != embedded_obs.shape[0]:
                    raise ValueError(f"Expected {name} of shape ({embedded_obs.shape[0]},) matching embedded_obs, got tensor with shape "
                                     f"{tuple(t.shape)}")
        return self.scatter_infill_aggregator(x=embedded_obs, batch_idx=batch_idx, pix=pix, bucket_id=local_platform * self.nchannel + local_channel,
                                              nbatch=nbatch, npix=npix)

    def _forward(self, obs, float_metadata, pix, local_channel, local_platform, obs_type, offsets, npix: int) -> torch.Tensor:
        tokens = self.obs_tokenizer(obs, float_metadata, obs_type)
        out = self.aggregate(tokens, pix, local_channel, local_platform, _offsets_to_batch_idx(offsets), offsets.numel(), npix)
        return out.view(*offsets.shape, npix, self.output_dim)

    def forward(self, obs, float_metadata, pix, local_channel, local_platform, obs_type, offsets, npix: int) -> torch.Tensor:
        if not torch.compiler.is_compiling():
            _check_obs(obs, float_metadata, (("pix", pix), ("local_channel", local_channel), ("local_platform", local_platform),
                                             ("obs_type", obs_type)))
            if offsets.ndim != 2:
                raise ValueError(f"Expected offsets of shape (batch, time), got {offsets.ndim}D tensor with shape {tuple(offsets.shape)}")
        args = (obs, float_metadata, pix, local_channel, local_platform, obs_type, offsets, npix)
        return checkpoint(self._forward, *args, use_reentrant=False) if self.gradient_checkpointing else self._forward(*args)


class MultiSensorObsEmbedder(torch.nn.Module):
    """One ``SensorEmbedder`` per sensor, fused to ``[B, fusion_dim, T, npix]``."""

    def __init__(self, nchannel_per_sensor: List[int], nplatform_per_sensor: List[int], sensor_names: Optional[List[str]] = None,
                 embed_dim: int = 32, meta_dim: int = 28, fusion_dim: int = 512, gradient_checkpointing: bool = False,
                 torch_compile: bool = False):
        super().__init__()
        n = len(nchannel_per_sensor)
        if len(nplatform_per_sensor) != n:
            raise ValueError(f"nchannel_per_sensor and nplatform_per_sensor must have the same length, got {n} and {len(nplatform_per_sensor)}")
        if sensor_names is None:
            sensor_names = [f"sensor_{i}" for i in range(n)]
        elif len(set(sensor_names)) != n:
            raise ValueError(f"sensor_names must be unique and match length of nchannel_per_sensor, got {len(set(sensor_names))} unique names "
                             f"and {n} sensors")
        self.nchannel_per_sensor, self.nplatform_per_sensor = list(nchannel_per_sensor), list(nplatform_per_sensor)
        self.sensor_names, self.fusion_dim = list(sensor_names), fusion_dim
        self.embedders = torch.nn.ModuleDict({
            name: SensorEmbedder(sensor_embed_dim=embed_dim, meta_dim=meta_dim, output_dim=fusion_dim, nchannel=c, nplatform=p,
                                 gradient_checkpointing=gradient_checkpointing)
            for name, c, p in zip(sensor_names, nchannel_per_sensor, nplatform_per_sensor)})
        self.sensor_fusion = UniformFusion(fusion_dim=fusion_dim)
        self.output_norm = torch.nn.LayerNorm(fusion_dim)
        # torch_compile is accepted for interface compatibility; the layers here run eagerly

    def forward(self, obs, float_metadata, pix, local_channel, local_platform, obs_type, offsets, npix: int) -> torch.Tensor:
        if not torch.compiler.is_compiling():
            _check_obs(obs, float_metadata, (("pix", pix), ("local_channel", local_channel), ("local_platform", local_platform),
                                             ("obs_type", obs_type)))
            if offsets.ndim != 3:
                raise ValueError(f"Expected offsets of shape (sensors, batch, time), got {offsets.ndim}D tensor with shape {tuple(offsets.shape)}")
            if offsets.shape[0] != len(self.embedders):
                raise ValueError(f"Expected sensors={len(self.embedders)} in offsets (matching nchannel_per_sensor), got {offsets.shape[0]} in "
                                 f"tensor with shape {tuple(offsets.shape)}")
        per_sensor = _split_by_sensor((obs, float_metadata, pix, local_channel, local_platform, obs_type), offsets)
        stacked = torch.stack([emb(*part, npix=npix) for part, emb in zip(per_sensor, self.embedders.values())], dim=0)
        return self.output_norm(self.sensor_fusion(stacked)).permute(0, 3, 1, 2)
