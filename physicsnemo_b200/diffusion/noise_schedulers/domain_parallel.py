"""Noise scheduler for domain-parallel (``ShardTensor``) training.

Parity: ``physicsnemo/diffusion/noise_schedulers/domain_parallel.py:40-374`` — wraps a
linear-Gaussian scheduler: training times are drawn on the first rank of the domain mesh and
broadcast so that all shards of a sample see the same noise level; latents are created as
``Shard(shard_dim)`` ShardTensors; ``add_noise`` draws noise per shard.
"""
from __future__ import annotations

from typing import Tuple

import torch
import torch.distributed as dist
from torch import Tensor

from ...parallel import Replicate, Shard, ShardTensor
from ...parallel.spec import chunk_sizes
from .schedulers import LinearGaussianNoiseScheduler


class DomainParallelNoiseScheduler:
    def __init__(self, scheduler: LinearGaussianNoiseScheduler, mesh, shard_dim: int = 2):
        if mesh.ndim != 1:
            raise ValueError("DomainParallelNoiseScheduler expects a 1-D domain mesh")
        self.scheduler, self.mesh, self.shard_dim = scheduler, mesh, shard_dim

    def __getattr__(self, name):
        return getattr(self.scheduler, name)

    def sample_time(self, N: int, *, device=None, dtype=None) -> Tensor:
        t = self.scheduler.sample_time(N, device=device, dtype=dtype)
        group = self.mesh.get_group()
        if dist.get_world_size(group) > 1:
            dist.broadcast(t, src=dist.get_global_rank(group, 0), group=group)
        return t

    def add_noise(self, x0, time: Tensor):
        if isinstance(x0, ShardTensor):
            loc = x0.to_local()
            tb = time.reshape((-1,) + (1,) * (loc.ndim - 1))
            out = self.scheduler.alpha(tb) * loc + self.scheduler.sigma(tb) * torch.randn_like(loc)
            return ShardTensor(out, x0.spec)
        return self.scheduler.add_noise(x0, time)

    def init_latents(self, spatial_shape: Tuple[int, ...], tN: Tensor, *, device=None, dtype=None) -> ShardTensor:
        full = (tN.shape[0], *spatial_shape)
        n, r = self.mesh.size(0), self.mesh.get_local_rank(0)
        sizes = chunk_sizes(full[self.shard_dim], n)
        shape = list(full)
        shape[self.shard_dim] = sizes[r]
        noise = torch.randn(shape, device=device, dtype=dtype)
        loc = self.scheduler.sigma(tN.reshape((-1,) + (1,) * len(spatial_shape))) * noise
        return ShardTensor.from_local(loc, self.mesh, [Shard(self.shard_dim)], sharding_shapes={0: sizes})
