"""Small helpers of the diffusion tool-kit (parity: ``physicsnemo/diffusion/utils/utils.py``)."""
from __future__ import annotations

from typing import Iterator, List, Optional, Sequence

import numpy as np
import torch
from torch import Tensor


def apply_loss_weight(w: Tensor, data_ndim: int) -> Tensor:
    """Reshape a per-sample ``(N,)`` or per-sample-per-channel ``(N, C)`` weight for broadcasting."""
    if w.ndim not in (1, 2):
        raise ValueError(f"loss weight must have shape (N,) or (N, C), got {tuple(w.shape)}")
    return w.reshape(*w.shape, *([1] * (data_ndim - w.ndim)))


class StackedRandomGenerator:
    """One ``torch.Generator`` per sample so that results do not depend on the batch composition."""

    def __init__(self, device, seeds: Sequence[int]):
        self.generators = [torch.Generator(device).manual_seed(int(seed) % (1 << 32)) for seed in seeds]

    def _check(self, size):
        if size[0] != len(self.generators):
            raise ValueError(f"Expected first dimension of size {len(self.generators)}, got {size[0]}")

    def randn(self, size, **kwargs) -> Tensor:
        self._check(size)
        return torch.stack([torch.randn(size[1:], generator=g, **kwargs) for g in self.generators])

    def randn_like(self, input: Tensor) -> Tensor:
        return self.randn(input.shape, dtype=input.dtype, layout=input.layout, device=input.device)

    def randt(self, nu: int, size, **kwargs) -> Tensor:
        """Student-t samples with ``nu`` degrees of freedom."""
        self._check(size)
        outs = []
        for g in self.generators:
            z = torch.randn(size[1:], generator=g, **kwargs)
            chi = torch.stack([torch.randn(size[1:], generator=g, **kwargs) ** 2 for _ in range(nu)]).sum(0)
            outs.append(z / torch.sqrt(chi / nu))
        return torch.stack(outs)

    def randint(self, *args, size, **kwargs) -> Tensor:
        self._check(size)
        return torch.stack([torch.randint(*args, size=size[1:], generator=g, **kwargs) for g in self.generators])


class InfiniteSampler(torch.utils.data.Sampler):
    """Endless shuffled index stream, disjoint across ranks, with a sliding shuffle window."""

    def __init__(self, dataset, rank: int = 0, num_replicas: int = 1, shuffle: bool = True, seed: int = 0,
                 window_size: float = 0.5, start_idx: int = 0):
        if not len(dataset) > 0:
            raise ValueError("Dataset must contain at least one item")
        if not num_replicas > 0 or not 0 <= rank < num_replicas or not 0 <= window_size <= 1:
            raise ValueError("invalid sampler arguments")
        super().__init__()
        self.dataset, self.rank, self.num_replicas = dataset, rank, num_replicas
        self.shuffle, self.seed, self.window_size, self.start_idx = shuffle, seed, window_size, start_idx

    def __iter__(self) -> Iterator[int]:
        order = np.arange(len(self.dataset))
        rnd, window = None, 0
        if self.shuffle:
            rnd = np.random.RandomState(self.seed)
            rnd.shuffle(order)
            window = int(np.rint(order.size * self.window_size))
        idx = self.start_idx
        while True:
            i = idx % order.size
            if idx % self.num_replicas == self.rank:
                yield int(order[i])
            if window >= 2:
                j = (i - rnd.randint(window)) % order.size
                order[i], order[j] = order[j], order[i]
            idx += 1
