"""Distributed sampler whose position can be saved and restored in the middle of an epoch.

Parity: ``physicsnemo/experimental/datapipes/healda/samplers.py`` (``RestartableDistributedSampler``).
The order of epoch ``e`` is ``randperm(len, seed + e)`` cut to a multiple of the replica count and
strided by rank, so every rank can rebuild it from ``(seed, epoch)`` alone.
"""
from __future__ import annotations

import torch
import torch.utils.data


class RestartableDistributedSampler(torch.utils.data.Sampler):
    def __init__(self, dataset, rank: int = 0, num_replicas: int = 1, shuffle: bool = True, drop_last: bool = True, seed: int = 42):
        super().__init__()
        if not 0 <= rank < num_replicas:
            raise ValueError(f"rank {rank} is outside [0, {num_replicas})")
        self.len = len(dataset)
        self.rank, self.num_replicas, self.shuffle, self.seed = rank, num_replicas, shuffle, seed
        self.epoch = self.iteration = 0
        self.permutation = None

    def __len__(self) -> int:
        return self.len // self.num_replicas

    def _order(self, epoch: int) -> torch.Tensor:
        if self.shuffle:
            order = torch.randperm(self.len, generator=torch.Generator().manual_seed(self.seed + epoch))
        else:
            order = torch.arange(self.len)
        usable = self.len - self.len % self.num_replicas
        return order[:usable][self.rank::self.num_replicas]

    def set_epoch(self, epoch: int) -> None:
        self.epoch, self.iteration = epoch, 0
        self.permutation = self._order(epoch)

    def restart(self, epoch: int, iteration: int, seed=None) -> None:
        """Continue at sample ``iteration`` of ``epoch`` (what ``state_dict`` recorded)."""
        self.seed = seed or self.seed
        self.set_epoch(epoch)
        self.iteration = iteration

    def state_dict(self) -> dict:
        return {"epoch": self.epoch, "iteration": self.iteration, "seed": self.seed}

    def load_state_dict(self, state: dict) -> None:
        self.restart(state["epoch"], state["iteration"], state.get("seed"))

    def __iter__(self):
        if self.permutation is None:
            self.set_epoch(self.epoch)
        return _EpochIterator(self)

    def __next__(self) -> int:
        """Next index of the current epoch; at its end the sampler moves to the next epoch and raises ``StopIteration``."""
        if self.iteration >= len(self):
            self.set_epoch(self.epoch + 1)
            raise StopIteration
        index = int(self.permutation[self.iteration])
        self.iteration += 1
        return index


class _EpochIterator:
    """One pass over the sampler's current epoch.

    The sampler re-arms itself for the next epoch when it ends, so an iterator that merely forwarded
    ``next`` would never stay exhausted; batch samplers that keep pulling after the first
    ``StopIteration`` (``itertools.islice`` in a loop) would then run on for ever.
    """

    def __init__(self, sampler: RestartableDistributedSampler):
        self._sampler, self._done = sampler, False

    def __iter__(self):
        return self

    def __next__(self) -> int:
        if self._done:
            raise StopIteration
        try:
            return next(self._sampler)
        except StopIteration:
            self._done = True
            raise
