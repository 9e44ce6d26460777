"""Batched iteration with stream-based prefetch.

Parity: ``physicsnemo/datapipes/dataloader.py`` — sequential / random / user samplers, ``drop_last``, pluggable
collation, and a prefetch path in which an ``IOPump`` keeps ``prefetch_factor × batch_size`` loads in flight, each
consumed on one of ``num_streams`` side CUDA streams; the consumer stream waits once per batch on the recorded
events.  Iterable (generator) datasets are passed through, batched when they do not batch themselves.
"""
from __future__ import annotations

import itertools
import warnings
from typing import Any, Callable, Iterator, Optional

import torch
from torch.utils.data import RandomSampler, Sampler, SequentialSampler

from ._rng import fork_generator
from .collate import Collator, get_collator
from .io_pump import BATCH_BOUNDARY, IOPump
from .protocols import DatasetBase, IterableDatasetBase
from .registry import register


@register()
class DataLoader:
    def __init__(self, dataset: DatasetBase | IterableDatasetBase, *, batch_size: int = 1, shuffle: bool = False,
                 sampler: Optional[Sampler] = None, drop_last: bool = False,
                 collate_fn: Optional[Collator | Callable] = None, collate_metadata: bool = False, prefetch_factor: int = 2,
                 num_streams: int = 4, use_streams: bool = True, seed: int | None = None) -> None:
        if batch_size < 1:
            raise ValueError(f"batch_size must be >= 1, got {batch_size}")
        self.dataset, self.batch_size, self.shuffle, self.drop_last = dataset, batch_size, shuffle, drop_last
        self.prefetch_factor = prefetch_factor
        self._saved_prefetch_factor = prefetch_factor if prefetch_factor > 0 else 2
        self.num_streams = num_streams
        self.use_streams = use_streams and torch.cuda.is_available()
        self._seed, self._epoch = seed, 0
        self._iterable = isinstance(dataset, IterableDatasetBase)
        sampler_gen = None
        if seed is not None:
            master = torch.Generator()
            master.manual_seed(seed)
            sampler_gen, data_gen = fork_generator(master, 2)
            if hasattr(dataset, "set_generator"):
                dataset.set_generator(data_gen)
        if self._iterable:
            if sampler is not None or shuffle:
                warnings.warn("shuffle/sampler are ignored for iterable datasets; the generator controls sample order.", stacklevel=2)
            self.sampler = None
        elif sampler is not None:
            self.sampler = sampler
        elif shuffle:
            self.sampler = RandomSampler(dataset, generator=sampler_gen)
        else:
            self.sampler = SequentialSampler(dataset)
        self.collate_fn = get_collator(collate_fn, collate_metadata=collate_metadata)
        self._streams = [torch.cuda.Stream() for _ in range(num_streams)] if self.use_streams else []

    def __len__(self) -> int:
        if self._iterable:
            raise TypeError("len() is undefined for an iterable (generator) dataset")
        n = len(self.sampler) if hasattr(self.sampler, "__len__") else len(self.dataset)
        return n // self.batch_size if self.drop_last else (n + self.batch_size - 1) // self.batch_size

    def set_epoch(self, epoch: int) -> None:
        self._epoch = epoch
        if hasattr(self.sampler, "set_epoch"):
            self.sampler.set_epoch(epoch)
        if hasattr(self.dataset, "set_epoch"):
            self.dataset.set_epoch(epoch)

    def _generate_batches(self) -> Iterator[list[int]]:
        batch: list[int] = []
        for idx in self.sampler:
            batch.append(idx)
            if len(batch) == self.batch_size:
                yield batch
                batch = []
        if batch and not self.drop_last:
            yield batch

    def __iter__(self):
        if self._iterable:
            yield from self._iter_iterable()
        elif self.prefetch_factor > 0:
            yield from self._iter_prefetch()
        else:
            for batch in self._generate_batches():
                yield self.collate_fn([self.dataset[i] for i in batch])

    def _work_stream(self) -> Iterator[Any]:
        for batch in self._generate_batches():
            yield from batch
            yield BATCH_BOUNDARY

    def _iter_prefetch(self):
        use_streams = bool(self._streams)
        main = torch.cuda.current_stream() if use_streams else None
        counter = itertools.count()

        def dispatch(index):
            stream = self._streams[next(counter) % self.num_streams] if use_streams else None
            return self.dataset.submit(index, stream=stream)

        depth = max(self.prefetch_factor * self.batch_size, 1)
        if use_streams:
            depth = max(depth, self.num_streams)
        samples: list = []
        with IOPump(self._work_stream(), dispatch, depth=depth) as pump:
            for item in pump:
                if item is BATCH_BOUNDARY:
                    if use_streams and hasattr(self.dataset, "_pop_events"):
                        for ev in self.dataset._pop_events():
                            main.wait_event(ev)
                    yield self.collate_fn(samples)
                    samples = []
                else:
                    samples.append(self.dataset.consume(item, defer_sync=use_streams))

    def _iter_iterable(self):
        if getattr(self.dataset, "yields_batches", False):
            yield from self.dataset
            return
        samples: list = []
        for s in self.dataset:
            samples.append(s if isinstance(s, tuple) else (s, {}))
            if len(samples) == self.batch_size:
                yield self.collate_fn(samples)
                samples = []
        if samples and not self.drop_last:
            yield self.collate_fn(samples)

    def disable_prefetch(self) -> None:
        self.prefetch_factor = 0

    def enable_prefetch(self) -> None:
        self.prefetch_factor = self._saved_prefetch_factor

    def close(self) -> None:
        if hasattr(self.dataset, "close"):
            self.dataset.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc) -> None:
        self.close()

    def __repr__(self) -> str:
        return (f"DataLoader(dataset={type(self.dataset).__name__}, batch_size={self.batch_size}, shuffle={self.shuffle}, "
                f"prefetch_factor={self.prefetch_factor}, num_streams={self.num_streams})")
