"""Small data-loading helpers (parity: ``physicsnemo/experimental/utils/{cached_dataset,prefetch}.py``)."""
from __future__ import annotations

import os
import tempfile
from abc import ABC, abstractmethod
from collections.abc import Callable, Iterable, Iterator
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import Any, Sequence

import torch
from torch.utils.data import Dataset


class CachedPreprocessingDataset(Dataset, ABC):
    """Map-style dataset over files whose ``preprocess`` result is cached as ``<cache_dir>/<stem>.pt`` on first access."""

    def __init__(self, sample_paths: Sequence[Path | str], cache_dir: Path | str | None = None):
        self.sample_paths = [Path(p) for p in sample_paths]
        self.cache_dir = Path(cache_dir) if cache_dir is not None else None
        if not self.sample_paths:
            raise ValueError("sample_paths is empty; the dataset must contain at least one sample.")
        if self.cache_dir is not None:
            self.cache_dir.mkdir(parents=True, exist_ok=True)
        missing = [p for p in self.sample_paths if not p.exists()]
        if missing:
            raise FileNotFoundError(f"The following sample paths were given, but do not exist:\n{missing}")

    def __len__(self) -> int:
        return len(self.sample_paths)

    def __getitem__(self, index) -> Any:
        path = self.sample_paths[index]
        cache = (self.cache_dir / path.name).with_suffix(".pt") if self.cache_dir is not None else None
        if cache is not None and cache.exists():
            return torch.load(cache, weights_only=False)
        sample = self.preprocess(sample_path=path)
        if cache is not None:                                  # write-then-rename: concurrent workers never read a partial file
            fd, tmp = tempfile.mkstemp(dir=self.cache_dir, suffix=".tmp")
            os.close(fd)
            torch.save(sample, tmp)
            os.replace(tmp, cache)
        return sample

    @staticmethod
    @abstractmethod
    def preprocess(sample_path: Path) -> Any: ...


class _PrefetchMap:
    def __init__(self, iterable: Iterable, fn: Callable) -> None:
        self._iterable, self._fn = iterable, fn

    def __iter__(self) -> Iterator:
        with ThreadPoolExecutor(max_workers=1) as pool:
            it = iter(self._iterable)
            try:
                future = pool.submit(self._fn, next(it))
            except StopIteration:
                return
            for item in it:                                    # item i+1 is being mapped while the consumer works on item i
                nxt = pool.submit(self._fn, item)
                yield future.result()
                future = nxt
            yield future.result()

    def __len__(self) -> int:
        return len(self._iterable)


def prefetch_map(iterable: Iterable, fn: Callable) -> _PrefetchMap:
    """``map(fn, iterable)`` evaluated one element ahead on a worker thread (e.g. host-to-device copies)."""
    return _PrefetchMap(iterable, fn)


__all__ = ["CachedPreprocessingDataset", "prefetch_map"]
