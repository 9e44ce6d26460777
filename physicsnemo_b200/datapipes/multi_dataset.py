"""Concatenation of datasets behind one index space (parity: ``physicsnemo/datapipes/multi_dataset.py``):
``output_strict`` checks that all members expose the same fields; metadata gains ``dataset_index``."""
from __future__ import annotations

import bisect
from typing import Any, Iterator, Optional, Sequence

import torch

from ._rng import fork_generator
from .protocols import DatasetBase
from .registry import register

DATASET_INDEX_METADATA_KEY = "dataset_index"


def _validate_strict_outputs(datasets: Sequence[DatasetBase]) -> list[str]:
    ref = sorted(datasets[0].field_names)
    for i, d in enumerate(datasets[1:], start=1):
        if sorted(d.field_names) != ref:
            raise ValueError(f"output_strict=True requires identical fields; dataset 0 has {ref}, dataset {i} has {sorted(d.field_names)}")
    return ref


@register()
class MultiDataset:
    def __init__(self, *datasets: DatasetBase, output_strict: bool = True) -> None:
        if len(datasets) == 1 and isinstance(datasets[0], (list, tuple)):
            datasets = tuple(datasets[0])
        if not datasets:
            raise ValueError("MultiDataset requires at least one dataset")
        self.datasets = list(datasets)
        self.output_strict = output_strict
        self._field_names = _validate_strict_outputs(self.datasets) if output_strict else None
        self._ends = list(torch.tensor([len(d) for d in self.datasets]).cumsum(0).tolist())

    def _index_to_dataset_and_local(self, index: int) -> tuple[int, int]:
        n = len(self)
        if index < 0:
            index += n
        if not 0 <= index < n:
            raise IndexError(f"Index {index} out of range for MultiDataset with {n} samples")
        which = bisect.bisect_right(self._ends, index)
        return which, index - (self._ends[which - 1] if which else 0)

    def __len__(self) -> int:
        return self._ends[-1]

    def set_generator(self, generator: torch.Generator) -> None:
        for g, d in zip(fork_generator(generator, len(self.datasets)), self.datasets):
            if hasattr(d, "set_generator"):
                d.set_generator(g)

    def set_epoch(self, epoch: int) -> None:
        for d in self.datasets:
            if hasattr(d, "set_epoch"):
                d.set_epoch(epoch)

    def _tag(self, out, which):
        data, meta = out
        meta = dict(meta or {})
        meta[DATASET_INDEX_METADATA_KEY] = which
        return data, meta

    def __getitem__(self, index: int):
        which, local = self._index_to_dataset_and_local(index)
        return self._tag(self.datasets[which][local], which)

    def submit(self, index: int, stream: Optional[Any] = None):
        which, local = self._index_to_dataset_and_local(index)
        return which, self.datasets[which].submit(local, stream=stream)

    def consume(self, handle, *, defer_sync: bool = False):
        which, inner = handle
        return self._tag(self.datasets[which].consume(inner, defer_sync=defer_sync), which)

    def _pop_events(self) -> list:
        return [e for d in self.datasets for e in d._pop_events()]

    def prefetch(self, index: int, stream: Optional[Any] = None) -> None:
        which, local = self._index_to_dataset_and_local(index)
        self.datasets[which].prefetch(local, stream=stream)

    def cancel_prefetch(self, index: Optional[int] = None) -> None:
        if index is None:
            for d in self.datasets:
                d.cancel_prefetch()
        else:
            which, local = self._index_to_dataset_and_local(index)
            self.datasets[which].cancel_prefetch(local)

    def __iter__(self) -> Iterator:
        for i in range(len(self)):
            yield self[i]

    @property
    def field_names(self) -> list[str]:
        return self._field_names if self._field_names is not None else self.datasets[0].field_names

    def close(self) -> None:
        for d in self.datasets:
            d.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc) -> None:
        self.close()

    def __repr__(self) -> str:
        return f"MultiDataset(n_datasets={len(self.datasets)}, len={len(self)}, output_strict={self.output_strict})"
