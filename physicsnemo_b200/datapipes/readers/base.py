"""``Reader``: random access to samples of a data source as CPU ``TensorDict``s (parity:
``physicsnemo/datapipes/readers/base.py``)."""
from __future__ import annotations

import logging
from abc import ABC, abstractmethod
from typing import Any, Iterator

import torch

from .._rng import spawn_generator
from ..tensordict import TensorDict

logger = logging.getLogger(__name__)


class Reader(ABC):
    def __init__(self, *, pin_memory: bool = False, include_index_in_metadata: bool = True,
                 coordinated_subsampling: dict[str, Any] | None = None) -> None:
        self.pin_memory = pin_memory
        self.include_index_in_metadata = include_index_in_metadata
        self._coordinated_subsampling_config = coordinated_subsampling
        self._seed_base: int | None = None
        self._epoch: int = 0

    @abstractmethod
    def _load_sample(self, index: int) -> dict[str, torch.Tensor]:
        raise NotImplementedError

    @abstractmethod
    def __len__(self) -> int:
        raise NotImplementedError

    def _get_field_names(self) -> list[str]:
        return list(self._load_sample(0).keys()) if len(self) else []

    def _get_sample_metadata(self, index: int) -> dict[str, Any]:
        return {}

    @property
    def _supports_coordinated_subsampling(self) -> bool:
        return False

    @property
    def field_names(self) -> list[str]:
        return self._get_field_names()

    def __getitem__(self, index: int) -> tuple[TensorDict, dict[str, Any]]:
        n = len(self)
        if index < 0:
            index += n
        if not 0 <= index < n:
            raise IndexError(f"Index {index} out of range for reader with {n} samples")
        fields = self._load_sample(index)
        meta = self._get_sample_metadata(index)
        if self.include_index_in_metadata:
            meta["index"] = index
        if self.pin_memory and torch.cuda.is_available():
            fields = {k: v.pin_memory() for k, v in fields.items()}
        return TensorDict(fields, device=torch.device("cpu")), meta

    def __iter__(self) -> Iterator[tuple[TensorDict, dict[str, Any]]]:
        for i in range(len(self)):
            try:
                yield self[i]
            except Exception as e:
                msg = f"Sample {i} failed with exception: {type(e).__name__}: {e}"
                logger.error(msg)
                raise RuntimeError(msg) from e

    def set_generator(self, generator: torch.Generator) -> None:
        self._seed_base = generator.initial_seed()

    def set_epoch(self, epoch: int) -> None:
        self._epoch = epoch

    def _index_generator(self, index: int) -> torch.Generator | None:
        """Random stream of one (epoch, sample): identical no matter which worker loads it."""
        return None if self._seed_base is None else spawn_generator(self._seed_base, self._epoch, index)

    def _subsample_slice(self, index: int, total: int) -> slice | None:
        """Contiguous random window shared by all large fields of a sample (coordinated sub-sampling)."""
        cfg = self._coordinated_subsampling_config
        if not cfg:
            return None
        n = int(cfg["n_points"])
        if total <= n:
            return slice(0, total)
        g = self._index_generator(index)
        start = int(torch.randint(0, total - n + 1, (1,), generator=g))
        return slice(start, start + n)

    def close(self) -> None:
        return None

    def __enter__(self) -> "Reader":
        return self

    def __exit__(self, *exc) -> None:
        self.close()

    def __repr__(self) -> str:
        return f"{self.__class__.__name__}(len={len(self)}, pin_memory={self.pin_memory})"
