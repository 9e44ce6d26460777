"""Collators: turn a list of ``(TensorDict, metadata)`` samples into a batch (parity:
``physicsnemo/datapipes/collate.py``): ``DefaultCollator`` stacks equal-shape samples, ``ConcatCollator``
concatenates ragged ones and adds a ``batch_idx`` field, ``FunctionCollator`` wraps a callable."""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any, Callable, Optional, Sequence

import torch

from .tensordict import TensorDict, cat_tensordicts, stack_tensordicts


class Collator(ABC):
    @abstractmethod
    def __call__(self, samples: Sequence[tuple[TensorDict, dict[str, Any]]]):
        raise NotImplementedError


def _split(samples):
    if not samples:
        raise ValueError("Cannot collate empty sequence of samples")
    return [d for d, _ in samples], [m for _, m in samples]


class DefaultCollator(Collator):
    def __init__(self, *, stack_dim: int = 0, keys: Optional[list[str]] = None, collate_metadata: bool = False) -> None:
        self.stack_dim, self.keys, self.collate_metadata = stack_dim, keys, collate_metadata

    def __call__(self, samples):
        data, meta = _split(samples)
        if self.keys is not None:
            data = [d.select(*self.keys) for d in data]
        batch = stack_tensordicts(data, dim=self.stack_dim)
        return (batch, list(meta)) if self.collate_metadata else batch


class ConcatCollator(Collator):
    def __init__(self, *, dim: int = 0, add_batch_idx: bool = True, batch_idx_key: str = "batch_idx",
                 keys: Optional[list[str]] = None, collate_metadata: bool = False) -> None:
        self.dim, self.add_batch_idx, self.batch_idx_key = dim, add_batch_idx, batch_idx_key
        self.keys, self.collate_metadata = keys, collate_metadata

    def __call__(self, samples):
        data, meta = _split(samples)
        keys = self.keys or list(data[0].keys())
        for d in data:
            for k in keys:
                if k not in d.keys():
                    raise ValueError(f"Data missing key '{k}'")
        batch = cat_tensordicts([d.select(*keys) for d in data], dim=self.dim)
        if self.add_batch_idx:
            sizes = torch.tensor([d[keys[0]].shape[self.dim] for d in data], device=data[0][keys[0]].device)
            batch[self.batch_idx_key] = torch.repeat_interleave(torch.arange(len(data), device=sizes.device), sizes)
        return (batch, list(meta)) if self.collate_metadata else batch


class FunctionCollator(Collator):
    def __init__(self, fn: Callable) -> None:
        self.fn = fn

    def __call__(self, samples):
        return self.fn(samples)


_default = DefaultCollator()


def default_collate(samples):
    return _default(samples)


def concat_collate(samples, dim: int = 0, add_batch_idx: bool = True):
    return ConcatCollator(dim=dim, add_batch_idx=add_batch_idx)(samples)


def get_collator(collate_fn=None, *, collate_metadata: bool = False) -> Collator:
    if collate_fn is None:
        return DefaultCollator(collate_metadata=collate_metadata)
    if isinstance(collate_fn, Collator):
        return collate_fn
    if callable(collate_fn):
        return FunctionCollator(collate_fn)
    raise TypeError(f"collate_fn must be Collator, callable, or None, got {type(collate_fn).__name__}")
