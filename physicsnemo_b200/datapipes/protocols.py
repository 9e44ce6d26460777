"""Dataset protocols and the prefetch machinery shared by every dataset.

Parity: ``physicsnemo/datapipes/protocols.py`` — ``DatasetBase`` splits loading into a host half
(``_load_host``: file IO / decoding in a thread pool) and a device half (``_consume``: host→device copy and
transforms on a side CUDA stream, ordered against the consumer's stream by an event).  ``submit`` / ``consume``
and ``prefetch`` / ``__getitem__`` are the two ways to drive it.
"""
from __future__ import annotations

import contextlib
import threading
from abc import ABC, abstractmethod
from collections.abc import Mapping
from concurrent.futures import Future, ThreadPoolExecutor
from dataclasses import dataclass, field
from typing import Any, Iterator, Optional

import torch

from .tensordict import is_tensor_collection


@contextlib.contextmanager
def preprocessing_stream(stream):
    if stream is None:
        yield
        return
    with torch.cuda.stream(stream):
        yield


def record_consumer_stream(data: Any, stream) -> None:
    """Tell the caching allocator that ``stream`` uses the tensors produced on the side stream."""
    if isinstance(data, torch.Tensor):
        if data.is_cuda:
            data.record_stream(stream)
    elif is_tensor_collection(data):
        for leaf in data.values(include_nested=True, leaves_only=True):
            if isinstance(leaf, torch.Tensor) and leaf.is_cuda:
                leaf.record_stream(stream)
    elif isinstance(data, Mapping):
        for v in data.values():
            record_consumer_stream(v, stream)
    elif isinstance(data, (list, tuple)):
        for v in data:
            record_consumer_stream(v, stream)


@dataclass
class HostPayload:
    work_item: Any
    data: Any = None
    metadata: Optional[dict[str, Any]] = field(default=None)
    error: Optional[Exception] = field(default=None)


@dataclass
class PrefetchHandle:
    future: Future
    stream: Any = None


class DatasetBase(ABC):
    def __init__(self, *, num_workers: int = 2) -> None:
        self._executor: Optional[ThreadPoolExecutor] = None
        self._num_workers = num_workers
        self._lock = threading.Lock()
        self._inflight: set[Future] = set()
        self._prefetch_handles: dict[int, PrefetchHandle] = {}
        self._events_pending: list = []

    def _pop_events(self) -> list:
        out, self._events_pending = self._events_pending, []
        return out

    @abstractmethod
    def _load(self, index: int) -> tuple[Any, dict[str, Any]]: ...

    @abstractmethod
    def __len__(self) -> int: ...

    def _load_host(self, work_item: Any) -> HostPayload:
        try:
            data, meta = self._load(work_item)
            return HostPayload(work_item=work_item, data=data, metadata=meta)
        except Exception as e:  # noqa: BLE001
            return HostPayload(work_item=work_item, error=e)

    def _consume(self, payload: HostPayload, stream=None, *, defer_sync: bool = False):
        if payload.error is not None:
            raise payload.error
        return payload.data, payload.metadata

    def _ensure_executor(self) -> ThreadPoolExecutor:
        with self._lock:
            if self._executor is None:
                self._executor = ThreadPoolExecutor(max_workers=self._num_workers, thread_name_prefix="datapipe_prefetch")
            return self._executor

    def submit(self, work_item: Any, stream=None) -> PrefetchHandle:
        fut = self._ensure_executor().submit(self._load_host, work_item)
        with self._lock:
            self._inflight.add(fut)
        fut.add_done_callback(self._discard_inflight)
        return PrefetchHandle(future=fut, stream=stream)

    def consume(self, handle: PrefetchHandle, *, defer_sync: bool = False):
        return self._consume(handle.future.result(), handle.stream, defer_sync=defer_sync)

    def __getitem__(self, index: int):
        with self._lock:
            handle = self._prefetch_handles.pop(index, None)
        return self.consume(handle) if handle is not None else self._load(index)

    def prefetch(self, index: int, stream=None) -> None:
        with self._lock:
            if index in self._prefetch_handles:
                return
        handle = self.submit(index, stream)
        with self._lock:
            self._prefetch_handles.setdefault(index, handle)

    def cancel_prefetch(self, index: Optional[int] = None) -> None:
        with self._lock:
            if index is None:
                self._prefetch_handles.clear()
            else:
                self._prefetch_handles.pop(index, None)

    def _discard_inflight(self, fut: Future) -> None:
        with self._lock:
            self._inflight.discard(fut)

    def close(self) -> None:
        with self._lock:
            futs = list(self._inflight)
            self._prefetch_handles.clear()
        for f in futs:
            try:
                f.result(timeout=30.0)
            except Exception:  # noqa: BLE001, S110
                pass
        with self._lock:
            self._inflight.clear()
        if self._executor is not None:
            self._executor.shutdown(wait=True)
            self._executor = None

    def __iter__(self) -> Iterator:
        for i in range(len(self)):
            yield self[i]

    def __enter__(self):
        return self

    def __exit__(self, *exc) -> None:
        self.close()


class IterableDatasetBase(ABC):
    """Generator-style dataset (e.g. the on-device PDE generators); ``yields_batches`` marks pre-batched output."""

    yields_batches: bool = False

    @abstractmethod
    def __iter__(self) -> Iterator[Any]: ...

    def set_epoch(self, epoch: int) -> None:
        return None

    def set_generator(self, generator: torch.Generator) -> None:
        return None

    def close(self) -> None:
        return None

    def __enter__(self):
        return self

    def __exit__(self, *exc) -> None:
        self.close()
