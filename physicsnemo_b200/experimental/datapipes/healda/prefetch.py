"""Run a batch transform (typically the host-to-device stage) one or more batches ahead on a side stream.

Parity: ``physicsnemo/experimental/datapipes/healda/prefetch.py`` (``prefetch_map``).  A worker thread
pulls batches from the loader, applies ``transform`` under its own CUDA stream, records an event and
queues the result; the consumer makes its current stream wait on that event (no host-side stream
synchronisation) and marks the tensors as used on it.  Without CUDA the transform simply runs in the
worker thread.
"""
from __future__ import annotations

import dataclasses
import queue
import threading
from typing import Any, Callable, Iterable, Optional

import torch

_END = object()


def _each_tensor(obj, fn) -> None:
    if isinstance(obj, torch.Tensor):
        fn(obj)
    elif isinstance(obj, dict):
        for v in obj.values():
            _each_tensor(v, fn)
    elif isinstance(obj, (list, tuple)):
        for v in obj:
            _each_tensor(v, fn)
    elif dataclasses.is_dataclass(obj) and not isinstance(obj, type):
        for f in dataclasses.fields(obj):
            _each_tensor(getattr(obj, f.name), fn)


class _PrefetchIterator:
    def __init__(self, dataloader: Iterable, transform: Callable[[Any], Any], queue_size: int = 2, cuda_stream=None):
        self.dataloader, self.transform, self.queue_size = dataloader, transform, queue_size
        self._cuda = torch.cuda.is_available()
        self.cuda_stream = cuda_stream if cuda_stream is not None else (torch.cuda.Stream() if self._cuda else None)
        self._queue: "queue.Queue" = queue.Queue(maxsize=queue_size)
        self._thread: Optional[threading.Thread] = None
        self._stop = threading.Event()

    def _put(self, item) -> bool:
        while not self._stop.is_set():
            try:
                self._queue.put(item, timeout=0.1)
                return True
            except queue.Full:
                continue
        return False

    def _work(self, source) -> None:
        try:
            for batch in source:
                if self._stop.is_set():
                    return
                ready = None
                if self._cuda:
                    with torch.cuda.stream(self.cuda_stream):
                        out = self.transform(batch)
                        ready = torch.cuda.Event()
                        ready.record(self.cuda_stream)
                else:
                    out = self.transform(batch)
                if not self._put((out, ready, None)):
                    return
            self._put((_END, None, None))
        except Exception as exc:  # surfaced in the consumer
            self._put((None, None, exc))

    def __len__(self) -> int:
        return len(self.dataloader)

    def __iter__(self):
        self.close()
        self._stop.clear()
        self._queue = queue.Queue(maxsize=self.queue_size)
        self._thread = threading.Thread(target=self._work, args=(iter(self.dataloader),), daemon=True)
        self._thread.start()
        return self

    def __next__(self):
        if self._thread is None:
            raise RuntimeError("Iterator not started. Call __iter__ first.")
        out, ready, error = self._queue.get()
        if error is not None:
            self.close()
            raise error
        if out is _END:
            self.close()
            raise StopIteration
        if ready is not None:
            current = torch.cuda.current_stream()
            current.wait_event(ready)
            _each_tensor(out, lambda t: t.record_stream(current) if t.is_cuda else None)
        return out

    def close(self) -> None:
        self._stop.set()
        if self._thread is not None and self._thread.is_alive():
            self._thread.join(timeout=1.0)
        self._thread = None

    def __del__(self):
        self.close()


def prefetch_map(dataloader: Iterable, transform: Callable[[Any], Any], queue_size: int = 2, cuda_stream=None) -> _PrefetchIterator:
    """Iterator over ``transform(batch)`` for the batches of ``dataloader``, computed ``queue_size`` batches ahead."""
    return _PrefetchIterator(dataloader, transform, queue_size, cuda_stream)
