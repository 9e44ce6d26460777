"""Bounded producer thread that keeps ``depth`` loads in flight ahead of the consumer.

Parity: ``physicsnemo/datapipes/io_pump.py`` — the pump walks a stream of work items (sample indices interleaved
with ``BATCH_BOUNDARY`` markers), dispatches each to the dataset's thread pool and hands the resulting handles to
the consumer in order; a semaphore caps the number of outstanding loads, and errors surface at the consumer.
"""
from __future__ import annotations

import queue
import threading
from typing import Any, Callable, Iterable, Iterator

BATCH_BOUNDARY = object()
_DONE = object()


class _Failure:
    __slots__ = ("exc",)

    def __init__(self, exc: BaseException) -> None:
        self.exc = exc


class IOPump:
    def __init__(self, source: Iterable[Any], dispatch_fn: Callable[[Any], Any], depth: int) -> None:
        self._source, self._dispatch = source, dispatch_fn
        self._slots = threading.Semaphore(max(1, int(depth)))
        self._ready: queue.Queue = queue.Queue()
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, name="datapipe_pump", daemon=True)
        self._thread.start()

    def _run(self) -> None:
        try:
            for item in self._source:
                if self._stop.is_set():
                    break
                if item is BATCH_BOUNDARY:
                    self._ready.put(BATCH_BOUNDARY)
                    continue
                self._slots.acquire()
                if self._stop.is_set():
                    break
                self._ready.put(self._dispatch(item))
        except BaseException as exc:  # noqa: BLE001
            self._ready.put(_Failure(exc))
            return
        self._ready.put(_DONE)

    def __iter__(self) -> Iterator[Any]:
        while True:
            item = self._ready.get()
            if item is _DONE:
                return
            if isinstance(item, _Failure):
                raise item.exc
            yield item
            if item is not BATCH_BOUNDARY:
                self._slots.release()

    def stop(self) -> None:
        if not self._stop.is_set():
            self._stop.set()
            self._slots.release()
            self._thread.join(timeout=5.0)

    def __enter__(self) -> "IOPump":
        return self

    def __exit__(self, *exc) -> None:
        self.stop()
