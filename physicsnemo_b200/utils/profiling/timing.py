"""Device-side timing helpers for benchmarks.

``DeviceTimer`` brackets a region with CUDA events on the launching stream and reports the
maximum over ranks.  ``ExposedCommMeter`` measures how much of the communication kernels'
time is *not* overlapped by compute: it records event pairs on a compute stream and a
communication stream and computes the length of the communication intervals that are not
covered by any compute interval (all timestamps relative to one reference event).
"""
from __future__ import annotations

from typing import List, Tuple

import torch


class DeviceTimer:
    def __init__(self, group=None):
        self.group = group
        self.pairs: List[Tuple[torch.cuda.Event, torch.cuda.Event]] = []

    def __enter__(self):
        self._start = torch.cuda.Event(enable_timing=True)
        self._end = torch.cuda.Event(enable_timing=True)
        self._start.record()
        return self

    def __exit__(self, *exc):
        self._end.record()
        self.pairs.append((self._start, self._end))
        return False

    def total_ms(self, reduce_max: bool = True) -> float:
        torch.cuda.synchronize()
        ms = sum(a.elapsed_time(b) for a, b in self.pairs)
        if reduce_max and torch.distributed.is_available() and torch.distributed.is_initialized():
            t = torch.tensor([ms], dtype=torch.float64, device="cuda")
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX, group=self.group)
            ms = t.item()
        return ms


def _uncovered(intervals: List[Tuple[float, float]], cover: List[Tuple[float, float]]) -> float:
    """Total length of ``intervals`` not covered by the union of ``cover``."""
    cover = sorted(cover)
    merged: List[List[float]] = []
    for a, b in cover:
        if merged and a <= merged[-1][1]:
            merged[-1][1] = max(merged[-1][1], b)
        else:
            merged.append([a, b])
    total = 0.0
    for a, b in intervals:
        cur = a
        for ca, cb in merged:
            if cb <= cur:
                continue
            if ca >= b:
                break
            if ca > cur:
                total += ca - cur
            cur = max(cur, cb)
            if cur >= b:
                break
        if cur < b:
            total += b - cur
    return total


class ExposedCommMeter:
    """Collects (start, end) event pairs tagged "compute" or "comm" and reports exposed comm time."""

    def __init__(self):
        self.ref = torch.cuda.Event(enable_timing=True)
        self.ref.record()
        self.events = {"compute": [], "comm": []}

    def region(self, kind: str, stream=None):
        meter = self

        class _R:
            def __enter__(self_inner):
                self_inner.s = torch.cuda.Event(enable_timing=True)
                self_inner.e = torch.cuda.Event(enable_timing=True)
                self_inner.s.record(stream)
                return self_inner

            def __exit__(self_inner, *exc):
                self_inner.e.record(stream)
                meter.events[kind].append((self_inner.s, self_inner.e))
                return False

        return _R()

    def exposed_ms(self) -> float:
        torch.cuda.synchronize()
        to_t = lambda pair: (self.ref.elapsed_time(pair[0]), self.ref.elapsed_time(pair[1]))  # noqa: E731
        comm = [to_t(p) for p in self.events["comm"]]
        comp = [to_t(p) for p in self.events["compute"]]
        return _uncovered(comm, comp)
