"""Sample indexing over a time axis with gaps: every sample is a window of frames inside one gap-free segment.

Parity: ``physicsnemo/experimental/datapipes/healda/indexing.py`` (``split_array_contiguous``,
``FrameIndexGenerator``, ``MultiCoordIndex``, ``get_flat_indexer``).
"""
from __future__ import annotations

import numpy as np


def split_array_contiguous(x: np.ndarray) -> list:
    """Cut ``x`` wherever the step differs from the first step ``x[1] - x[0]``."""
    x = np.asarray(x)
    if x.size == 0:
        return []
    if x.size == 1:
        return [x]
    breaks = np.flatnonzero(np.diff(x) != x[1] - x[0]) + 1
    return [seg for seg in np.split(x, breaks) if seg.size]


class FrameIndexGenerator:
    """Logical sample index → physical frame indices.

    A window has ``time_length`` frames ``frame_step`` apart and must fit inside one segment, so a
    segment of ``n`` frames offers ``n - (time_length - 1) · frame_step`` windows.  With model
    parallelism over time, rank ``r`` of ``w`` keeps frames ``[r · time_length / w, (r + 1) · time_length / w)``.
    """

    def __init__(self, times, time_length: int, frame_step: int, model_rank: int, model_world_size: int):
        self.time_length, self.frame_step = time_length, frame_step
        self.model_rank, self.model_world_size = model_rank, model_world_size
        self.segments = split_array_contiguous(np.asarray(times))
        self.sizes = [len(s) for s in self.segments]
        span = (time_length - 1) * frame_step
        self.segment_valid_lengths = [max(n - span, 0) for n in self.sizes]
        self._first_frame = np.concatenate([[0], np.cumsum(self.sizes)]).astype(np.int64)
        self._first_sample = np.concatenate([[0], np.cumsum(self.segment_valid_lengths)]).astype(np.int64)
        self.total_samples = int(sum(self.sizes))
        self.valid_length = int(self._first_sample[-1])

    def get_valid_length(self) -> int:
        return self.valid_length

    def _map_logical_to_physical(self, logical_idx: int) -> int:
        if not 0 <= logical_idx < self.valid_length:
            raise IndexError(f"Sample index {logical_idx} out of bounds for {self.valid_length} valid samples")
        seg = int(np.searchsorted(self._first_sample, logical_idx, side="right")) - 1
        return int(self._first_frame[seg] + logical_idx - self._first_sample[seg])

    def generate_frame_indices(self, sample_indices) -> list:
        share = self.time_length // self.model_world_size
        lo, hi = self.model_rank * share, (self.model_rank + 1) * share
        out = []
        for s in sample_indices:
            start = self._map_logical_to_physical(int(s))
            out.append([start + k * self.frame_step for k in range(self.time_length)][lo:hi])
        return out


class MultiCoordIndex:
    """Flat index over ``(sample dims …, window)``; item ``i`` is a ``{dim: index, frame_dim: [frames]}`` mapping."""

    def __init__(self, sample_dims, sample_sizes, frame_dim, frame_indexer: FrameIndexGenerator):
        self.sample_dims, self.sample_sizes = list(sample_dims), [int(s) for s in sample_sizes]
        self.sequence_dim, self._frame_indexer = frame_dim, frame_indexer

    def __len__(self) -> int:
        return int(np.prod(self.sample_sizes, dtype=np.int64)) * self._frame_indexer.get_valid_length()

    def __getitem__(self, i: int) -> dict:
        if not 0 <= i < len(self):
            raise IndexError(i)
        *outer, window = np.unravel_index(i, [*self.sample_sizes, self._frame_indexer.get_valid_length()])
        coords = {d: int(v) for d, v in zip(self.sample_dims, outer)}
        coords[self.sequence_dim] = self._frame_indexer.generate_frame_indices([window])[0]
        return coords


def get_flat_indexer(ds, sample_dims, frame_dim, time_length, frame_step, model_rank, model_world_size) -> MultiCoordIndex:
    """``ds[frame_dim]`` gives the time values (an array, or an object with ``.values``); ``ds.sizes[dim]`` the other extents."""
    times = ds[frame_dim]
    times = np.asarray(times.values if hasattr(times, "values") else times)
    frames = FrameIndexGenerator(times, time_length, frame_step, model_rank, model_world_size)
    return MultiCoordIndex(sample_dims, [ds.sizes[d] for d in sample_dims], frame_dim, frames)
