"""State and observation sources that need no archive format: arrays in memory (or memory-mapped) and per-window tables.

Parity: the roles of ``physicsnemo/experimental/datapipes/healda/loaders/{era5,ufs_obs}.py``: a state
store indexed by time and an asynchronous observation loader that returns, for every analysis time,
all observations inside ``[t + lo, t + hi]`` hours (``obs_context_hours``), joined with the channel
attributes, filtered, normalised and tagged with local channel and sensor ids.  The reference reads
zarr / parquet archives of a fixed layout; these classes take the same information as arrays.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional, Sequence

import numpy as np

from .configs import SensorRegistry, concat_tables, empty_table, take_rows
from .transforms.obs_filtering import filter_observations
from .types import BatchInfo


class ArrayStateStore:
    """``data[time, channel, pixel]`` with its time axis and channel names; ``sizes`` / ``["time"]`` mimic a labelled array."""

    def __init__(self, data, times, channels: Sequence[str], center=None, scales=None, time_step: int = 6):
        self.data, self.times, self.channels = data, np.asarray(times).astype("datetime64[ns]"), list(channels)
        if data.shape[0] != self.times.shape[0] or data.shape[1] != len(self.channels):
            raise ValueError(f"data {tuple(data.shape)} does not match {self.times.shape[0]} times x {len(self.channels)} channels")
        n = len(self.channels)
        self.batch_info = BatchInfo(channels=self.channels, time_step=time_step,
                                    center=np.zeros(n) if center is None else np.asarray(center),
                                    scales=np.ones(n) if scales is None else np.asarray(scales))

    @property
    def sizes(self) -> dict:
        return {"time": self.data.shape[0], "variable": self.data.shape[1], "pixel": self.data.shape[2]}

    def __getitem__(self, key: str):
        if key == "time":
            return self.times
        raise KeyError(key)

    def isel_time(self, keep) -> "ArrayStateStore":
        keep = np.asarray(keep)
        rows = np.flatnonzero(keep) if keep.dtype == bool else keep
        store = ArrayStateStore.__new__(ArrayStateStore)
        store.data, store.times, store.channels, store.batch_info = _Rows(self.data, rows), self.times[rows], self.channels, self.batch_info
        return store

    def frames(self, indices: Sequence[int]) -> np.ndarray:
        return np.stack([np.asarray(self.data[int(i)], dtype=np.float32) for i in indices])


class _Rows:
    """Lazy row selection of an array-like (keeps a memory-mapped store on disk)."""

    def __init__(self, base, rows):
        self.base, self.rows = base, np.asarray(rows)
        self.shape = (len(self.rows),) + tuple(base.shape[1:])

    def __getitem__(self, i):
        return self.base[int(self.rows[i])]


class TableObsLoader:
    """Observation loader over per-window tables ``{window time → {column → array}}``.

    ``sel_time(times)`` gathers, for each requested time ``t``, the windows ``t + lo + spacing, …,
    t + hi`` (hours, every ``data_spacing``), adds the channel attributes from the sensor registry,
    applies :func:`filter_observations`, normalises ``Observation`` with the channel mean / standard
    deviation and returns one table per time under ``"obs"``.
    """

    def __init__(self, windows: Mapping, registry: SensorRegistry, sensors: Optional[Sequence[str]] = None,
                 obs_context_hours=(-3, 3), data_spacing: int = 3, qc_filter: bool = False,
                 drop_obs_channel_ids: Sequence[int] = (), **conventional_options):
        self.registry, self.qc_filter = registry, qc_filter
        self.sensors = list(sensors) if sensors is not None else [s.name for s in registry.sensors]
        unknown = [s for s in self.sensors if s not in registry]
        if unknown:
            raise ValueError(f"Unconfigured sensor: {unknown[0]}. Available: {list(registry.name_to_id)}")
        self.windows = {np.datetime64(k, "ns"): v for k, v in windows.items()}
        self.obs_context_hours, self.data_spacing = obs_context_hours, data_spacing
        self.drop_obs_channel_ids = np.asarray(list(drop_obs_channel_ids), dtype=np.int64)
        self.conventional_options = conventional_options
        self._stats = registry.channel_stats()
        self._sensor_ids = np.asarray([registry.name_to_id[s] for s in self.sensors], dtype=np.int64)
        self._ready: Dict = {}

    def interval_times(self, t) -> np.ndarray:
        lo, hi = self.obs_context_hours
        hours = np.arange(lo + self.data_spacing, hi + 1, self.data_spacing)
        return np.datetime64(t, "ns") + hours.astype("timedelta64[h]")

    def _prepare(self, window) -> Optional[dict]:
        if window in self._ready:
            return self._ready[window]
        table = self.windows.get(window)
        if table is not None and len(table["Observation"]):
            ch = np.asarray(table["Global_Channel_ID"]).astype(np.int64)
            table = dict(table)
            for name in ("sensor_id", "local_channel_id", "min_valid", "max_valid", "mean", "stddev", "is_conv"):
                table[name] = self._stats[name][ch]
            table = take_rows(table, np.isin(table["sensor_id"], self._sensor_ids))
            table = filter_observations(table, self.qc_filter, **self.conventional_options)
            if self.drop_obs_channel_ids.size:
                table = take_rows(table, ~np.isin(table["Global_Channel_ID"], self.drop_obs_channel_ids))
            table["Observation"] = ((table["Observation"] - table["mean"]) / table["stddev"]).astype(np.float32)
            for extra in ("min_valid", "max_valid", "mean", "stddev", "is_conv"):
                table.pop(extra)
        else:
            table = None
        self._ready[window] = table
        return table

    async def sel_time(self, times) -> dict:
        out = []
        for t in times:
            parts = [self._prepare(w) for w in self.interval_times(t)]
            parts = [p for p in parts if p is not None]
            out.append(concat_tables(parts) if parts else empty_table())
        return {"obs": out}
