"""Time-series samples on the HEALPix grid for the DLWP-HEALPix models.

Parity: ``physicsnemo/datapipes/healpix/timeseries_dataset.py`` (``TimeSeriesDataset``).  The store holds
``inputs [T, C_in, F, H, W]``, ``targets [T, C_out, F, H, W]`` (F = 12 faces), their times, the cell latitudes /
longitudes and optional ``constants [C_c, F, H, W]``.  One ITEM is a whole batch of consecutive start times: the time
axis is read once as one contiguous slab (the access pattern chunked stores like), scaled, and fanned out into
``batch_size`` windows by index tables computed at construction.  Shapes returned: inputs ``[B, F, T_in, C_in, H, W]``,
optional insolation ``[B, F, T_in + T_out, 1, H, W]``, constants ``[F, C_c, H, W]``, targets ``[B, F, T_out, C_out, H, W]``.
In forecast mode (``forecast_init_times``) an item is one initial condition and no target is produced.

The reference reads ``xarray`` / zarr; an ``xarray.Dataset`` is accepted when that package is importable, otherwise the
store is a mapping of arrays (``numpy`` arrays or memory maps) under the same names.
"""
from __future__ import annotations

from typing import Mapping, Optional, Sequence, Union

import numpy as np

from ...utils.insolation import insolation

TimeStep = Union[int, str, np.timedelta64]


def to_timedelta(step: TimeStep) -> np.timedelta64:
    """Integer hours, a ``"6h"`` / ``"30min"`` / ``"1d"`` string or a timedelta → ``numpy.timedelta64[s]``."""
    if isinstance(step, np.timedelta64):
        return step.astype("timedelta64[s]")
    if isinstance(step, (int, np.integer)):
        return np.timedelta64(int(step) * 3600, "s")
    text = str(step).strip().lower()
    for suffix, seconds in (("min", 60), ("h", 3600), ("d", 86400), ("s", 1)):
        if text.endswith(suffix):
            return np.timedelta64(int(float(text[: -len(suffix)]) * seconds), "s")
    raise ValueError(f"cannot read a time step from {step!r}")


class ArrayStore:
    """Uniform view of the data source: attributes ``inputs``, ``targets``, ``time``, ``lat``, ``lon``, ``constants``,
    ``channel_in``, ``channel_out`` (names)."""

    def __init__(self, source):
        get = (lambda k: source[k]) if isinstance(source, Mapping) else (lambda k: getattr(source, k))
        has = (lambda k: k in source) if isinstance(source, Mapping) else (lambda k: hasattr(source, k) or k in getattr(source, "variables", {}))
        raw = lambda k: getattr(get(k), "values", get(k))                    # noqa: E731  (xarray DataArray -> ndarray)
        self.inputs = get("inputs")
        self.targets = get("targets") if has("targets") else None
        self.time = np.asarray(raw("time")).astype("datetime64[s]")
        self.lat, self.lon = np.asarray(raw("lat")), np.asarray(raw("lon"))
        self.constants = np.asarray(raw("constants"), dtype=np.float32) if has("constants") else None
        self.channel_in = [str(c) for c in np.asarray(raw("channel_in"))] if has("channel_in") else None
        self.channel_out = [str(c) for c in np.asarray(raw("channel_out"))] if has("channel_out") else self.channel_in
        self.channel_c = [str(c) for c in np.asarray(raw("channel_c"))] if has("channel_c") else None

    @staticmethod
    def slab(array, start: int, stop: int) -> np.ndarray:
        part = array[start:stop]
        return np.asarray(getattr(part, "values", part), dtype=np.float32)

    def sel(self, channel_in=None, channel_out=None, channel_c=None, time=None) -> "ArrayStore":
        """Sub-store by names / time range, like ``xarray.Dataset.sel`` on the reference's archives.

        ``channel_in`` / ``channel_out`` list variable names in the wanted order; ``channel_c`` lists
        constant names (needs ``channel_c`` names in the source) or indices; ``time`` is a
        ``slice(start, stop)`` of anything ``numpy.datetime64`` accepts, both ends inclusive.  The data
        stay where they are: the result indexes into the parent lazily.
        """
        out = ArrayStore.__new__(ArrayStore)
        out.__dict__.update(self.__dict__)
        t0, t1 = 0, len(self.time)
        if time is not None:
            if time.start is not None:
                t0 = int(np.searchsorted(self.time, np.datetime64(time.start).astype("datetime64[s]"), side="left"))
            if time.stop is not None:
                t1 = int(np.searchsorted(self.time, np.datetime64(time.stop).astype("datetime64[s]"), side="right"))
            out.time = self.time[t0:t1]

        def pick(array, names, wanted):
            if array is None:
                return None, names
            cols = None
            if wanted is not None:
                if names is None:
                    raise KeyError("selecting variables by name needs the channel names of the data")
                missing = [w for w in wanted if w not in names]
                if missing:
                    raise KeyError(f"variables {missing} are not in the data (available: {names})")
                cols = np.asarray([names.index(w) for w in wanted])
                names = list(wanted)
            return (_LazyRows(array, t0, t1, cols) if (cols is not None or time is not None) else array), names

        out.inputs, out.channel_in = pick(self.inputs, self.channel_in, channel_in)
        out.targets, out.channel_out = pick(self.targets, self.channel_out if self.targets is not None else None, channel_out)
        if self.targets is None:
            out.channel_out = out.channel_in if channel_out is None else list(channel_out)
        if channel_c is not None and self.constants is not None:
            names_c = getattr(self, "channel_c", None)
            idx = [names_c.index(c) if isinstance(c, str) else int(c) for c in channel_c] if names_c or all(
                not isinstance(c, str) for c in channel_c) else list(range(len(channel_c)))
            out.constants = self.constants[idx]
            out.channel_c = [str(c) for c in channel_c]
        return out


class _LazyRows:
    """``base[t0:t1][:, cols]`` evaluated per requested time slab (keeps memory-mapped archives on disk)."""

    def __init__(self, base, t0: int, t1: int, cols):
        self.base, self.t0, self.t1, self.cols = base, t0, t1, cols
        n_ch = base.shape[1] if cols is None else len(cols)
        self.shape = (t1 - t0, n_ch) + tuple(base.shape[2:])

    def __len__(self) -> int:
        return self.shape[0]

    def __getitem__(self, key):
        if not isinstance(key, slice):
            raise TypeError("only time slices are supported")
        start, stop, _ = key.indices(self.shape[0])
        part = self.base[self.t0 + start:self.t0 + stop]
        part = np.asarray(getattr(part, "values", part))
        return part if self.cols is None else part[:, self.cols]


class TimeSeriesDataset:
    def __init__(self, dataset, scaling: Optional[Mapping] = None, input_time_dim: int = 1, output_time_dim: int = 1,
                 data_time_step: TimeStep = "3h", time_step: TimeStep = "6h", gap: Optional[TimeStep] = None, batch_size: int = 32,
                 drop_last: bool = False, add_insolation: bool = False, forecast_init_times: Optional[Sequence] = None, meta=None):
        self.ds = dataset if isinstance(dataset, ArrayStore) else ArrayStore(dataset)
        self.scaling = dict(scaling) if scaling else None
        self.input_time_dim, self.output_time_dim = input_time_dim, output_time_dim
        self.data_time_step, self.time_step = to_timedelta(data_time_step), to_timedelta(time_step)
        self.gap = to_timedelta(gap if gap is not None else time_step)
        self.batch_size, self.drop_last, self.add_insolation = batch_size, drop_last, add_insolation
        self.forecast_init_times = forecast_init_times
        self.forecast_mode = forecast_init_times is not None
        dts = int(self.data_time_step / np.timedelta64(1, "s"))
        for label, value in (("time_step", self.time_step), ("gap", self.gap)):
            if int(value / np.timedelta64(1, "s")) % dts:
                raise ValueError(f"'{label}' ({value}) must be a whole number of data time steps ({self.data_time_step})")
        self.interval = int(self.time_step / self.data_time_step)
        gap_steps = int(self.gap / self.data_time_step)
        self._window_length = self.interval * (input_time_dim - 1) + 1 + gap_steps + self.interval * (output_time_dim - 1)
        self._output_delay = self.interval * (input_time_dim - 1) + gap_steps
        if self.forecast_mode:
            self._batch_window = self._window_length
            self.batch_size = 1
            stamps = np.asarray(forecast_init_times).astype("datetime64[s]")
            first = np.searchsorted(self.ds.time, stamps) - self.interval * (input_time_dim - 1)
            if (first < 0).any() or (self.ds.time[np.clip(first + self.interval * (input_time_dim - 1), 0, len(self.ds.time) - 1)] != stamps).any():
                raise ValueError("a forecast initialisation time (or its input history) is not in the data")
            self._forecast_init_indices = first
        else:
            self._batch_window = self._window_length + batch_size - 1
        starts = np.arange(self.batch_size)[:, None]
        self._input_indices = starts + self.interval * np.arange(input_time_dim)[None]
        self._output_indices = starts + self._output_delay + self.interval * np.arange(output_time_dim)[None]
        self.spatial_dims = tuple(self.ds.inputs.shape[2:])
        self.input_scaling = self.target_scaling = None
        self._get_scaling_da()
        self.constants = self.get_constants()

    # ------------------------------------------------------------- scaling
    def _scale_vectors(self, names: Optional[Sequence[str]], count: int):
        if self.scaling is None:
            return {"mean": np.zeros((1, count, 1, 1, 1), np.float32), "std": np.ones((1, count, 1, 1, 1), np.float32)}
        if names is None:
            raise KeyError("scaling by variable name needs the channel names of the data")
        missing = [n for n in names if n not in self.scaling]
        if missing:
            raise KeyError(f"no scaling parameters for the variables {missing}")
        mean = np.array([self.scaling[n]["mean"] for n in names], np.float32).reshape(1, -1, 1, 1, 1)
        std = np.array([self.scaling[n]["std"] for n in names], np.float32).reshape(1, -1, 1, 1, 1)
        return {"mean": mean, "std": std}

    def _get_scaling_da(self) -> None:
        self.input_scaling = self._scale_vectors(self.ds.channel_in, self.ds.inputs.shape[1])
        if self.ds.targets is not None:
            self.target_scaling = self._scale_vectors(self.ds.channel_out, self.ds.targets.shape[1])

    def get_constants(self):
        """Constant fields as ``[F, C_c, H, W]`` (face first, like the model's other inputs), or None."""
        if self.ds.constants is None:
            return None
        return np.ascontiguousarray(np.swapaxes(self.ds.constants, 0, 1))

    # -------------------------------------------------------------- access
    def __len__(self) -> int:
        if self.forecast_mode:
            return len(self._forecast_init_indices)
        n = (len(self.ds.time) - self._window_length + 1) / self.batch_size
        return int(np.floor(n)) if self.drop_last else int(np.ceil(n))

    def _get_time_index(self, item: int):
        if self.forecast_mode:
            start = int(self._forecast_init_indices[item])
            return (start, start + self._window_length), 1
        start = item * self.batch_size
        stop = start + self._batch_window
        size = self.batch_size
        if stop > len(self.ds.time):
            size -= stop - len(self.ds.time)
            stop = len(self.ds.time)
        return (start, stop), size

    def _get_forecast_sol_times(self, item: int) -> np.ndarray:
        (start, stop), _ = self._get_time_index(item)
        return self.ds.time[start:stop]

    def __getitem__(self, item: int):
        if item < 0:
            item += len(self)
        if not 0 <= item < len(self):
            raise IndexError(f"item {item} outside a dataset of {len(self)} batches")
        (start, stop), size = self._get_time_index(item)
        x = (ArrayStore.slab(self.ds.inputs, start, stop) - self.input_scaling["mean"]) / self.input_scaling["std"]
        inputs = x[self._input_indices[:size]]                                   # [B, T_in, C, F, H, W]
        out = [np.ascontiguousarray(np.transpose(inputs, (0, 3, 1, 2, 4, 5)))]
        if self.add_insolation:
            sol = insolation(self._get_forecast_sol_times(item), self.ds.lat, self.ds.lon)[:, None].astype(np.float32)
            both = np.concatenate([self._input_indices[:size], self._output_indices[:size]], axis=1)
            out.append(np.ascontiguousarray(np.transpose(sol[both], (0, 3, 1, 2, 4, 5))))
        if self.constants is not None:
            out.append(self.constants)
        if self.forecast_mode:
            return out
        y = (ArrayStore.slab(self.ds.targets, start, stop) - self.target_scaling["mean"]) / self.target_scaling["std"]
        targets = np.transpose(y[self._output_indices[:size]], (0, 3, 1, 2, 4, 5))
        return out, np.ascontiguousarray(targets)
