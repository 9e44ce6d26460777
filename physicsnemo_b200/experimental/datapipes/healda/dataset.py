"""Map-style dataset of (state window, observations) samples.

Parity: ``physicsnemo/experimental/datapipes/healda/dataset.py`` (``ObsERA5Dataset``, ``identity_collate``).
``__getitems__`` returns an already collated batch (the host stage of the transform), so the
``DataLoader`` is used with ``collate_fn=identity_collate`` and a batch sampler.
"""
from __future__ import annotations

import asyncio
from typing import Sequence, Union

import numpy as np

from .indexing import get_flat_indexer
from .loaders import ArrayStateStore
from .protocols import ObsLoader, Transform
from .time_utils import as_cftime

DEFAULT_TEST_YEAR = 2022


def _years(times: np.ndarray) -> np.ndarray:
    return times.astype("datetime64[Y]").astype(int) + 1970


class ObsERA5Dataset:
    def __init__(self, era5_data: ArrayStateStore, obs_loader: ObsLoader, transform: Transform, *,
                 split: Union[str, Sequence[int]] = "", time_length: int = 1, frame_step: int = 1, model_rank: int = 0,
                 model_world_size: int = 1, test_year: int = DEFAULT_TEST_YEAR):
        years = _years(era5_data.times)
        if isinstance(split, str):
            masks = {"train": years != test_year, "test": years == test_year, "": np.ones(years.shape, dtype=bool)}
            if split not in masks:
                raise ValueError(f"split must be 'train', 'test', '' or a list of years, got {split!r}")
            keep = masks[split]
        else:
            keep = np.isin(years, np.asarray(list(split)))
        self._era5 = era5_data.isel_time(keep)
        self.batch_info = era5_data.batch_info
        self._obs_loader, self.transform, self.time_length = obs_loader, transform, time_length
        self.npix = self._era5.data.shape[-1]
        self._indexer = get_flat_indexer(self._era5, [], "time", time_length=time_length, frame_step=frame_step,
                                         model_rank=model_rank, model_world_size=model_world_size)

    def __len__(self) -> int:
        return len(self._indexer)

    @property
    def times(self) -> np.ndarray:
        return self._era5.times

    def get(self, i: int):
        """``(times, frames)`` of sample ``i``: one ``{"state", "obs"}`` mapping per frame this rank owns."""
        frames = self._indexer[i]["time"]
        when = self._era5.times[frames]
        state = self._era5.frames(frames)
        obs = asyncio.run(self._obs_loader.sel_time(when))["obs"]
        return [as_cftime(t) for t in when], [{"state": state[k], "obs": obs[k]} for k in range(len(frames))]

    def __getitem__(self, i: int):
        return self.__getitems__([i])

    def __getitems__(self, indexes):
        times, frames = zip(*(self.get(int(i)) for i in indexes))
        return self.transform.transform(list(times), list(frames))


def identity_collate(obj):
    return obj
