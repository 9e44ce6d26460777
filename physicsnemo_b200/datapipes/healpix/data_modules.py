"""Dataset assembly and loaders for the HEALPix time-series pipes.

Parity: ``physicsnemo/datapipes/healpix/data_modules.py`` (``create_time_series_dataset_classic`` ``:216``,
``open_time_series_dataset_classic_prebuilt`` ``:185``, ``…_on_the_fly`` ``:66``, ``TimeSeriesDataModule``
``:363``, ``CoupledTimeSeriesDataModule`` ``:796``).  The reference merges per-variable netCDF files into a
zarr store with ``xarray``; neither package is installed here, so the archive format of this module is
a directory of ``.npy`` arrays (memory-mapped on opening), with per-variable ``.npy`` / ``.npz`` sources:

* source: ``<src>/<prefix><variable><suffix>.npy`` ``[time, face, height, width]`` per variable, and
  ``<src>/<prefix>coords<suffix>.npz`` with ``time``, ``lat``, ``lon`` (constants: one ``.npy``
  ``[face, height, width]`` per constant file name);
* archive: ``<dst>/<dataset_name>/{inputs,targets,constants}.npy`` + ``meta.npz``.
"""
from __future__ import annotations

import os
from typing import Mapping, Optional, Sequence

import numpy as np
import torch
from torch.utils.data import DataLoader
from torch.utils.data.distributed import DistributedSampler

from ...distributed import DistributedManager
from .coupledtimeseries_dataset import CoupledTimeSeriesDataset
from .timeseries_dataset import ArrayStore, TimeSeriesDataset


def _get_file_name(path: str, prefix: Optional[str], var: str, suffix: Optional[str], ext: str = ".npy") -> str:
    return os.path.join(path, f"{prefix or ''}{var}{suffix or ''}{ext}")


def _read_sources(directory, variables, prefix, suffix) -> np.ndarray:
    return np.stack([np.load(_get_file_name(directory, prefix, v, suffix), mmap_mode="r") for v in variables], axis=1)


def _coords(directory, prefix, suffix) -> dict:
    with np.load(_get_file_name(directory, prefix, "coords", suffix, ".npz")) as z:
        return {k: z[k] for k in ("time", "lat", "lon")}


def open_time_series_dataset_classic_on_the_fly(directory: str, input_variables: Sequence[str],
                                                output_variables: Optional[Sequence[str]] = None,
                                                constants: Optional[Mapping[str, str]] = None, prefix: Optional[str] = None,
                                                suffix: Optional[str] = None, batch_size: int = 32) -> ArrayStore:
    """Stack the per-variable source files in memory (no archive is written)."""
    source = dict(_coords(directory, prefix, suffix), inputs=_read_sources(directory, input_variables, prefix, suffix),
                  channel_in=np.asarray(list(input_variables)))
    if output_variables is not None and list(output_variables) != list(input_variables):
        source["targets"] = _read_sources(directory, output_variables, prefix, suffix)
        source["channel_out"] = np.asarray(list(output_variables))
    if constants:
        source["constants"] = np.stack([np.load(_get_file_name(directory, prefix, f, suffix)) for f in constants])
        source["channel_c"] = np.asarray(list(constants.values()))
    return ArrayStore(source)


def create_time_series_dataset_classic(src_directory: str, dst_directory: str, dataset_name: str,
                                       input_variables: Sequence[str], output_variables: Optional[Sequence[str]] = None,
                                       constants: Optional[Mapping[str, str]] = None, prefix: Optional[str] = None,
                                       suffix: Optional[str] = None, batch_size: int = 32, scaling: Optional[Mapping] = None,
                                       overwrite: bool = False) -> str:
    """Merge the per-variable sources into one archive directory (time-major arrays); returns its path.

    An existing archive is reused unless ``overwrite``.  ``scaling`` is only checked for completeness
    here (every variable needs ``mean`` / ``std``); the data are stored unscaled.
    """
    out = os.path.join(dst_directory, dataset_name)
    if os.path.exists(os.path.join(out, "meta.npz")) and not overwrite:
        return out
    if scaling is not None:
        missing = [v for v in list(input_variables) + list(output_variables or []) if v not in scaling]
        if missing:
            raise KeyError(f"no scaling parameters for the variables {missing}")
    os.makedirs(out, exist_ok=True)
    store = open_time_series_dataset_classic_on_the_fly(src_directory, input_variables, output_variables, constants, prefix, suffix)
    np.save(os.path.join(out, "inputs.npy"), np.ascontiguousarray(store.inputs))
    meta = dict(time=store.time, lat=store.lat, lon=store.lon, channel_in=np.asarray(store.channel_in))
    if store.targets is not None:
        np.save(os.path.join(out, "targets.npy"), np.ascontiguousarray(store.targets))
        meta["channel_out"] = np.asarray(store.channel_out)
    if store.constants is not None:
        np.save(os.path.join(out, "constants.npy"), store.constants)
        meta["channel_c"] = np.asarray(store.channel_c)
    np.savez(os.path.join(out, "meta.npz"), **meta)
    return out


def open_time_series_dataset_classic_prebuilt(directory: str, dataset_name: str, constants: bool = False,
                                              batch_size: int = 32) -> ArrayStore:
    """Open an archive written by :func:`create_time_series_dataset_classic`; the big arrays stay memory-mapped."""
    root = os.path.join(directory, dataset_name)
    if not os.path.exists(os.path.join(root, "meta.npz")):
        raise FileNotFoundError(f"Dataset doesn't appear to exist at {root}")
    with np.load(os.path.join(root, "meta.npz")) as z:
        source = {k: z[k] for k in z.files}
    source["inputs"] = np.load(os.path.join(root, "inputs.npy"), mmap_mode="r")
    if os.path.exists(os.path.join(root, "targets.npy")):
        source["targets"] = np.load(os.path.join(root, "targets.npy"), mmap_mode="r")
    if constants:
        source["constants"] = np.load(os.path.join(root, "constants.npy"))
    else:
        source.pop("channel_c", None)
    return ArrayStore(source)


class TimeSeriesDataModule:
    """Builds the train / validation / test datasets of one archive and hands out their loaders.

    ``splits`` holds ``{train,val,test}_date_{start,end}``; without it (or with ``forecast_init_times``)
    only ``test_dataset`` exists and covers the whole archive.  A dataset item is already a batch, so
    the loaders use ``batch_size=None``.  ``dataset`` may be passed directly (an :class:`ArrayStore` or
    a mapping of arrays) instead of directories.
    """

    dataset_class = TimeSeriesDataset

    def __init__(self, src_directory: str = ".", dst_directory: str = ".", dataset_name: str = "dataset",
                 prefix: Optional[str] = None, suffix: Optional[str] = None, data_format: str = "classic", batch_size: int = 32,
                 drop_last: bool = False, input_variables: Optional[Sequence[str]] = None,
                 output_variables: Optional[Sequence[str]] = None, constants: Optional[Mapping[str, str]] = None,
                 scaling: Optional[Mapping] = None, splits: Optional[Mapping] = None, presteps: int = 0, input_time_dim: int = 1,
                 output_time_dim: int = 1, data_time_step="3h", time_step="6h", gap=None, shuffle: bool = True,
                 add_insolation: bool = False, cube_dim: int = 64, num_workers: int = 4, pin_memory: bool = True,
                 prebuilt_dataset: bool = True, forecast_init_times: Optional[Sequence] = None, dataset=None):
        if data_format != "classic":
            raise ValueError("'data_format' must be one of ['classic']")
        self.src_directory, self.dst_directory, self.dataset_name = src_directory, dst_directory, dataset_name
        self.prefix, self.suffix, self.data_format = prefix, suffix, data_format
        self.batch_size, self.drop_last = batch_size, drop_last
        self.input_variables = list(input_variables) if input_variables is not None else None
        self.output_variables = list(output_variables) if output_variables is not None else self.input_variables
        self.constants, self.scaling, self.splits = constants, scaling, splits
        self.presteps = presteps
        self.input_time_dim = input_time_dim + presteps * input_time_dim
        self.output_time_dim, self.data_time_step, self.time_step, self.gap = output_time_dim, data_time_step, time_step, gap
        self.shuffle, self.add_insolation, self.cube_dim = shuffle, add_insolation, cube_dim
        self.num_workers, self.pin_memory, self.prebuilt_dataset = num_workers, pin_memory, prebuilt_dataset
        self.forecast_init_times = forecast_init_times
        self._given = dataset
        self.train_dataset = self.val_dataset = self.test_dataset = None
        self.dataset_batch_size, self.dataloader_batch_size, self.collate_fn = batch_size, None, None
        self.setup()

    # ------------------------------------------------------------ assembly
    def _archive_variables(self) -> list:
        return list(self.input_variables)

    def _open(self) -> ArrayStore:
        if self._given is not None:
            return self._given if isinstance(self._given, ArrayStore) else ArrayStore(self._given)
        want_in = self._archive_variables()
        if not self.prebuilt_dataset:
            return open_time_series_dataset_classic_on_the_fly(self.dst_directory, want_in, self.output_variables, self.constants,
                                                               self.prefix, self.suffix, self.batch_size)
        if not DistributedManager.is_initialized():
            DistributedManager.initialize()
        rank = DistributedManager().rank
        if rank == 0:                                     # one writer; the others wait for the finished archive
            create_time_series_dataset_classic(self.src_directory, self.dst_directory, self.dataset_name, want_in,
                                               self.output_variables, self.constants, self.prefix, self.suffix, self.batch_size,
                                               self.scaling)
        if torch.distributed.is_initialized():
            torch.distributed.barrier()
        return open_time_series_dataset_classic_prebuilt(self.dst_directory, self.dataset_name, self.constants is not None,
                                                         self.batch_size)

    def _dataset_args(self) -> dict:
        return dict(scaling=self.scaling, input_time_dim=self.input_time_dim, output_time_dim=self.output_time_dim,
                    data_time_step=self.data_time_step, time_step=self.time_step, gap=self.gap, batch_size=self.dataset_batch_size,
                    drop_last=self.drop_last, add_insolation=self.add_insolation)

    def setup(self) -> None:
        store = self._open()
        if self.input_variables is not None:
            store = store.sel(channel_in=self._archive_variables(),
                              channel_out=self.output_variables if store.targets is not None else None)
        if self.constants is not None and store.constants is not None and store.channel_c is not None:
            store = store.sel(channel_c=list(self.constants.values()))
        make = lambda s, **extra: self.dataset_class(s, **self._dataset_args(), **extra)  # noqa: E731
        if self.splits is not None and self.forecast_init_times is None:
            sp = self.splits
            part = lambda which: store.sel(time=slice(sp[f"{which}_date_start"], sp[f"{which}_date_end"]))  # noqa: E731
            self.train_dataset, self.val_dataset, self.test_dataset = make(part("train")), make(part("val")), make(part("test"))
        else:
            self.test_dataset = make(store, forecast_init_times=self.forecast_init_times)

    def get_constants(self) -> Optional[np.ndarray]:
        if self.constants is None:
            return None
        source = self.train_dataset if self.train_dataset is not None else self.test_dataset
        return source.get_constants()

    # ------------------------------------------------------------- loaders
    def _loader(self, dataset, shuffle: bool, num_shards: int, shard_id: int, drop_last_shard: bool):
        sampler = None
        if num_shards > 1:
            sampler = DistributedSampler(dataset, num_replicas=num_shards, rank=shard_id, shuffle=shuffle, drop_last=drop_last_shard)
            shuffle = False
        loader = DataLoader(dataset=dataset, pin_memory=self.pin_memory and torch.cuda.is_available(), num_workers=self.num_workers,
                            shuffle=shuffle, drop_last=False, sampler=sampler, collate_fn=self.collate_fn,
                            batch_size=self.dataloader_batch_size)
        return loader, sampler

    def train_dataloader(self, num_shards: int = 1, shard_id: int = 0):
        return self._loader(self.train_dataset, self.shuffle, num_shards, shard_id, True)

    def val_dataloader(self, num_shards: int = 1, shard_id: int = 0):
        return self._loader(self.val_dataset, False, num_shards, shard_id, False)

    def test_dataloader(self, num_shards: int = 1, shard_id: int = 0):
        return self._loader(self.test_dataset, False, num_shards, shard_id, False)


class CoupledTimeSeriesDataModule(TimeSeriesDataModule):
    """The same with :class:`CoupledTimeSeriesDataset`: the archive also holds the variables the couplers read."""

    dataset_class = CoupledTimeSeriesDataset

    def __init__(self, *args, couplings: Sequence = (), add_train_noise: bool = False, train_noise_params: Optional[Mapping] = None,
                 train_noise_seed: int = 42, **kwargs):
        self.couplings, self.add_train_noise = list(couplings), add_train_noise
        self.train_noise_params, self.train_noise_seed = train_noise_params, train_noise_seed
        self._base_input_time_dim = kwargs.get("input_time_dim", 1)
        super().__init__(*args, **kwargs)

    def _get_coupled_vars(self) -> list:
        out = []
        for c in self.couplings:
            out += list(c["params"]["variables"])
        return out

    def _archive_variables(self) -> list:
        extra = [v for v in self._get_coupled_vars() if v not in self.input_variables]
        return list(self.input_variables) + extra

    def _dataset_args(self) -> dict:
        args = super()._dataset_args()
        args.update(input_variables=self.input_variables, output_variables=self.output_variables,
                    input_time_dim=self._base_input_time_dim, presteps=self.presteps, couplings=self.couplings,
                    add_train_noise=self.add_train_noise, train_noise_params=self.train_noise_params,
                    train_noise_seed=self.train_noise_seed)
        return args
