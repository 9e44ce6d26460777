"""ERA5-style time-series datapipe over per-year arrays ``[time, channel, lat, lon]`` with device-side prefetch.

Parity: ``physicsnemo/datapipes/climate/era5_hdf5.py`` (``ERA5HDF5Datapipe``: yearly files with a ``fields`` dataset,
``channels`` subset, ``stride`` between input and targets, ``num_steps`` targets, ``num_history`` extra inputs,
normalisation by ``global_means`` / ``global_stds`` arrays ``[1, C, 1, 1]``, optional ``latlon`` / cos-zenith features,
sharding of the samples over ranks, shuffling per epoch).  The reference builds this on NVIDIA DALI; here the yearly
files are memory-mapped ``.npy`` arrays (or HDF5 files when ``h5py`` is importable), batches are assembled in pinned
host buffers by a background thread and copied to the GPU on a side stream one batch ahead, and normalisation runs on
the device.  Each item is ``[{"invar": [B, (H+1)·C?, …] …}]`` in the reference's layout:
``invar [B, C, lat, lon]`` (``[B, H+1, C, lat, lon]`` when ``num_history > 0``) and ``outvar [B, num_steps, C, lat, lon]``.
"""
from __future__ import annotations

import queue
import threading
from pathlib import Path
from typing import Iterator, List, Sequence

import numpy as np
import torch


def _open_year(path: Path):
    if path.suffix == ".npy":
        return np.load(path, mmap_mode="r")
    try:
        import h5py
    except ImportError as e:  # pragma: no cover
        raise ImportError("reading .h5 yearly files needs h5py; convert them to .npy or install h5py") from e
    return h5py.File(path, "r")["fields"]


class ERA5Datapipe:
    def __init__(self, data_dir: str, stats_dir: str | None = None, channels: Sequence[int] | None = None, batch_size: int = 1, num_steps: int = 1,
                 stride: int = 1, num_history: int = 0, patch_size: Sequence[int] | int | None = None, shuffle: bool = True, device: str | torch.device = "cuda",
                 process_rank: int = 0, world_size: int = 1, seed: int = 0, prefetch: int = 2, drop_last: bool = True):
        self.data_dir = Path(data_dir)
        if not self.data_dir.is_dir():
            raise IOError(f"Error, data directory {self.data_dir} does not exist")
        self.files = sorted([p for p in self.data_dir.iterdir() if p.suffix in (".npy", ".h5", ".hdf5")])
        if not self.files:
            raise IOError(f"no yearly .npy / .h5 files in {self.data_dir}")
        self.arrays = [_open_year(p) for p in self.files]
        shape0 = self.arrays[0].shape
        if any(a.shape[1:] != shape0[1:] for a in self.arrays):
            raise ValueError("all yearly files must share their channel and grid shape")
        self.channels = list(channels) if channels is not None else list(range(shape0[1]))
        if max(self.channels) >= shape0[1]:
            raise ValueError(f"Provided channel has indexes greater than the number of channels {shape0[1]}")
        self.batch_size, self.num_steps, self.stride, self.num_history = batch_size, num_steps, stride, num_history
        self.shuffle, self.seed, self.rank, self.world = shuffle, seed, process_rank, world_size
        self.prefetch, self.drop_last = max(1, prefetch), drop_last
        self.device = torch.device(device if (str(device) != "cuda" or torch.cuda.is_available()) else "cpu")
        lat, lon = shape0[2:]
        if patch_size is not None:
            ps = (patch_size, patch_size) if isinstance(patch_size, int) else tuple(patch_size)
            lat, lon = ps[0] * (lat // ps[0]), ps[1] * (lon // ps[1])            # crop to a multiple of the patch size
        self.img_shape = (lat, lon)
        span = (num_history + num_steps) * stride
        self.index: List[tuple] = [(y, t) for y, a in enumerate(self.arrays) for t in range(num_history * stride, a.shape[0] - num_steps * stride)]
        if not self.index:
            raise ValueError(f"yearly files are shorter than one sample window of {span + 1} steps")
        self.mu = self.sd = None
        if stats_dir is not None:
            mu, sd = np.load(Path(stats_dir) / "global_means.npy"), np.load(Path(stats_dir) / "global_stds.npy")
            self.mu = torch.as_tensor(mu[:, self.channels], dtype=torch.float32, device=self.device)
            self.sd = torch.as_tensor(sd[:, self.channels], dtype=torch.float32, device=self.device)
        self.epoch = 0

    def __len__(self) -> int:
        per_rank = len(self.index) // self.world
        return per_rank // self.batch_size if self.drop_last else -(-per_rank // self.batch_size)

    def _order(self) -> np.ndarray:
        order = np.arange(len(self.index))
        if self.shuffle:
            np.random.default_rng(self.seed + self.epoch).shuffle(order)
        per_rank = len(order) // self.world
        return order[self.rank * per_rank:(self.rank + 1) * per_rank]

    def _read(self, y: int, t: int):
        a, ch, (lat, lon), s = self.arrays[y], self.channels, self.img_shape, self.stride
        take = lambda tt: np.asarray(a[tt][ch][:, :lat, :lon], dtype=np.float32)  # noqa: E731
        inv = np.stack([take(t - h * s) for h in range(self.num_history, -1, -1)]) if self.num_history else take(t)
        out = np.stack([take(t + (k + 1) * s) for k in range(self.num_steps)])
        return inv, out

    def _host_batches(self, order) -> Iterator[tuple]:
        pin = self.device.type == "cuda"
        for b in range(0, len(order), self.batch_size):
            ids = order[b:b + self.batch_size]
            if len(ids) < self.batch_size and self.drop_last:
                return
            pairs = [self._read(*self.index[i]) for i in ids]
            inv = torch.from_numpy(np.stack([p[0] for p in pairs]))
            out = torch.from_numpy(np.stack([p[1] for p in pairs]))
            yield (inv.pin_memory(), out.pin_memory()) if pin else (inv, out)

    def __iter__(self):
        order = self._order()
        self.epoch += 1
        q: queue.Queue = queue.Queue(maxsize=self.prefetch)
        stop = threading.Event()

        def producer():
            try:
                for item in self._host_batches(order):
                    if stop.is_set():
                        return
                    q.put(item)
                q.put(None)
            except BaseException as e:  # surface reader errors in the consumer
                q.put(e)

        th = threading.Thread(target=producer, daemon=True)
        th.start()
        cuda = self.device.type == "cuda"
        side = torch.cuda.Stream(self.device) if cuda else None

        def stage(item):
            if item is None or isinstance(item, BaseException):
                return item
            if not cuda:
                return [self._normalise(t) for t in item]
            with torch.cuda.stream(side):
                dev = [self._normalise(t.to(self.device, non_blocking=True)) for t in item]
                ev = torch.cuda.Event()
                ev.record(side)
            return dev, ev, item                                   # the pinned buffers stay alive until the copy is waited for

        try:
            nxt = stage(q.get())
            while nxt is not None:
                if isinstance(nxt, BaseException):
                    raise nxt
                cur, nxt = nxt, stage(q.get())                     # next batch's copy is in flight while this one is consumed
                if cuda:
                    dev, ev, _host = cur
                    torch.cuda.current_stream(self.device).wait_event(ev)
                    for t in dev:
                        t.record_stream(torch.cuda.current_stream(self.device))
                else:
                    dev = cur
                yield [{"invar": dev[0], "outvar": dev[1]}]
        finally:
            stop.set()

    def _normalise(self, t: torch.Tensor) -> torch.Tensor:
        if self.mu is None:
            return t
        shape = (1,) * (t.dim() - 3) + (-1, 1, 1)
        return (t - self.mu.reshape(shape)) / self.sd.reshape(shape)
