"""File-backed dataset of CAE samples (surface / volume fields, geometry) with read-ahead and side-stream uploads.

Counterpart of ``physicsnemo/datapipes/cae/cae_dataset.py`` (``BackendReader`` :59 and the npy / npz / zarr readers
:198-:853, ``CAEDataset`` :863, ``compute_mean_std_min_max`` :1261).

One sample per file (or per directory).  Supported layouts, detected from the data directory:

* ``*.npy`` – a pickled dict of arrays;
* ``*.npz`` – an archive of arrays;
* directories of ``<key>.npy`` files – one memory-mapped array per key: a volume sub-sample touches only the pages of
  the sampled block, so samples larger than host memory stream straight from disk (the role chunked Zarr stores play
  in the reference);
* ``*.zarr`` directories – read through ``zarr`` when it is installed.

Sharded reads: with a 1-D device mesh every rank reads only its slice of the leading axis of each array (large arrays)
and gets ``ShardTensor`` s back.

Pipeline: ``preload_depth`` worker threads read upcoming files into (optionally pinned) host memory and enqueue the
host-to-device copies on a dedicated stream; the consumer stream waits on the copy's event only when the sample is
handed out, so file reads and PCIe / C2C transfers overlap the training step.
"""

from __future__ import annotations

import pathlib
import time
from abc import ABC, abstractmethod
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

__all__ = ["BackendReader", "NpyFileReader", "NpzFileReader", "NpyDirectoryReader", "ZarrFileReader", "CAEDataset",
           "compute_mean_std_min_max"]

_SHARD_MIN_ROWS = 1024          # arrays with fewer rows are replicated instead of sharded


def _split_sizes(n: int, parts: int) -> List[int]:
    base, extra = divmod(n, parts)
    return [base + (1 if r < extra else 0) for r in range(parts)]


def _cyclic_block(total: int, count: int, start: Optional[int]) -> np.ndarray:
    """``count`` consecutive indices modulo ``total`` beginning at ``start`` (a contiguous read with one wrap at most)."""
    if start is None:
        return np.arange(count)
    return (start + np.arange(count)) % total


class BackendReader(ABC):
    """Reads one sample into a dict of CPU tensors; ``keys_to_read_if_available`` supplies defaults for optional keys."""

    def __init__(self, keys_to_read: Optional[List[str]], keys_to_read_if_available: Optional[Dict[str, torch.Tensor]]):
        self.keys_to_read = list(keys_to_read or [])
        self.keys_to_read_if_available = dict(keys_to_read_if_available or {})
        self.volume_sampling_size: Optional[int] = None
        self.is_volumetric = any("volume" in k for k in self.keys_to_read)

    @abstractmethod
    def read_file(self, filename: pathlib.Path) -> Dict[str, torch.Tensor]:
        ...

    def read_file_attributes(self, filename: pathlib.Path) -> Dict[str, torch.Tensor]:
        return {}

    def read_file_sharded(self, filename: pathlib.Path, device_mesh) -> Tuple[Dict[str, torch.Tensor], Dict[str, tuple]]:
        raise NotImplementedError(f"{type(self).__name__} cannot read a slice of a file; use the npy-directory or zarr layout")

    def fill_optional_keys(self, data: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        for key, default in self.keys_to_read_if_available.items():
            data.setdefault(key, default)
        return data

    def _check_keys(self, found, filename) -> None:
        missing = set(self.keys_to_read) - set(found)
        if missing:
            raise ValueError(f"Keys {missing} not found in file {filename}")

    def _get_slice_boundaries(self, array_shape: tuple, this_rank: int, n_splits: int, split_dim: int = 0):
        sizes = _split_sizes(array_shape[split_dim], n_splits)
        start = sum(sizes[:this_rank])
        chunks = tuple(array_shape[:split_dim] + (s,) + array_shape[split_dim + 1:] for s in sizes)
        return start, start + sizes[this_rank], chunks

    def set_volume_sampling_size(self, volume_sampling_size: int) -> None:
        self.volume_sampling_size = volume_sampling_size

    def select_random_sections_from_slice(self, slice_start: int, slice_stop: int, n_points: int) -> np.ndarray:
        total = slice_stop - slice_start
        if total < n_points:
            raise ValueError(f"Slice size {total} is less than the number of points {n_points}")
        start = None if n_points in (0, total) else int(np.random.randint(total))
        return _cyclic_block(total, n_points, start) + slice_start

    def _volume_rows(self, n_rows: int):
        if self.volume_sampling_size is None:
            return slice(0, n_rows)
        return self.select_random_sections_from_slice(0, n_rows, self.volume_sampling_size)


class NpyFileReader(BackendReader):
    """``.npy`` file holding a pickled dict of arrays (whole-file reads only)."""

    def read_file(self, filename):
        data = np.load(filename, allow_pickle=True).item()
        self._check_keys(data.keys(), filename)
        return self.fill_optional_keys({k: torch.from_numpy(np.asarray(data[k])) for k in self.keys_to_read})

    def set_volume_sampling_size(self, volume_sampling_size: int) -> None:
        raise NotImplementedError("volume sampling directly from disk is not supported for npy files.")


class NpzFileReader(BackendReader):
    """``.npz`` archive; a volume sub-sample is cut after the member is decompressed."""

    def read_file(self, filename):
        with np.load(filename) as archive:
            self._check_keys(archive.keys(), filename)
            rows = None
            out = {}
            for k in self.keys_to_read:
                arr = archive[k]
                if "volume" in k:
                    rows = self._volume_rows(arr.shape[0]) if rows is None else rows
                    arr = arr[rows]
                out[k] = torch.from_numpy(np.ascontiguousarray(arr))
        return self.fill_optional_keys(out)


class NpyDirectoryReader(BackendReader):
    """A directory with one ``<key>.npy`` per array, memory-mapped: partial and sharded reads touch only what they need."""

    @staticmethod
    def _open(filename: pathlib.Path, key: str):
        return np.load(filename / f"{key}.npy", mmap_mode="r")

    def read_file(self, filename):
        self._check_keys({p.stem for p in filename.glob("*.npy")}, filename)
        rows, out = None, {}
        for k in self.keys_to_read:
            arr = self._open(filename, k)
            if "volume" in k and arr.ndim:
                rows = self._volume_rows(arr.shape[0]) if rows is None else rows
                arr = arr[rows]
            out[k] = torch.from_numpy(np.array(arr))                   # copy out of the mapping
        return self.fill_optional_keys(out)

    def read_file_sharded(self, filename, device_mesh):
        import torch.distributed as dist
        from torch.distributed.tensor.placement_types import Replicate, Shard

        rank, world = device_mesh.get_local_rank(), dist.get_world_size(group=device_mesh.get_group())
        self._check_keys({p.stem for p in filename.glob("*.npy")}, filename)
        data, specs = {}, {}
        for k in self.keys_to_read:
            arr = self._open(filename, k)
            if arr.ndim == 0 or arr.shape[0] < max(_SHARD_MIN_ROWS, world):
                data[k], specs[k] = torch.from_numpy(np.array(arr)), ([Replicate()], None)
                continue
            lo, hi, chunks = self._get_slice_boundaries(tuple(arr.shape), rank, world)
            data[k] = torch.from_numpy(np.array(arr[lo:hi]))
            specs[k] = ([Shard(0)], {0: chunks})
        return self.fill_optional_keys(data), specs


class ZarrFileReader(BackendReader):
    """``.zarr`` group (needs the ``zarr`` package); attributes can serve as keys."""

    def __init__(self, keys_to_read, keys_to_read_if_available):
        super().__init__(keys_to_read, keys_to_read_if_available)
        try:
            import zarr  # noqa: F401
        except ImportError as e:                                      # pragma: no cover - depends on the environment
            raise ImportError("reading .zarr samples needs the 'zarr' package; convert the data to the npy-directory layout "
                              "or install zarr") from e

    def read_file_attributes(self, filename):
        import zarr

        return dict(zarr.open_group(filename, mode="r").attrs)

    def read_file(self, filename):                                     # pragma: no cover - needs zarr
        import zarr

        group, attrs = zarr.open_group(filename, mode="r"), self.read_file_attributes(filename)
        self._check_keys(set(group.keys()) | set(attrs), filename)
        rows, out = None, {}
        for k in self.keys_to_read:
            if k in attrs:
                out[k] = torch.tensor(attrs[k])
            elif group[k].shape == ():
                out[k] = torch.from_numpy(np.array(group[k])).to(torch.float32)
            elif "volume" in k:
                rows = self._volume_rows(group[k].shape[0]) if rows is None else rows
                out[k] = torch.from_numpy(group[k].oindex[rows] if not isinstance(rows, slice) else group[k][rows])
            else:
                out[k] = torch.from_numpy(group[k][:])
        return self.fill_optional_keys(out)


def _pick_reader(data_dir: pathlib.Path, keys, optional) -> Tuple[BackendReader, List[pathlib.Path]]:
    files = sorted(data_dir.iterdir())
    if not files:
        raise ValueError(f"No samples found in {data_dir}")
    if all(f.suffix == ".npy" and f.is_file() for f in files):
        return NpyFileReader(keys, optional), files
    if all(f.suffix == ".npz" for f in files):
        return NpzFileReader(keys, optional), files
    if all(f.suffix == ".zarr" and f.is_dir() for f in files):
        return ZarrFileReader(keys, optional), files
    if all(f.is_dir() and any(f.glob("*.npy")) for f in files):
        return NpyDirectoryReader(keys, optional), files
    raise ValueError(f"Unsupported file type: {files[0]}")


class CAEDataset:
    """Indexable / iterable dataset over the samples of ``data_dir`` with threaded read-ahead.

    ``dataset[i]`` returns a dict of tensors on ``output_device`` (``ShardTensor`` s under a device mesh).  Iterating
    keeps ``preload_depth`` samples in flight; ``set_indices`` restricts / reorders the epoch.
    """

    def __init__(self, data_dir, keys_to_read: Optional[List[str]], keys_to_read_if_available: Optional[Dict[str, torch.Tensor]],
                 output_device: torch.device, preload_depth: int = 2, pin_memory: bool = False, device_mesh=None, placements=None,
                 consumer_stream: Optional["torch.cuda.Stream"] = None):
        data_dir = pathlib.Path(data_dir)
        if not data_dir.exists():
            raise FileNotFoundError(f"Data directory {data_dir} does not exist")
        if not data_dir.is_dir():
            raise NotADirectoryError(f"Data directory {data_dir} is not a directory")
        self.output_device = torch.device(output_device)
        optional = {k: v.to(self.output_device) for k, v in (keys_to_read_if_available or {}).items()}
        self.file_reader, self._filenames = _pick_reader(data_dir, keys_to_read, optional)
        self.pin_memory, self.preload_depth = pin_memory, preload_depth
        self.device_mesh, self.placements = device_mesh, placements
        if device_mesh is not None and device_mesh.ndim != 1:
            raise ValueError("Device mesh must be one dimensional")
        on_gpu = self.output_device.type == "cuda"
        self._copy_stream = torch.cuda.Stream(self.output_device) if on_gpu else None
        self.consumer_stream = consumer_stream if consumer_stream is not None or not on_gpu else torch.cuda.current_stream(self.output_device)
        self._inflight: Dict[int, "object"] = {}
        self._copied: Dict[int, "torch.cuda.Event"] = {}
        self._specs: Dict[int, dict] = {}
        self.preload_executor = ThreadPoolExecutor(max_workers=max(1, preload_depth))
        self.i = 0

    # ---- index space -------------------------------------------------------------------------------------------
    def set_indices(self, indices: List[int]) -> None:
        self.indices = list(indices)

    def idx_to_index(self, idx: int) -> int:
        return self.indices[idx] if hasattr(self, "indices") else idx

    def _epoch_length(self) -> int:
        return len(self.indices) if hasattr(self, "indices") else len(self._filenames)

    def __len__(self) -> int:
        return len(self._filenames)

    # ---- loading -----------------------------------------------------------------------------------------------
    def _read(self, idx: int) -> Dict[str, torch.Tensor]:
        if self.device_mesh is None:
            data = self.file_reader.read_file(self._filenames[idx])
        else:
            data, self._specs[idx] = self.file_reader.read_file_sharded(self._filenames[idx], self.device_mesh)
        if "stl_faces" in data:
            data["stl_faces"] = data["stl_faces"].to(torch.int32)
        return data

    def _upload(self, data: Dict[str, torch.Tensor], idx: int) -> Dict[str, torch.Tensor]:
        if self._copy_stream is None:
            return data
        out = {}
        with torch.cuda.stream(self._copy_stream):
            for k, v in data.items():
                if v.device == self.output_device:
                    out[k] = v
                    continue
                out[k] = (v.pin_memory() if self.pin_memory else v).to(self.output_device, non_blocking=True)
                out[k].record_stream(self.consumer_stream)
            done = torch.cuda.Event()
            done.record(self._copy_stream)
        self._copied[idx] = done
        return out

    def preload(self, idx: int) -> None:
        """Start reading (and uploading) sample ``idx`` in the background."""
        if idx not in self._inflight:
            self._inflight[idx] = self.preload_executor.submit(lambda: self._upload(self._read(idx), idx))

    def get_preloaded(self, idx: int) -> Optional[Dict[str, torch.Tensor]]:
        fut = self._inflight.pop(idx, None)
        return None if fut is None else fut.result()

    def __getitem__(self, idx: int):
        if idx >= len(self._filenames):
            raise IndexError(f"Index {idx} out of range for dataset of size {len(self._filenames)}")
        data = self.get_preloaded(idx)
        if data is None:
            data = self._upload(self._read(idx), idx)
        done = self._copied.pop(idx, None)
        if done is not None:
            self.consumer_stream.wait_event(done)
        if self.device_mesh is not None:
            from ...domain_parallel import ShardTensor

            spec = self._specs.pop(idx)
            data = {k: (ShardTensor.from_local(local_tensor=v, device_mesh=self.device_mesh, placements=spec[k][0], sharding_shapes=spec[k][1])
                        if k in spec else v) for k, v in data.items()}
        return data

    def __iter__(self):
        self.i = 0
        for ahead in range(min(self.preload_depth, self._epoch_length())):
            self.preload(self.idx_to_index(ahead))
        return self

    def __next__(self):
        n = self._epoch_length()
        if self.i >= n:
            self.i = 0
            raise StopIteration
        for ahead in range(1, self.preload_depth + 1):
            if self.i + ahead < n:
                self.preload(self.idx_to_index(self.i + ahead))
        data = self[self.idx_to_index(self.i)]
        self.i += 1
        return data

    def set_volume_sampling_size(self, volume_sampling_size: int) -> None:
        self.file_reader.set_volume_sampling_size(volume_sampling_size)

    def close(self) -> None:
        ex, self.preload_executor = getattr(self, "preload_executor", None), None
        if ex is not None:
            ex.shutdown(wait=True)

    def __del__(self):
        self.close()


def compute_mean_std_min_max(dataset: CAEDataset, field_keys: List[str], max_samples: int = 20, verbose: bool = False):
    """Per-channel mean / std (Chan's parallel update in fp64) and min / max without 9-sigma outliers over up to
    ``max_samples`` randomly chosen samples.  Returns four dicts keyed by field."""
    order = np.random.permutation(len(dataset))[:max_samples]
    n: Dict[str, int] = {k: 0 for k in field_keys}
    mean: Dict[str, torch.Tensor] = {}
    m2: Dict[str, torch.Tensor] = {}
    t0 = time.perf_counter()
    for j in order:
        data = dataset[int(j)]
        for k in field_keys:
            x = data[k].double()
            bn, bmean = x.shape[0], x.mean(0)
            bm2 = ((x - bmean) ** 2).sum(0)
            if k not in mean:
                mean[k], m2[k] = torch.zeros_like(bmean), torch.zeros_like(bmean)
            delta, tot = bmean - mean[k], n[k] + bn
            mean[k] = mean[k] + delta * (bn / tot)
            m2[k] = m2[k] + bm2 + delta ** 2 * (n[k] * bn / tot)
            n[k] = tot
    std = {k: torch.sqrt(m2[k] / max(n[k] - 1, 1)) for k in field_keys}
    lo = {k: torch.full_like(mean[k], float("inf"), dtype=torch.float32) for k in field_keys}
    hi = {k: torch.full_like(mean[k], float("-inf"), dtype=torch.float32) for k in field_keys}
    for j in order:
        data = dataset[int(j)]
        for k in field_keys:
            x = data[k].float()
            keep = (x >= (mean[k] - 9 * std[k]).float()) & (x <= (mean[k] + 9 * std[k]).float())
            lo[k] = torch.minimum(lo[k], torch.where(keep, x, torch.full_like(x, float("inf"))).amin(0))
            hi[k] = torch.maximum(hi[k], torch.where(keep, x, torch.full_like(x, float("-inf"))).amax(0))
    if verbose:
        print(f"statistics over {len(order)} samples in {time.perf_counter() - t0:.2f} s")
    return mean, std, lo, hi
