"""HDF5 reader (parity: ``physicsnemo/datapipes/readers/hdf5.py``): one file whose datasets are indexed along
dim 0, or a directory of per-sample files; ``h5py`` is imported on first use."""
from __future__ import annotations

from pathlib import Path
from typing import Any, Optional

import numpy as np
import torch

from .._indexing import _cyclic_block_indices
from ..registry import register
from .base import Reader


def _h5py():
    try:
        import h5py
    except ImportError as e:  # pragma: no cover
        raise ImportError("HDF5Reader requires h5py (`pip install h5py`).") from e
    return h5py


@register()
class HDF5Reader(Reader):
    def __init__(self, path: str | Path, *, fields: Optional[list[str]] = None,
                 default_values: Optional[dict[str, torch.Tensor]] = None, file_pattern: str = "*.h5",
                 index_key: Optional[str] = None, pin_memory: bool = False, include_index_in_metadata: bool = True,
                 coordinated_subsampling: Optional[dict[str, Any]] = None) -> None:
        super().__init__(pin_memory=pin_memory, include_index_in_metadata=include_index_in_metadata,
                         coordinated_subsampling=coordinated_subsampling)
        h5py = _h5py()
        self.path = Path(path).expanduser().resolve()
        if not self.path.exists():
            raise FileNotFoundError(f"Path not found: {self.path}")
        self._user_fields, self.default_values = fields, default_values or {}
        self._file = None
        if self.path.is_dir():
            self._mode = "directory"
            self._files = sorted(list(self.path.glob(file_pattern)) + list(self.path.glob("*.hdf5")))
            if not self._files:
                raise ValueError(f"No HDF5 files found in {self.path}")
            with h5py.File(self._files[0], "r") as f:
                self._available = [k for k in f.keys() if hasattr(f[k], "shape")]
            self._length = len(self._files)
        else:
            self._mode = "single"
            self._file = h5py.File(self.path, "r")
            self._available = [k for k in self._file.keys() if hasattr(self._file[k], "shape")]
            key = index_key or (self._available[0] if self._available else None)
            self._length = self._file[key].shape[0] if key else 0

    @property
    def fields(self) -> list[str]:
        return self._user_fields if self._user_fields is not None else self._available

    def _read(self, f, row, generator):
        cfg = self._coordinated_subsampling_config
        pick, targets = None, set()
        if cfg is not None:
            targets = set(cfg["target_keys"])
            for k in targets:
                if k in f:
                    n = f[k].shape[0] if row is None else f[k].shape[1]
                    pick = _cyclic_block_indices(n, cfg["n_points"], generator=generator).numpy()
                    break
        out = {}
        for k in self.fields:
            if k in f:
                ds = f[k]
                if pick is not None and k in targets:
                    runs = np.split(pick, np.where(np.diff(pick) != 1)[0] + 1)   # ≤ 2 contiguous hyperslabs
                    parts = [ds[r[0]:r[-1] + 1] if row is None else ds[row, r[0]:r[-1] + 1] for r in runs]
                    arr = np.concatenate(parts, axis=0)
                else:
                    arr = ds[()] if row is None else ds[row]
                out[k] = torch.from_numpy(np.asarray(arr))
            elif k in self.default_values:
                out[k] = self.default_values[k].clone()
            else:
                raise KeyError(f"Required field '{k}' not found. Available: {list(f.keys())}")
        return out

    def _load_sample(self, index: int) -> dict[str, torch.Tensor]:
        g = self._index_generator(index)
        if self._mode == "directory":
            with _h5py().File(self._files[index], "r") as f:
                return self._read(f, None, g)
        return self._read(self._file, index, g)

    def __len__(self) -> int:
        return self._length

    def _get_field_names(self) -> list[str]:
        return self.fields

    def _get_sample_metadata(self, index: int) -> dict[str, Any]:
        p = self._files[index] if self._mode == "directory" else self.path
        return {"source_file": str(p), "source_filename": p.name}

    @property
    def _supports_coordinated_subsampling(self) -> bool:
        return True

    def close(self) -> None:
        if self._file is not None:
            self._file.close()
            self._file = None
