"""``.npz`` reader: one file holding arrays indexed along dim 0, or a directory with one file per sample
(parity: ``physicsnemo/datapipes/readers/numpy.py``)."""
from __future__ import annotations

from pathlib import Path
from typing import Any, Optional

import numpy as np
import torch

from .._indexing import _cyclic_block_indices
from ..registry import register
from .base import Reader


@register()
class NumpyReader(Reader):
    def __init__(self, path: str | Path, *, fields: Optional[list[str]] = None,
                 default_values: Optional[dict[str, torch.Tensor]] = None, file_pattern: str = "*.npz",
                 index_key: Optional[str] = None, pin_memory: bool = False, include_index_in_metadata: bool = True,
                 coordinated_subsampling: Optional[dict[str, Any]] = None) -> None:
        super().__init__(pin_memory=pin_memory, include_index_in_metadata=include_index_in_metadata,
                         coordinated_subsampling=coordinated_subsampling)
        self.path = Path(path).expanduser().resolve()
        self._user_fields, self.default_values = fields, default_values or {}
        self.file_pattern, self.index_key = file_pattern, index_key
        if not self.path.exists():
            raise FileNotFoundError(f"Path not found: {self.path}")
        self._files: Optional[list[Path]] = None
        self._data = None
        if self.path.is_dir():
            self._mode = "directory"
            self._files = sorted(self.path.glob(file_pattern))
            if not self._files:
                raise ValueError(f"No files matching '{file_pattern}' found in {self.path}")
            self._length = len(self._files)
            with np.load(self._files[0]) as npz:
                self._available_fields = list(npz.files)
        elif self.path.suffix == ".npz":
            self._mode = "single"
            self._data = np.load(self.path)
            self._available_fields = list(self._data.files)
            key = index_key if index_key is not None else (self._available_fields[0] if self._available_fields else None)
            self._length = self._data[key].shape[0] if key is not None else 0
        else:
            raise ValueError(f"Unsupported file type: {self.path.suffix}. Expected .npz file or directory of .npz files.")

    @property
    def fields(self) -> list[str]:
        return self._user_fields if self._user_fields is not None else self._available_fields

    def _read(self, npz, row: Optional[int], where: str, generator) -> dict[str, torch.Tensor]:
        missing = set(self.fields) - set(self.default_values) - set(npz.files)
        if missing:
            raise KeyError(f"Required fields {missing} not found in {where}. Available: {list(npz.files)}")
        cfg = self._coordinated_subsampling_config
        pick, targets = None, set()
        if cfg is not None:
            targets = set(cfg["target_keys"])
            for f in targets:
                if f in npz.files:
                    pick = _cyclic_block_indices(npz[f].shape[0], cfg["n_points"], generator=generator).numpy()
                    break
        out = {}
        for f in self.fields:
            if f in npz.files:
                arr = npz[f]
                if row is not None:
                    arr = arr[row]
                if pick is not None and f in targets:
                    arr = arr[pick]
                out[f] = torch.from_numpy(np.array(arr))
            else:
                out[f] = self.default_values[f].clone()
        return out

    def _load_sample(self, index: int) -> dict[str, torch.Tensor]:
        g = self._index_generator(index)
        if self._mode == "directory":
            with np.load(self._files[index]) as npz:
                return self._read(npz, None, str(self._files[index]), g)
        return self._read(self._data, index, str(self.path), g)

    def __len__(self) -> int:
        return self._length

    def _get_field_names(self) -> list[str]:
        return self.fields

    def _get_sample_metadata(self, index: int) -> dict[str, Any]:
        p = self._files[index] if self._mode == "directory" else self.path
        return {"source_file": str(p), "source_filename": p.name}

    @property
    def _supports_coordinated_subsampling(self) -> bool:
        return self._mode == "directory"

    def close(self) -> None:
        if self._data is not None and hasattr(self._data, "close"):
            self._data.close()
        self._data = None

    def __repr__(self) -> str:
        cfg = self._coordinated_subsampling_config
        sub = f", subsampling={cfg['n_points']} points" if cfg else ""
        return f"NumpyReader(path={self.path}, mode={self._mode}, len={len(self)}, fields={self.fields}{sub})"
