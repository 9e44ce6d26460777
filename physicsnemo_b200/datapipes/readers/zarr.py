"""Zarr readers (parity: ``physicsnemo/datapipes/readers/zarr.py`` and ``tensorstore_zarr.py``): a directory of
``*.zarr`` groups, one per sample.  ``TensorStoreZarrReader`` reads through tensorstore when it is installed and
otherwise falls back to the zarr package."""
from __future__ import annotations

from pathlib import Path
from typing import Any, Optional

import numpy as np
import torch

from .._indexing import _cyclic_block_indices
from ..registry import register
from .base import Reader


@register()
class ZarrReader(Reader):
    def __init__(self, path: str | Path, *, fields: Optional[list[str]] = None,
                 default_values: Optional[dict[str, torch.Tensor]] = None, group_pattern: str = "*.zarr",
                 pin_memory: bool = False, include_index_in_metadata: bool = True,
                 coordinated_subsampling: Optional[dict[str, Any]] = None) -> None:
        super().__init__(pin_memory=pin_memory, include_index_in_metadata=include_index_in_metadata,
                         coordinated_subsampling=coordinated_subsampling)
        try:
            import zarr  # noqa: F401
        except ImportError as e:  # pragma: no cover
            raise ImportError(f"{type(self).__name__} requires the zarr package (`pip install zarr`).") from e
        self.path = Path(path).expanduser().resolve()
        if not self.path.exists():
            raise FileNotFoundError(f"Path not found: {self.path}")
        self._groups = [self.path] if self.path.suffix == ".zarr" else sorted(self.path.glob(group_pattern))
        if not self._groups:
            raise ValueError(f"No zarr groups matching '{group_pattern}' found in {self.path}")
        self._user_fields, self.default_values = fields, default_values or {}
        self._available = list(self._open(self._groups[0]).array_keys())

    def _open(self, p):
        import zarr

        return zarr.open_group(str(p), mode="r")

    @property
    def fields(self) -> list[str]:
        return self._user_fields if self._user_fields is not None else self._available

    def _load_sample(self, index: int) -> dict[str, torch.Tensor]:
        g = self._open(self._groups[index])
        cfg = self._coordinated_subsampling_config
        pick, targets = None, set()
        if cfg is not None:
            targets = set(cfg["target_keys"])
            for k in targets:
                if k in g:
                    pick = _cyclic_block_indices(g[k].shape[0], cfg["n_points"], generator=self._index_generator(index)).numpy()
                    break
        out = {}
        for k in self.fields:
            if k in g:
                arr = g[k]
                if pick is not None and k in targets:
                    runs = np.split(pick, np.where(np.diff(pick) != 1)[0] + 1)
                    data = np.concatenate([arr[r[0]:r[-1] + 1] for r in runs], axis=0)
                else:
                    data = arr[...]
                out[k] = torch.from_numpy(np.asarray(data))
            elif k in self.default_values:
                out[k] = self.default_values[k].clone()
            else:
                raise KeyError(f"Required field '{k}' not found in {self._groups[index]}")
        return out

    def __len__(self) -> int:
        return len(self._groups)

    def _get_field_names(self) -> list[str]:
        return self.fields

    def _get_sample_metadata(self, index: int) -> dict[str, Any]:
        return {"source_file": str(self._groups[index]), "source_filename": self._groups[index].name}

    @property
    def _supports_coordinated_subsampling(self) -> bool:
        return True


@register()
class TensorStoreZarrReader(ZarrReader):
    """Same layout as ``ZarrReader``; reads are issued concurrently through tensorstore futures when available."""

    def _load_sample(self, index: int) -> dict[str, torch.Tensor]:
        try:
            import tensorstore as ts
        except ImportError:
            return super()._load_sample(index)
        root = self._groups[index]
        futures = {}
        for k in self.fields:
            if (root / k).exists():
                spec = {"driver": "zarr", "kvstore": {"driver": "file", "path": str(root / k)}}
                futures[k] = ts.open(spec, read=True).result().read()
        out = {k: torch.from_numpy(np.asarray(f.result())) for k, f in futures.items()}
        for k in self.fields:
            if k not in out:
                if k not in self.default_values:
                    raise KeyError(f"Required field '{k}' not found in {root}")
                out[k] = self.default_values[k].clone()
        return out
