"""Map-style dataset of ``Mesh`` samples stored one per file, with a chain of mesh transforms.

Parity: ``physicsnemo/datapipes/mesh_dataset.py`` (``MeshDataset``) and ``readers/mesh.py`` (``MeshReader``): samples are
read lazily, optionally sub-sampled at read time, pushed through ``transforms`` (deterministic and random; random ones are
re-seeded per epoch through ``set_epoch``) and moved to ``device``.  The reference reads its meshes from Zarr / tensorstore /
PyVista files; those libraries are not available here, so ``MeshReader`` reads the ``.npz`` layout written by
``save_mesh_npz``: ``points``, ``cells`` and arrays named ``point_data/<name>``, ``cell_data/<name>``, ``global_data/<name>``.
"""
from __future__ import annotations

from pathlib import Path
from typing import Callable, Sequence

import numpy as np
import torch

from ..mesh import Mesh


def save_mesh_npz(mesh: Mesh, path: str | Path) -> None:
    arrays = {"points": mesh.points.cpu().numpy(), "cells": mesh.cells.cpu().numpy()}
    for store in ("point_data", "cell_data", "global_data"):
        for k, v in getattr(mesh, store).items():
            arrays[f"{store}/{k}"] = v.cpu().numpy()
    np.savez(str(path), **arrays)


class MeshReader:
    """Reads ``.npz`` meshes from a directory (sorted) or an explicit list of files."""

    def __init__(self, path: str | Path | Sequence[str | Path], pattern: str = "*.npz", subsample_n_cells: int | None = None, seed: int = 0):
        if isinstance(path, (str, Path)):
            p = Path(path)
            self.files = sorted(p.glob(pattern)) if p.is_dir() else [p]
        else:
            self.files = [Path(f) for f in path]
        if not self.files:
            raise FileNotFoundError(f"no mesh files found under {path}")
        self.subsample_n_cells, self.seed = subsample_n_cells, seed

    def __len__(self) -> int:
        return len(self.files)

    def __getitem__(self, i: int) -> Mesh:
        with np.load(self.files[i]) as z:
            cells = torch.from_numpy(z["cells"]).long()
            keep = None
            if self.subsample_n_cells is not None and cells.shape[0] > self.subsample_n_cells:
                g = torch.Generator().manual_seed(self.seed + i)
                keep = torch.randperm(cells.shape[0], generator=g)[:self.subsample_n_cells].sort().values
                cells = cells[keep]
            stores = {"point_data": {}, "cell_data": {}, "global_data": {}}
            for key in z.files:
                if "/" in key:
                    store, name = key.split("/", 1)
                    v = torch.from_numpy(z[key])
                    stores[store][name] = v[keep] if (store == "cell_data" and keep is not None) else v
            return Mesh(torch.from_numpy(z["points"]), cells, stores["point_data"], stores["cell_data"], stores["global_data"])


class MeshDataset(torch.utils.data.Dataset):
    def __init__(self, reader, transforms: Sequence[Callable] | None = None, device: str | torch.device | None = None, seed: int = 0):
        self.reader, self.transforms, self.seed = reader, list(transforms or []), seed
        self.device = torch.device(device) if device is not None else None
        for i, t in enumerate(self.transforms):
            if getattr(t, "stochastic", False):
                t.set_generator(torch.Generator().manual_seed(seed + 1000 * (i + 1)))
        self.set_epoch(0)

    def set_epoch(self, epoch: int) -> None:
        for t in self.transforms:
            if hasattr(t, "set_epoch"):
                t.set_epoch(epoch)

    def __len__(self) -> int:
        return len(self.reader)

    def __getitem__(self, i: int):
        sample = self.reader[i]
        if self.device is not None:
            sample = sample.to(self.device)
        for t in self.transforms:
            sample = t(sample)
        return sample
