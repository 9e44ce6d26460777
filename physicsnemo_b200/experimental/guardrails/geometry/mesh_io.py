"""Feature extraction over a directory of STL files.

Parity: ``physicsnemo/experimental/guardrails/geometry/mesh_io.py`` (``load_features_from_dir``).  Files
are parsed by the package's own STL reader (ASCII and binary), so no visualisation package is needed;
unreadable or degenerate geometries are skipped and reported, and it is an error when none is left.
"""
from __future__ import annotations

import logging
import multiprocessing as mp
from pathlib import Path
from typing import Optional

import numpy as np

logger = logging.getLogger(__name__)


def _process_stl(path_str: str):
    """``(file name, feature vector or None, error text or None)``; runs in a worker process."""
    from ....mesh.io import read_stl
    from .feature_extraction import extract_features, validate_mesh

    path = Path(path_str)
    try:
        mesh = read_stl(path)
        if mesh.n_points == 0:
            raise ValueError("Mesh has no points")
        if mesh.n_cells == 0:
            raise ValueError(f"Mesh has no cells (n_points={mesh.n_points})")
        validate_mesh(mesh)
        return path.name, extract_features(mesh, return_tensor=False, skip_validation=True), None
    except Exception as exc:  # noqa: BLE001  (a bad file must not stop the scan)
        return path.name, None, f"{path.name}: {type(exc).__name__}: {exc}"


def load_features_from_dir(stl_dir, n_workers: Optional[int] = None):
    """Features of every ``*.stl`` in ``stl_dir`` (sorted by name): ``(list of feature vectors, list of file names)``.

    ``n_workers`` processes (default: all cores but one) parse and featurise in parallel; ``n_workers=0``
    or ``1`` stays in the calling process.
    """
    paths = sorted(p.as_posix() for p in Path(stl_dir).glob("*.stl"))
    if n_workers is None:
        n_workers = max(1, mp.cpu_count() - 1)
    if n_workers <= 1 or len(paths) <= 1:
        results = [_process_stl(p) for p in paths]
    else:
        with mp.get_context("spawn").Pool(processes=min(n_workers, len(paths))) as pool:
            results = pool.map(_process_stl, paths)
    feats = [np.asarray(f) for _, f, err in results if err is None]
    names = [n for n, _, err in results if err is None]
    errors = [err for _, _, err in results if err is not None]
    if not feats:
        message = f"No valid STL files found in {stl_dir}"
        if errors:
            message += f"\n{len(errors)} files failed to load. First error: {errors[0]}"
        raise RuntimeError(message)
    if errors:
        logger.warning("[geometry guardrail] skipped %d invalid geometries: %s%s", len(errors), "; ".join(errors[:5]),
                       f" ... and {len(errors) - 5} more" if len(errors) > 5 else "")
    return feats, names
