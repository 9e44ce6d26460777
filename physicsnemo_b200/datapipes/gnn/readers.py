"""File readers of the graph datasets, gated on what is installed.

The reference reads VTK poly-data (``.vtp`` / ``.vtk``, through ``vtk`` / ``pyvista``) and TFRecord trajectories
(through ``tensorflow``).  Where those packages are importable the readers below use them; everywhere else a sample is
an ``.npz`` file (or an in-memory dict) with the same arrays under the same names, which is also what the tests use.
"""
from __future__ import annotations

from pathlib import Path
from typing import Dict

import numpy as np


def _have(module: str) -> bool:
    import importlib.util

    return importlib.util.find_spec(module) is not None


def read_surface_sample(path) -> Dict[str, np.ndarray]:
    """``pos [N, 3]``, ``cells [C, 3]`` (triangles) and every point array of a surface sample.

    ``.npz``: the arrays as stored.  ``.vtp`` / ``.vtk`` / ``.stl``: read with ``pyvista`` (cell data is averaged to the
    points, polygons are triangulated); raises ``ImportError`` with that hint when ``pyvista`` is absent."""
    path = Path(path)
    if path.suffix == ".npz":
        with np.load(path, allow_pickle=False) as f:
            return {k: f[k] for k in f.files}
    if not _have("pyvista"):
        raise ImportError(f"reading {path.suffix} files needs `pyvista` (VTK); convert the sample to .npz with the arrays "
                          "`pos`, `cells` and one array per field, or install pyvista")
    import pyvista as pv  # noqa: WPS433 (optional dependency)

    mesh = pv.read(str(path)).triangulate().cell_data_to_point_data()
    out = {"pos": np.asarray(mesh.points, dtype=np.float32), "cells": np.asarray(mesh.faces).reshape(-1, 4)[:, 1:]}
    for name in mesh.point_data.keys():
        out[name] = np.asarray(mesh.point_data[name])
    return out


def read_tfrecord_trajectories(path, meta: dict):
    """Yield dicts of arrays from a MeshGraphNets / GNS ``.tfrecord`` file described by ``meta`` (the dataset's
    ``meta.json``).  Needs ``tensorflow``; raises ``ImportError`` otherwise (use ``.npz`` trajectories instead)."""
    if not _have("tensorflow"):
        raise ImportError("TFRecord trajectories need `tensorflow`; convert them to .npz files with the same field names")
    import tensorflow as tf  # noqa: WPS433

    def parse(proto):
        feats = {k: tf.io.VarLenFeature(tf.string) for k in meta["field_names"]}
        ex = tf.io.parse_single_example(proto, feats)
        out = {}
        for key, field in meta["features"].items():
            data = tf.io.decode_raw(ex[key].values, getattr(tf, field["dtype"]))
            out[key] = tf.reshape(data, field["shape"])
        return out

    for rec in tf.data.TFRecordDataset(str(path)).map(parse):
        yield {k: v.numpy() for k, v in rec.items()}
