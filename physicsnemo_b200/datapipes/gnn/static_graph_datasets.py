"""Steady-state surrogate datasets on surface / planar meshes: Ahmed body, DrivAerNet, Stokes flow.

Parity: ``physicsnemo/datapipes/gnn/{ahmed_body_dataset,drivaernet_dataset,stokes_dataset}.py``.  One sample is one
graph: nodes are mesh vertices, edges the (bidirectional) mesh edges with features (relative displacement, length),
node inputs are the concatenation of ``invar_keys`` (position, per-case scalars broadcast to all nodes, normals,
boundary markers), node targets the concatenation of ``outvar_keys`` (pressure, wall shear stress, velocity).
Statistics come from the training split and are stored next to the data (``node_stats.json`` / ``edge_stats.json``) so
that validation / test use the same normalisation; ``denormalize`` inverts it.  The reference's in-memory
pre-processing (all graphs built at construction, statistics by a running pass) is kept; file formats follow
``gnn/readers.py``.
"""
from __future__ import annotations

from pathlib import Path
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np
import torch
from torch.utils.data import Dataset

from ...nn.module.gnn_layers.graph_types import Graph
from .readers import read_surface_sample
from .utils import cells_to_edges, edge_features, load_json, save_json

_SPLITS = ("train", "validation", "test")


def _as_2d(a) -> torch.Tensor:
    t = torch.as_tensor(np.asarray(a), dtype=torch.float32)
    return t.reshape(t.shape[0], -1) if t.ndim else t.reshape(1, 1)


class StaticMeshGraphDataset(Dataset):
    """Shared machinery; subclasses set the default keys and how a raw sample becomes node arrays."""

    default_invar: Tuple[str, ...] = ("pos",)
    default_outvar: Tuple[str, ...] = ()
    default_normalize: Tuple[str, ...] = ()
    bounds: Optional[Tuple[float, float]] = None         # min-max normalisation to these bounds; None: z-score

    def __init__(self, data_dir=None, split: str = "train", num_samples: int = 10, invar_keys: Optional[Iterable[str]] = None,
                 outvar_keys: Optional[Iterable[str]] = None, normalize_keys: Optional[Iterable[str]] = None,
                 name: str = "dataset", samples: Optional[Sequence[dict]] = None, stats_dir=None):
        if split not in _SPLITS:
            raise ValueError(f"split must be one of {_SPLITS}, got {split!r}")
        self.name, self.split = name, split
        self.input_keys = list(invar_keys if invar_keys is not None else self.default_invar)
        self.output_keys = list(outvar_keys if outvar_keys is not None else self.default_outvar)
        self.normalize_keys = list(normalize_keys if normalize_keys is not None else self.default_normalize)
        raw = list(samples) if samples is not None else self._read_dir(Path(data_dir) / split, num_samples)
        if not raw:
            raise IOError("no samples found")
        self.stats_dir = Path(stats_dir) if stats_dir is not None else (Path(data_dir) if data_dir is not None else None)
        self.graphs: List[Graph] = []
        self.case_ids: List[str] = []
        self._raw_nodes: List[Dict[str, torch.Tensor]] = []
        for i, s in enumerate(raw[:num_samples]):
            nodes = self.node_arrays(s)
            pos = nodes["pos"]
            ei = self.edges_of(s, pos)
            self._raw_nodes.append(nodes)
            self.case_ids.append(str(s.get("case_id", i)))
            self.graphs.append(Graph(ei, num_nodes=pos.shape[0], pos=pos, edge_attr=edge_features(pos, ei)))
        self._fit_or_load_stats()
        self._finalise()

    # ------------------------------------------------------------------ hooks
    def node_arrays(self, sample: dict) -> Dict[str, torch.Tensor]:
        """``{key: [N, c] float tensor}`` for every key this dataset may use, including ``pos``."""
        pos = _as_2d(sample["pos"])
        out = {"pos": pos}
        for k, v in sample.items():
            if k in ("pos", "cells", "edges", "case_id"):
                continue
            arr = np.asarray(v)
            if arr.ndim == 0 or arr.size == 1:                      # per-case scalar: one column, same value at all nodes
                out[k] = torch.full((pos.shape[0], 1), float(arr.reshape(-1)[0]))
            elif arr.shape[0] == pos.shape[0]:
                out[k] = _as_2d(arr)
        return out

    def edges_of(self, sample: dict, pos: torch.Tensor) -> torch.Tensor:
        if "edges" in sample:
            e = torch.as_tensor(np.asarray(sample["edges"])).long().reshape(-1, 2)
            e = torch.unique(e.sort(dim=1).values, dim=0)
            return torch.cat([e, e.flip(1)]).t().contiguous()
        return cells_to_edges(torch.as_tensor(np.asarray(sample["cells"])).long())

    # ------------------------------------------------------------- statistics
    def _read_dir(self, folder: Path, num_samples: int) -> List[dict]:
        files = sorted(p for p in folder.iterdir() if p.suffix in (".npz", ".vtp", ".vtk"))[:num_samples]
        out = []
        for p in files:
            s = dict(read_surface_sample(p))
            s.setdefault("case_id", p.stem)
            info = p.with_name(p.stem + "_info.txt")
            if info.exists():
                s.update(self.read_info_file(info))
            out.append(s)
        return out

    @staticmethod
    def read_info_file(path) -> Dict[str, float]:
        """``name : value`` lines of a case description (Ahmed body); names are lower-cased with spaces as underscores."""
        out = {}
        for line in Path(path).read_text().splitlines():
            if ":" in line:
                k, v = line.split(":", 1)
                try:
                    out[k.strip().lower().replace(" ", "_")] = float(v.split()[0])
                except (ValueError, IndexError):
                    continue
        return out

    def _stack(self, key: str) -> torch.Tensor:
        return torch.cat([n[key] for n in self._raw_nodes if key in n])

    def _fit_or_load_stats(self) -> None:
        node_file = self.stats_dir / "node_stats.json" if self.stats_dir else None
        edge_file = self.stats_dir / "edge_stats.json" if self.stats_dir else None
        if self.split == "train":
            self.node_stats = {}
            for k in self.normalize_keys:
                x = self._stack(k)
                self.node_stats[k + "_mean"], self.node_stats[k + "_std"] = x.mean(0), x.std(0).clamp_min(1e-8)
                self.node_stats[k + "_min"], self.node_stats[k + "_max"] = x.amin(0), x.amax(0)
            e = torch.cat([g.edge_attr for g in self.graphs])
            self.edge_stats = {"edge_mean": e.mean(0), "edge_std": e.std(0).clamp_min(1e-8)}
            if node_file is not None:
                save_json(self.node_stats, node_file)
                save_json(self.edge_stats, edge_file)
        else:
            if node_file is None or not node_file.exists():
                raise IOError("validation / test splits need the statistics written by the training split "
                              "(node_stats.json, edge_stats.json)")
            self.node_stats, self.edge_stats = load_json(node_file), load_json(edge_file)

    def _norm(self, key: str, x: torch.Tensor) -> torch.Tensor:
        if key not in self.normalize_keys:
            return x
        s = self.node_stats
        if self.bounds is None:
            return (x - s[key + "_mean"]) / s[key + "_std"]
        lo, hi = self.bounds
        span = (s[key + "_max"] - s[key + "_min"]).clamp_min(1e-12)
        return (x - s[key + "_min"]) / span * (hi - lo) + lo

    def _finalise(self) -> None:
        for g, nodes in zip(self.graphs, self._raw_nodes):
            g.edge_attr = (g.edge_attr - self.edge_stats["edge_mean"]) / self.edge_stats["edge_std"]
            missing = [k for k in self.input_keys + self.output_keys if k not in nodes]
            if missing:
                raise KeyError(f"sample lacks the arrays {missing}")
            g.x = torch.cat([self._norm(k, nodes[k]) for k in self.input_keys], dim=1)
            g.y = torch.cat([self._norm(k, nodes[k]) for k in self.output_keys], dim=1) if self.output_keys else None

    def denormalize(self, pred: torch.Tensor, gt: torch.Tensor, device=None):
        """Undo the target normalisation column block by column block (order of ``outvar_keys``)."""
        outs = []
        for t in (pred, gt):
            cols, at = [], 0
            for k in self.output_keys:
                w = self._raw_nodes[0][k].shape[1]
                x = t[:, at:at + w]
                if k in self.normalize_keys:
                    s = {n: v.to(t.device) for n, v in self.node_stats.items() if n.startswith(k + "_")}
                    if self.bounds is None:
                        x = x * s[k + "_std"] + s[k + "_mean"]
                    else:
                        lo, hi = self.bounds
                        x = (x - lo) / (hi - lo) * (s[k + "_max"] - s[k + "_min"]) + s[k + "_min"]
                cols.append(x)
                at += w
            outs.append(torch.cat(cols, dim=1).to(device) if device is not None else torch.cat(cols, dim=1))
        return tuple(outs)

    def __len__(self) -> int:
        return len(self.graphs)

    def __getitem__(self, idx: int):
        return self.graphs[idx]


def _vertex_normals_and_areas(pos: torch.Tensor, cells: torch.Tensor):
    p = pos[cells]
    n = torch.linalg.cross(p[:, 1] - p[:, 0], p[:, 2] - p[:, 0])
    area = 0.5 * n.norm(dim=1)
    vn = torch.zeros_like(pos).index_add_(0, cells.reshape(-1), n.repeat_interleave(3, dim=0))
    va = torch.zeros(pos.shape[0]).index_add_(0, cells.reshape(-1), (area / 3).repeat_interleave(3))
    return torch.nn.functional.normalize(vn, dim=1), va


class AhmedBodyDataset(StaticMeshGraphDataset):
    """Surface pressure and wall shear stress of Ahmed bodies; the body's dimensions, inflow velocity and Reynolds number
    are node inputs (constant per case).  ``compute_drag=True`` makes ``__getitem__`` also return the case id, the vertex
    normals, vertex areas and ``2 / (v² A_frontal)`` needed to integrate the drag coefficient."""

    default_invar = ("pos", "velocity", "reynolds_number", "length", "width", "height", "ground_clearance", "slant_angle",
                     "fillet_radius")
    default_outvar = ("p", "wallShearStress")
    default_normalize = ("p", "wallShearStress", "velocity", "reynolds_number", "length", "width", "height", "ground_clearance",
                         "slant_angle", "fillet_radius")
    bounds = (-1.0, 1.0)

    def __init__(self, data_dir=None, split="train", num_samples=10, invar_keys=None, outvar_keys=None, normalize_keys=None,
                 normalization_bound: Tuple[float, float] = (-1.0, 1.0), name="dataset", compute_drag: bool = False,
                 num_workers: Optional[int] = None, samples=None, stats_dir=None):
        self.bounds = tuple(normalization_bound)
        self.compute_drag = compute_drag
        self.normals, self.areas, self.coeff = [], [], []
        super().__init__(data_dir, split, num_samples, invar_keys, outvar_keys, normalize_keys, name, samples, stats_dir)

    def node_arrays(self, sample):
        out = super().node_arrays(sample)
        if "normals" in self.input_keys or self.compute_drag:
            vn, va = _vertex_normals_and_areas(out["pos"], torch.as_tensor(np.asarray(sample["cells"])).long())
            out.setdefault("normals", vn)
            if self.compute_drag:
                frontal = float(sample["width"]) * float(sample["height"]) / 2 * 1e-6          # mm² -> m², half body
                self.normals.append(vn)
                self.areas.append(va)
                self.coeff.append(2.0 / (float(sample["velocity"]) ** 2 * frontal))
        return out

    def __getitem__(self, idx):
        g = self.graphs[idx]
        if self.compute_drag:
            return g, self.case_ids[idx], self.normals[idx], self.areas[idx], self.coeff[idx]
        return g


class DrivAerNetDataset(StaticMeshGraphDataset):
    """DrivAerNet car surfaces: pressure and wall shear stress on the body, drag coefficient per design (``c_d`` of the
    sample, or looked up by design id in ``coeff_filename``, a CSV with the columns ``Design`` and ``Average Cd``)."""

    default_invar = ("pos",)
    default_outvar = ("p", "wallShearStress")
    default_normalize = ("p", "wallShearStress")

    def __init__(self, data_dir=None, split="train", num_samples=10, coeff_filename: Optional[str] = None, invar_keys=None,
                 outvar_keys=None, normalize_keys=None, cache_dir=None, name="dataset", force_reload: bool = False, samples=None,
                 stats_dir=None):
        self._cd = {}
        if coeff_filename is not None and Path(coeff_filename).exists():
            import csv

            with open(coeff_filename) as f:
                for row in csv.DictReader(f):
                    self._cd[row["Design"]] = float(row["Average Cd"])
        super().__init__(data_dir, split, num_samples, invar_keys, outvar_keys, normalize_keys, name, samples, stats_dir)
        for g, cid, s in zip(self.graphs, self.case_ids, (samples or [{}] * len(self.graphs))):
            cd = s.get("c_d", self._cd.get(cid))
            g.c_d = torch.tensor(float(cd)) if cd is not None else None


class StokesDataset(StaticMeshGraphDataset):
    """2-D Stokes flow past obstacles: inputs position and the one-hot boundary ``marker`` (interior / inlet / outlet /
    wall / obstacle), targets ``u``, ``v``, ``p``."""

    default_invar = ("pos", "marker")
    default_outvar = ("u", "v", "p")
    default_normalize = ("u", "v", "p")
    num_markers = 5

    def node_arrays(self, sample):
        out = super().node_arrays(sample)
        if "marker" in sample:
            m = torch.as_tensor(np.asarray(sample["marker"])).long().reshape(-1)
            out["marker"] = torch.nn.functional.one_hot(m, self.num_markers).float()
        return out
