"""Flood-routing graphs for HydroGraphNet: one watershed mesh, many hydrographs (rain / inflow events).

Parity: ``physicsnemo/datapipes/gnn/hydrographnet_dataset.py`` (``HydroGraphDataset``).  Static node data (cell
centres, area, elevation, slope, aspect, curvature, Manning roughness, flow accumulation, infiltration) is standardised
once; the graph links every cell to its ``k`` nearest cells with standardised (relative position, distance) edge
features.  Each hydrograph contributes water depth and volume per cell over time plus the scalar precipitation and
inflow series.  Training samples are sliding windows: node input = static ⊕ current inflow ⊕ current precipitation ⊕
``n_time_steps`` past depths ⊕ ``n_time_steps`` past volumes, target = the next step's depth and volume increments.
Test samples are whole events: the first window as graph plus the roll-out series.  ``return_physics`` (and the
push-forward noise mode) adds the quantities of the mass-balance loss.

Files (``.npy`` / ``.txt`` per field in the reference's layout, or one ``.npz`` per hydrograph): the loaders below take
arrays, ``from_directory`` reads ``{prefix}_static.npz`` and ``{prefix}_{id}.npz``.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch
from torch.utils.data import Dataset

from ...nn.module.gnn_layers.graph_types import Graph

STATIC_KEYS = ("area", "elevation", "slope", "aspect", "curvature", "manning", "flow_accum", "infiltration")
STATIC_NORM_STATS_FILE = "static_norm_stats.json"
DYNAMIC_NORM_STATS_FILE = "dynamic_norm_stats.json"
_NOISE = ("none", "pushforward", "gaussian", "correlated", "uniform", "only_last", "random_walk")


def _standardise(x: np.ndarray, stats: Optional[dict], key: str, out: dict) -> np.ndarray:
    if stats is None:
        out[key] = {"mean": float(np.mean(x)), "std": float(np.std(x) + 1e-8)}
    else:
        out[key] = stats[key]
    return (x - out[key]["mean"]) / out[key]["std"]


class HydroGraphDataset(Dataset):
    def __init__(self, name: str = "hydrograph_dataset", data_dir=None, prefix: str = "M80", num_samples: int = 500,
                 n_time_steps: int = 10, k: int = 4, noise_std: float = 0.01, noise_type: str = "none",
                 hydrograph_ids_file: Optional[str] = None, split: str = "train", rollout_length: Optional[int] = None,
                 return_physics: bool = False, static: Optional[Dict[str, np.ndarray]] = None,
                 hydrographs: Optional[Sequence[Dict[str, np.ndarray]]] = None, stats_dir=None, seed: int = 0):
        if split not in ("train", "test"):
            raise ValueError(f"split is 'train' or 'test', got {split!r}")
        if noise_type not in _NOISE:
            raise ValueError(f"noise_type must be one of {_NOISE}")
        self.name, self.prefix, self.split = name, prefix, split
        self.n_time_steps, self.k, self.noise_std, self.noise_type = n_time_steps, k, noise_std, noise_type
        self.rollout_length = rollout_length or 0
        self.return_physics = return_physics
        self.stats_dir = Path(stats_dir if stats_dir is not None else (data_dir or "."))
        self._rng = np.random.default_rng(seed)
        if static is None:
            static, hydrographs = self._read(Path(data_dir), prefix, hydrograph_ids_file, num_samples)
        hydrographs = list(hydrographs)[:num_samples]
        loaded_s = self.load_norm_stats(STATIC_NORM_STATS_FILE) if split == "test" else None
        loaded_d = self.load_norm_stats(DYNAMIC_NORM_STATS_FILE) if split == "test" else None
        # ---- static data and graph
        self.static_stats: dict = {}
        xy = np.asarray(static["xy_coords"], dtype=np.float64)
        lo, hi = (xy.min(0), xy.max(0)) if loaded_s is None else (np.array(loaded_s["xy"]["min"]), np.array(loaded_s["xy"]["max"]))
        self.static_stats["xy"] = {"min": lo.tolist(), "max": hi.tolist()}
        xy_n = (xy - lo) / np.maximum(hi - lo, 1e-12)
        self.static_data = {"xy_coords": xy_n.astype(np.float32), "area_denorm": np.asarray(static["area"], dtype=np.float32)}
        for key in STATIC_KEYS:
            col = np.asarray(static[key], dtype=np.float64).reshape(-1, 1)
            self.static_data[key] = _standardise(col, loaded_s, key, self.static_stats).astype(np.float32)
        self.static_data["edge_index"] = self._knn_edges(xy_n, k)
        self.static_data["edge_features"] = self.create_edge_features(xy_n, self.static_data["edge_index"])
        # ---- dynamic data
        self.dynamic_stats: dict = {}
        if loaded_d is None:
            for key in ("water_depth", "volume", "precipitation", "inflow_hydrograph"):
                allv = np.concatenate([np.asarray(h[key], dtype=np.float64).reshape(-1) for h in hydrographs])
                self.dynamic_stats[key] = {"mean": float(allv.mean()), "std": float(allv.std() + 1e-8)}
        else:
            self.dynamic_stats = loaded_d
        self.dynamic_data: List[dict] = []
        for h in hydrographs:
            d = {}
            for key in ("water_depth", "volume", "precipitation", "inflow_hydrograph"):
                s = self.dynamic_stats[key]
                d[key] = ((np.asarray(h[key], dtype=np.float64) - s["mean"]) / s["std"]).astype(np.float32)
            self.dynamic_data.append(d)
        if split == "train":
            self.save_norm_stats(self.static_stats, STATIC_NORM_STATS_FILE)
            self.save_norm_stats(self.dynamic_stats, DYNAMIC_NORM_STATS_FILE)
        # ---- sample index
        self.sample_index = []
        extra = 1 if noise_type == "pushforward" else 0
        for hi_, d in enumerate(self.dynamic_data):
            T = d["water_depth"].shape[0]
            if split == "train":
                self.sample_index += [(hi_, t) for t in range(T - n_time_steps - extra)]
            else:
                self.sample_index.append((hi_, 0))

    # ------------------------------------------------------------------ io
    @staticmethod
    def _read(folder: Path, prefix: str, ids_file: Optional[str], limit: int):
        static = dict(np.load(folder / f"{prefix}_static.npz"))
        if ids_file is not None:
            ids = [ln.strip() for ln in (folder / ids_file).read_text().splitlines() if ln.strip()]
        else:
            ids = sorted(p.stem[len(prefix) + 1:] for p in folder.glob(f"{prefix}_*.npz") if not p.stem.endswith("_static"))
        return static, [dict(np.load(folder / f"{prefix}_{i}.npz")) for i in ids[:limit]]

    def save_norm_stats(self, stats: dict, filename: str) -> None:
        self.stats_dir.mkdir(parents=True, exist_ok=True)
        (self.stats_dir / filename).write_text(json.dumps(stats))

    def load_norm_stats(self, filename: str) -> dict:
        path = self.stats_dir / filename
        if not path.exists():
            raise FileNotFoundError(f"{path} is written by the training split; build that first")
        return json.loads(path.read_text())

    # --------------------------------------------------------------- graph
    @staticmethod
    def _knn_edges(xy: np.ndarray, k: int) -> np.ndarray:
        from ...nn.functional.neighbors.knn import knn

        pts = torch.as_tensor(xy, dtype=torch.float32)
        idx, _ = knn(pts, pts, min(k + 1, pts.shape[0]))
        src = torch.arange(pts.shape[0]).repeat_interleave(idx.shape[1])
        dst = idx.reshape(-1)
        keep = src != dst
        return torch.stack([src[keep], dst[keep]]).numpy()

    @staticmethod
    def create_edge_features(xy: np.ndarray, edge_index: np.ndarray) -> np.ndarray:
        rel = xy[edge_index[0]] - xy[edge_index[1]]
        dist = np.linalg.norm(rel, axis=1)
        rel = (rel - rel.mean(0)) / (rel.std(0) + 1e-8)
        dist = (dist - dist.mean()) / (dist.std() + 1e-8)
        return np.hstack([rel, dist[:, None]]).astype(np.float32)

    def apply_noise_to_feature(self, window: np.ndarray, noise_type: str, std: float) -> np.ndarray:
        """``window``: [time, nodes].  gaussian / uniform: independent; correlated: one draw per node for all steps;
        only_last: the newest step only; random_walk: cumulative over the window."""
        T, N = window.shape
        if noise_type == "gaussian":
            n = self._rng.normal(0, std, (T, N))
        elif noise_type == "uniform":
            n = self._rng.uniform(-std, std, (T, N))
        elif noise_type == "correlated":
            n = np.repeat(self._rng.normal(0, std, (1, N)), T, axis=0)
        elif noise_type == "only_last":
            n = np.zeros((T, N))
            n[-1] = self._rng.normal(0, std, N)
        elif noise_type == "random_walk":
            n = np.cumsum(self._rng.normal(0, std / max(T, 1) ** 0.5, (T, N)), axis=0)
        else:
            return window
        return (window + n).astype(window.dtype)

    def create_node_features(self, depth_win: np.ndarray, volume_win: np.ndarray, precipitation: np.ndarray, inflow: np.ndarray,
                             t: int):
        sd = self.static_data
        if self.noise_type not in ("none", "pushforward"):
            depth_win = self.apply_noise_to_feature(depth_win[: self.n_time_steps], self.noise_type, self.noise_std)
            volume_win = self.apply_noise_to_feature(volume_win[: self.n_time_steps], self.noise_type, self.noise_std)
        n = sd["xy_coords"].shape[0]
        cols = [sd["xy_coords"]] + [sd[k] for k in STATIC_KEYS]
        cols += [np.full((n, 1), inflow[t], dtype=np.float32), np.full((n, 1), precipitation[t], dtype=np.float32)]
        cols += [depth_win[: self.n_time_steps].T, volume_win[: self.n_time_steps].T]
        return np.hstack(cols).astype(np.float32), float(inflow[t + self.n_time_steps]), float(precipitation[t + self.n_time_steps])

    def _graph(self) -> Graph:
        sd = self.static_data
        g = Graph(torch.as_tensor(sd["edge_index"]).long(), num_nodes=sd["xy_coords"].shape[0])
        g.edge_attr = torch.as_tensor(sd["edge_features"])
        return g

    def __len__(self) -> int:
        return len(self.sample_index)

    def __getitem__(self, idx: int):
        h, t = self.sample_index[idx]
        dyn = self.dynamic_data[h]
        n = self.n_time_steps
        g = self._graph()
        if self.split == "train":
            end = t + n + (1 if self.noise_type == "pushforward" else 0)
            x, fut_in, fut_pr = self.create_node_features(dyn["water_depth"][t:end], dyn["volume"][t:end], dyn["precipitation"],
                                                          dyn["inflow_hydrograph"], t)
            tgt, prev = t + n, t + n - 1
            g.x = torch.as_tensor(x)
            g.y = torch.as_tensor(np.stack([dyn["water_depth"][tgt] - dyn["water_depth"][prev],
                                            dyn["volume"][tgt] - dyn["volume"][prev]], axis=1))
            if not (self.return_physics or self.noise_type == "pushforward"):
                return g
            physics = {"flow_future": fut_in, "precip_future": fut_pr, "past_volume": float(dyn["volume"][prev].sum()),
                       "future_volume": float(dyn["volume"][tgt].sum()), "avg_inflow": float(dyn["inflow_hydrograph"][prev:tgt + 1].mean()),
                       "avg_precipitation": float(dyn["precipitation"][prev:tgt + 1].mean()),
                       "area_denorm": torch.as_tensor(self.static_data["area_denorm"])}
            return g, physics
        x, _, _ = self.create_node_features(dyn["water_depth"][:n], dyn["volume"][:n], dyn["precipitation"],
                                            dyn["inflow_hydrograph"], 0)
        g.x = torch.as_tensor(x)
        stop = n + self.rollout_length if self.rollout_length else dyn["water_depth"].shape[0]
        rollout = {k: torch.as_tensor(dyn[k][n:stop]) for k in ("water_depth", "volume", "precipitation", "inflow_hydrograph")}
        return g, rollout

    def denormalize(self, values: torch.Tensor, key: str) -> torch.Tensor:
        s = self.dynamic_stats[key]
        return values * s["std"] + s["mean"]
