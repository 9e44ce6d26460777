"""One-step-ahead mesh-graph datasets for MeshGraphNet-style simulators (vortex shedding and relatives).

Parity: ``physicsnemo/datapipes/gnn/vortex_shedding_dataset.py`` (``VortexSheddingDataset``) and the shared logic of the
other ``datapipes/gnn`` datasets: every trajectory is a fixed mesh (``mesh_pos [N, D]``, ``cells [C, V]``,
``node_type [N]``) with fields over time (``velocity [T, N, D]``, ``pressure [T, N, 1]``).  A sample is the graph at time
``t``: node features = velocity (+ optional training noise on normal nodes) ⊕ one-hot node type, edge features = relative
displacement ⊕ length (normalised by dataset statistics), target = normalised velocity increment ⊕ normalised pressure.
Statistics are computed once from the training split and reused for validation / test (``node_stats`` / ``edge_stats``
can be saved with ``gnn.utils.save_json``).

The reference reads TFRecord / VTK files; those readers are not available here, so trajectories come as dicts of arrays
or from ``.npz`` files with the same keys (``VortexSheddingDataset.from_npz_dir``).
"""
from __future__ import annotations

from pathlib import Path
from typing import Dict, List, Sequence

import numpy as np
import torch
from torch.utils.data import Dataset

from ...nn.module.gnn_layers.graph_types import Graph
from .utils import cells_to_edges, edge_features

NODE_NORMAL, NODE_OBSTACLE, NODE_AIRFOIL, NODE_HANDLE, NODE_INFLOW, NODE_OUTFLOW, NODE_WALL = 0, 1, 2, 3, 4, 5, 6


def _stats(x: torch.Tensor, eps: float = 1e-8) -> Dict[str, torch.Tensor]:
    flat = x.reshape(-1, x.shape[-1]).double()
    return {"mean": flat.mean(0).float(), "std": flat.std(0).clamp_min(eps).float()}


class MeshGraphTimeSeriesDataset(Dataset):
    def __init__(self, trajectories: Sequence[dict], split: str = "train", num_steps: int | None = None, noise_std: float = 0.02,
                 num_node_types: int = 7, node_stats: dict | None = None, edge_stats: dict | None = None, seed: int = 0):
        if split not in ("train", "valid", "test"):
            raise ValueError("split must be 'train', 'valid' or 'test'")
        if split != "train" and (node_stats is None or edge_stats is None):
            raise ValueError("validation / test splits reuse the statistics of the training split: pass node_stats and edge_stats")
        self.split, self.noise_std, self.num_node_types = split, noise_std, num_node_types
        self.graphs: List[dict] = []
        for tr in trajectories:
            pos = torch.as_tensor(np.asarray(tr["mesh_pos"]), dtype=torch.float32)
            cells = torch.as_tensor(np.asarray(tr["cells"])).long()
            vel = torch.as_tensor(np.asarray(tr["velocity"]), dtype=torch.float32)
            prs = torch.as_tensor(np.asarray(tr["pressure"]), dtype=torch.float32)
            if num_steps is not None:
                vel, prs = vel[:num_steps], prs[:num_steps]
            ntype = torch.as_tensor(np.asarray(tr["node_type"])).long().reshape(-1)
            ei = cells_to_edges(cells)
            self.graphs.append({"pos": pos, "edge_index": ei, "edge_attr": edge_features(pos, ei), "node_type": ntype, "velocity": vel,
                                "pressure": prs, "cells": cells})
        if not self.graphs:
            raise ValueError("no trajectories given")
        self.steps = [g["velocity"].shape[0] - 1 for g in self.graphs]
        self.offsets = np.cumsum([0] + self.steps)
        if node_stats is None:
            vel = torch.cat([g["velocity"].reshape(-1, g["velocity"].shape[-1]) for g in self.graphs])
            dv = torch.cat([(g["velocity"][1:] - g["velocity"][:-1]).reshape(-1, g["velocity"].shape[-1]) for g in self.graphs])
            prs = torch.cat([g["pressure"].reshape(-1, g["pressure"].shape[-1]) for g in self.graphs])
            sv, sd, sp = _stats(vel), _stats(dv), _stats(prs)
            node_stats = {"velocity_mean": sv["mean"], "velocity_std": sv["std"], "velocity_diff_mean": sd["mean"],
                          "velocity_diff_std": sd["std"], "pressure_mean": sp["mean"], "pressure_std": sp["std"]}
        if edge_stats is None:
            se = _stats(torch.cat([g["edge_attr"] for g in self.graphs]))
            edge_stats = {"edge_mean": se["mean"], "edge_std": se["std"]}
        self.node_stats, self.edge_stats = node_stats, edge_stats
        for g in self.graphs:
            g["edge_attr"] = (g["edge_attr"] - edge_stats["edge_mean"]) / edge_stats["edge_std"]
        self._gen = torch.Generator().manual_seed(seed)

    @classmethod
    def from_npz_dir(cls, data_dir: str | Path, **kwargs) -> "MeshGraphTimeSeriesDataset":
        files = sorted(Path(data_dir).glob("*.npz"))
        if not files:
            raise IOError(f"no .npz trajectories in {data_dir}")
        return cls([dict(np.load(f)) for f in files], **kwargs)

    def __len__(self) -> int:
        return int(self.offsets[-1])

    def __getitem__(self, idx: int) -> dict:
        gi = int(np.searchsorted(self.offsets, idx, side="right") - 1)
        t = idx - int(self.offsets[gi])
        g, s = self.graphs[gi], self.node_stats
        vel = g["velocity"][t]
        if self.split == "train" and self.noise_std > 0:
            noise = torch.randn(vel.shape, generator=self._gen) * self.noise_std
            vel = vel + noise * (g["node_type"] == NODE_NORMAL).unsqueeze(-1)
        onehot = torch.nn.functional.one_hot(g["node_type"].clamp_max(self.num_node_types - 1), self.num_node_types).float()
        x = torch.cat([(vel - s["velocity_mean"]) / s["velocity_std"], onehot], dim=-1)
        dv = (g["velocity"][t + 1] - vel - s["velocity_diff_mean"]) / s["velocity_diff_std"]      # the target absorbs the injected noise
        p = (g["pressure"][t + 1] - s["pressure_mean"]) / s["pressure_std"]
        return {"graph": Graph(g["edge_index"], num_nodes=g["pos"].shape[0]), "x": x, "edge_attr": g["edge_attr"], "y": torch.cat([dv, p], dim=-1),
                "mesh_pos": g["pos"], "cells": g["cells"], "node_type": g["node_type"]}

    def denormalize(self, pred: torch.Tensor) -> tuple:
        """Split a model output into velocity increment and pressure in physical units."""
        s, d = self.node_stats, self.node_stats["velocity_diff_mean"].shape[0]
        return pred[..., :d] * s["velocity_diff_std"] + s["velocity_diff_mean"], pred[..., d:] * s["pressure_std"] + s["pressure_mean"]


class VortexSheddingDataset(MeshGraphTimeSeriesDataset):
    """Cylinder-flow trajectories (2-D velocity + pressure on a triangle mesh); same sample layout as the reference dataset."""
