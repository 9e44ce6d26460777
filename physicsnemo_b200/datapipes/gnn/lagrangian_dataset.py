"""Particle (Lagrangian) dataset of the "Learning to Simulate" family for MeshGraphNet-style simulators.

Parity: ``physicsnemo/datapipes/gnn/lagrangian_dataset.py``.  A sample is the particle system at time ``t``: node
inputs = position ⊕ the last ``num_history`` normalised velocities ⊕ soft distances to the domain walls ⊕ one-hot
particle type; node targets = next position ⊕ next normalised velocity ⊕ next normalised acceleration.  Training
samples get a random-walk noise on the position history (none on kinematic particles).  The graph connects particles
closer than ``radius`` (self edges included) and carries (displacement, ``exp(−d²/r²)``) as edge features; on a GPU the
neighbour search is the library's cell-list radius kernel rather than a dense distance matrix.

Statistics, time step, radius and bounds come from the dataset's ``metadata.json``; trajectories from TFRecord files
when ``tensorflow`` is importable (``gnn/readers.py``), else from ``{split}/*.npz`` with ``position [T, N, D]`` and
``particle_type [N]``.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import List, Optional, Sequence

import numpy as np
import torch
import torch.nn.functional as F
from torch.utils.data import Dataset

from ...nn.module.gnn_layers.graph_types import Graph


def compute_edge_index(pos: torch.Tensor, radius: float) -> torch.Tensor:
    """Pairs ``(i, j)`` with ``|x_i − x_j| < radius`` (self pairs included), ``[2, E]``."""
    if pos.is_cuda and pos.shape[1] == 3:
        from ...nn.functional.neighbors.radius_search import radius_search

        pairs = radius_search(pos, pos, radius)                  # [2, E]: query, point
        return pairs.flip(0).contiguous()
    return torch.nonzero(torch.cdist(pos, pos) < radius).t().contiguous()


def compute_edge_attr(graph: Graph, radius: float = 0.015) -> Graph:
    src, dst = graph.edge_index
    disp = graph.pos[dst] - graph.pos[src]
    graph.edge_attr = torch.cat([disp, torch.exp(-disp.square().sum(-1, keepdim=True) / radius ** 2)], dim=-1)
    return graph


def graph_update(graph: Graph, radius: float) -> Graph:
    """Rebuild the connectivity and edge features for the graph's current positions (used during roll-outs)."""
    graph.edge_index = compute_edge_index(graph.pos, radius)
    graph.num_nodes = graph.num_src_nodes = graph.num_dst_nodes = graph.pos.shape[0]
    return compute_edge_attr(graph, radius)


class LagrangianDataset(Dataset):
    KINEMATIC_PARTICLE_ID = 3          # particle type of prescribed (obstacle) particles

    def __init__(self, name: str = "dataset", data_dir: Optional[str] = None, split: str = "train", num_sequences: int = 1000,
                 num_history: int = 5, num_steps: Optional[int] = None, noise_std: float = 0.0003, radius: Optional[float] = None,
                 dt: Optional[float] = None, bounds: Optional[Sequence[tuple]] = None, num_node_types: int = 6,
                 trajectories: Optional[Sequence[dict]] = None, metadata: Optional[dict] = None, seed: int = 0):
        self.name, self.data_dir, self.split = name, data_dir, split
        self.num_history, self.noise_std, self.num_node_types = num_history, noise_std, num_node_types
        if metadata is None:
            with open(Path(data_dir) / "metadata.json", encoding="utf-8") as f:
                metadata = json.load(f)
        self.dim = int(metadata["dim"])
        self.num_steps = int(metadata["sequence_length"]) + 1 if num_steps is None else num_steps
        self.dt = metadata["dt"] if dt is None else dt
        self.radius = metadata["default_connectivity_radius"] if radius is None else radius
        self.bounds = list(metadata["bounds"][0] if bounds is None else bounds[0])
        for key in ("vel_mean", "vel_std", "acc_mean", "acc_std"):
            setattr(self, key, torch.tensor(metadata[key], dtype=torch.float32).reshape(1, self.dim))
        if trajectories is None:
            trajectories = self._load(Path(data_dir), split, metadata)
        self.node_type: List[torch.Tensor] = []
        self.node_features: List[dict] = []
        for i, tr in enumerate(trajectories):
            if i >= num_sequences:
                break
            position = torch.as_tensor(np.asarray(tr["position"]), dtype=torch.float32)[: self.num_steps]
            if position.shape[0] != self.num_steps:
                raise ValueError(f"trajectory {i} has {position.shape[0]} steps, {self.num_steps} are needed")
            kinds = torch.as_tensor(np.asarray(tr["particle_type"])).long().reshape(-1)
            if kinds.shape[0] != position.shape[1]:
                raise ValueError(f"trajectory {i}: {kinds.shape[0]} particle types for {position.shape[1]} particles")
            self.node_type.append(F.one_hot(kinds, num_node_types).float())
            self.node_features.append({"position": position})
        self.num_sequences = len(self.node_features)
        self.num_samples_per_sequence = self.num_steps - self.num_history - 1
        self.length = self.num_sequences * self.num_samples_per_sequence
        self._gen = torch.Generator().manual_seed(seed)

    @staticmethod
    def _load(folder: Path, split: str, metadata: dict):
        record = folder / f"{split}.tfrecord"
        if record.exists():
            from .readers import read_tfrecord_trajectories

            return read_tfrecord_trajectories(record, metadata)
        files = sorted((folder / split).glob("*.npz"))
        if not files:
            raise IOError(f"neither {record} nor .npz trajectories under {folder / split}")
        return (dict(np.load(f)) for f in files)

    # ------------------------------------------------------------------ sample
    def __len__(self) -> int:
        return self.length

    def get_kinematic_mask(self, graph_idx: int) -> torch.Tensor:
        return self.node_type[graph_idx][:, self.KINEMATIC_PARTICLE_ID] != 0

    def random_walk_noise(self, num_steps: int, num_particles: int) -> torch.Tensor:
        """Position noise whose velocity noise is a random walk reaching ``noise_std`` at the last step."""
        n_vel = num_steps - 1
        vel = (self.noise_std / n_vel ** 0.5) * torch.randn(n_vel, num_particles, self.dim, generator=self._gen)
        vel = vel.cumsum(0)
        return torch.cat([torch.zeros(1, num_particles, self.dim), vel.cumsum(0)])

    @staticmethod
    def time_diff(x: torch.Tensor) -> torch.Tensor:
        return x[1:] - x[:-1]

    @staticmethod
    def compute_boundary_feature(position, radius=0.015, bounds=(0.1, 0.9)) -> torch.Tensor:
        d = torch.cat([position - bounds[0], bounds[1] - position], dim=-1)
        return torch.where(d > radius, torch.zeros_like(d), torch.exp(-d.square() / radius ** 2))

    @staticmethod
    def boundary_clamp(position, bounds=(0.1, 0.9), eps=0.001) -> torch.Tensor:
        return position.clamp(bounds[0] + eps, bounds[1] - eps)

    def normalize_velocity(self, v):
        return (v - self.vel_mean.to(v.device)) / self.vel_std.to(v.device)

    def denormalize_velocity(self, v):
        return v * self.vel_std.to(v.device) + self.vel_mean.to(v.device)

    def normalize_acceleration(self, a):
        return (a - self.acc_mean.to(a.device)) / self.acc_std.to(a.device)

    def denormalize_acceleration(self, a):
        return a * self.acc_std.to(a.device) + self.acc_mean.to(a.device)

    def pack_inputs(self, position, vel_history, node_type) -> torch.Tensor:
        walls = self.compute_boundary_feature(position, self.radius, self.bounds)
        hist = vel_history.permute(1, 0, 2).reshape(position.shape[0], -1)
        return torch.cat([position, hist, walls, node_type], dim=-1)

    def unpack_inputs(self, graph: Graph):
        x = graph.x
        pos = x[..., : self.dim]
        vel = x[..., self.dim: self.dim * (1 + self.num_history)].reshape(-1, self.num_history, self.dim).permute(1, 0, 2)
        return pos, vel, x[..., -self.num_node_types:]

    def unpack_targets(self, graph: Graph):
        y, d = graph.y, self.dim
        return y[..., :d], y[..., d: 2 * d], y[..., 2 * d: 3 * d]

    def __getitem__(self, idx: int) -> Graph:
        if not 0 <= idx < self.length:
            raise IndexError(f"index {idx} outside [0, {self.length})")
        gidx, tidx = divmod(idx, self.num_samples_per_sequence)
        t = tidx + self.num_history
        pos = self.node_features[gidx]["position"][tidx: t + 2].clone()          # num_history + 2 positions
        free = ~self.get_kinematic_mask(gidx)
        if self.split == "train" and self.noise_std > 0:
            pos = pos + self.random_walk_noise(*pos.shape[:2]) * free[None, :, None]
        vel = self.time_diff(pos)
        acc = self.normalize_acceleration(self.time_diff(vel[-2:]))
        vel = self.normalize_velocity(vel)
        current = pos[-2]
        g = Graph(torch.zeros(2, 0, dtype=torch.long), num_nodes=current.shape[0])
        g.x = self.pack_inputs(current, vel[:-1], self.node_type[gidx])
        g.y = torch.cat([pos[-1], vel[-1], acc[-1]], dim=-1)
        g.pos, g.mask = current, free
        g.t = torch.full((current.shape[0],), tidx)
        return graph_update(g, self.radius)
