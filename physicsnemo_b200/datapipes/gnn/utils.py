"""Helpers shared by the mesh-graph datasets (parity: ``physicsnemo/datapipes/gnn/utils.py``)."""
from __future__ import annotations

import json
from pathlib import Path

import torch


def load_json(file: str | Path) -> dict:
    """Load a stats file; lists become tensors."""
    with open(file) as f:
        return {k: torch.tensor(v) if isinstance(v, list) else v for k, v in json.load(f).items()}


def save_json(var: dict, file: str | Path) -> None:
    """Save a dict of tensors / scalars as JSON (the parent directory is created when missing)."""
    Path(file).parent.mkdir(parents=True, exist_ok=True)
    with open(file, "w") as f:
        json.dump({k: (v.tolist() if hasattr(v, "tolist") else v) for k, v in var.items()}, f)


def cells_to_edges(cells: torch.Tensor, bidirectional: bool = True) -> torch.Tensor:
    """Unique edges ``[2, E]`` of simplicial cells ``[C, V]``; both directions unless ``bidirectional`` is false."""
    V = cells.shape[1]
    pairs = torch.cat([cells[:, [i, j]] for i in range(V) for j in range(i + 1, V)], dim=0)
    pairs = torch.unique(pairs.sort(dim=1).values, dim=0)
    if bidirectional:
        pairs = torch.cat([pairs, pairs.flip(1)], dim=0)
    return pairs.t().contiguous()


def edge_features(pos: torch.Tensor, edge_index: torch.Tensor) -> torch.Tensor:
    """Relative displacement and its norm, ``[E, D + 1]``."""
    d = pos[edge_index[0]] - pos[edge_index[1]]
    return torch.cat([d, d.norm(dim=-1, keepdim=True)], dim=-1)
