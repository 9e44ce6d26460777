"""Tensor-rank bookkeeping of mesh data fields (parity: ``physicsnemo/mesh/fields.py``): a *rank spec* maps field
names to tensor ranks (0 scalar, 1 vector, 2 matrix), nested per association."""
from __future__ import annotations

from typing import Dict, Mapping, Union

import torch

RankSpecDict = Dict[str, Union[int, "RankSpecDict"]]


def flatten_rank_spec(spec: Mapping, prefix: str = "") -> Dict[str, int]:
    out: Dict[str, int] = {}
    for k, v in spec.items():
        name = f"{prefix}.{k}" if prefix else k
        if isinstance(v, Mapping):
            out.update(flatten_rank_spec(v, name))
        else:
            out[name] = int(v)
    return out


def rank_counts(spec: Mapping) -> Dict[int, int]:
    counts: Dict[int, int] = {}
    for r in flatten_rank_spec(spec).values():
        counts[r] = counts.get(r, 0) + 1
    return counts


def ranks_from_tensordict(data: Mapping[str, torch.Tensor]) -> Dict[str, int]:
    """Rank of every field = number of trailing dimensions after the entity dimension."""
    return {k: (v.ndim - 1 if isinstance(v, torch.Tensor) else ranks_from_tensordict(v)) for k, v in data.items()}


def validate_data_contains_ranks(data: Mapping[str, torch.Tensor], spec: Mapping) -> None:
    have = flatten_rank_spec(ranks_from_tensordict(data))
    for name, rank in flatten_rank_spec(spec).items():
        if name not in have:
            raise KeyError(f"field '{name}' required by the rank spec is missing; available: {sorted(have)}")
        if have[name] != rank:
            raise ValueError(f"field '{name}' has rank {have[name]}, expected {rank}")
