"""Padding, flattening and neighbour helpers for point-cloud transformers.

Parity: ``physicsnemo/experimental/nn/point_utils.py`` (``gather_rows`` ``:33``, ``counts_to_mask``
``:55``, ``flatten_padded_batch`` ``:88``, ``unflatten_to_padded`` ``:123``,
``compute_batch_offset_step`` ``:168``, ``flatten_batched_coords`` ``:225``, ``chunked_knn_indices``
``:285``, ``masked_mean`` ``:352``).  A padded batch is a ``(B, N_max, …)`` tensor with a boolean
``(B, N_max)`` mask; its flat form keeps the valid rows in batch order.
"""
from __future__ import annotations

from typing import Optional

import torch

from ...nn.functional.neighbors import knn


def gather_rows(x: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """``x[idx]`` for a ``(N, F)`` table and an index tensor of any shape → ``(*idx.shape, F)``."""
    return x.index_select(0, idx.reshape(-1)).reshape(*idx.shape, x.shape[-1])


def counts_to_mask(counts: torch.Tensor, max_len: Optional[int] = None) -> torch.Tensor:
    """``(B,)`` valid counts → ``(B, max_len)`` mask that is true on the first ``counts[b]`` columns."""
    if counts.ndim != 1:
        raise ValueError(f"counts_to_mask expects rank-1 counts, got {tuple(counts.shape)}")
    if max_len is None:
        max_len = int(counts.max()) if counts.numel() else 0
    return torch.arange(int(max_len), device=counts.device)[None, :] < counts[:, None]


def _check_padded(x: torch.Tensor, mask: torch.Tensor, who: str) -> None:
    if mask.ndim != 2 or x.ndim < 2 or tuple(x.shape[:2]) != tuple(mask.shape):
        raise ValueError(f"{who} expects x of shape (B, N, ...) and a (B, N) mask, "
                         f"got {tuple(x.shape)} and {tuple(mask.shape)}")


def flatten_padded_batch(x: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """Valid rows of a padded batch, in batch order: ``(B, N, …)`` → ``(mask.sum(), …)``."""
    _check_padded(x, mask, "flatten_padded_batch")
    return x[mask]


def unflatten_to_padded(flat: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`flatten_padded_batch`; padded slots are zero."""
    if mask.ndim != 2:
        raise ValueError(f"unflatten_to_padded expects a rank-2 mask, got {tuple(mask.shape)}")
    if flat.shape[0] != int(mask.sum()):
        raise ValueError(f"flat has {flat.shape[0]} rows but the mask selects {int(mask.sum())}")
    out = flat.new_zeros(tuple(mask.shape) + tuple(flat.shape[1:]))
    out[mask] = flat
    return out


def compute_batch_offset_step(coords: torch.Tensor, mask: Optional[torch.Tensor] = None) -> float:
    """Shift between consecutive batch items that keeps their clouds apart: ``4 · (largest extent + 1)``."""
    if coords.ndim not in (2, 3):
        raise ValueError(f"compute_batch_offset_step expects rank-2/3 coords, got {tuple(coords.shape)}")
    if mask is not None:
        if coords.ndim != 3:
            raise ValueError("mask is only supported for rank-3 coords.")
        _check_padded(coords, mask, "compute_batch_offset_step")
        pts = coords[mask]
    else:
        pts = coords.reshape(-1, coords.shape[-1])
    if pts.shape[0] == 0:
        return 1.0
    extent = float((pts.amax(0) - pts.amin(0)).abs().max())
    return max(4.0 * (extent + 1.0), 1.0)


def flatten_batched_coords(coords: torch.Tensor, mask: torch.Tensor, *, offset_step: float):
    """Flat coordinates, the same shifted along the first axis by ``batch · offset_step``, and batch ids.

    A neighbour search on the shifted coordinates cannot pair points of different batch items as
    long as ``offset_step`` exceeds the extent of every cloud.
    """
    if coords.ndim != 3:
        raise ValueError("flatten_batched_coords expects rank-3 coords and rank-2 mask.")
    _check_padded(coords, mask, "flatten_batched_coords")
    flat = coords[mask]
    batch_ids = mask.nonzero()[:, 0]
    shift = torch.zeros_like(flat)
    shift[:, 0] = batch_ids.to(flat.dtype) * float(offset_step)
    return flat, flat + shift, batch_ids


def chunked_knn_indices(*, query_coords: torch.Tensor, key_coords: torch.Tensor, k: int, chunk_size: int = 128,
                        dilation: int = 1) -> torch.Tensor:
    """Indices ``(Q, ≤k)`` of every ``dilation``-th of the ``k · dilation`` nearest keys of each query.

    ``chunk_size`` is accepted for interface parity; the neighbour search tiles internally.
    """
    if query_coords.ndim != 2 or key_coords.ndim != 2:
        raise ValueError("chunked_knn_indices expects rank-2 query_coords and key_coords.")
    if query_coords.shape[-1] != key_coords.shape[-1]:
        raise ValueError("query_coords and key_coords must have the same coordinate dimension.")
    if query_coords.shape[0] == 0 or key_coords.shape[0] == 0:
        raise ValueError("query_coords and key_coords must both contain at least one point.")
    if min(int(k), int(chunk_size), int(dilation)) <= 0:
        raise ValueError("k, chunk_size, and dilation must be positive.")
    wanted = min(int(k) * int(dilation), key_coords.shape[0])
    idx = knn(points=key_coords, queries=query_coords, k=wanted)[0].long()[:, ::int(dilation)]
    return idx[:, :min(int(k), idx.shape[1])]


def masked_mean(features: torch.Tensor, mask: Optional[torch.Tensor]) -> torch.Tensor:
    """Mean over the token axis (the one before the feature axis), kept as a size-1 axis.

    ``features`` is ``(N, F)`` with a ``(N,)`` mask or ``(B, N, F)`` with a ``(B, N)`` mask; only
    tokens whose mask is true count, and a set without valid tokens gives zeros.
    """
    if features.ndim not in (2, 3):
        raise ValueError(f"masked_mean expects (N, F) or (B, N, F) features, got {tuple(features.shape)}")
    if mask is None:
        return features.mean(dim=-2, keepdim=True)
    if tuple(mask.shape) != tuple(features.shape[:-1]):
        raise ValueError(f"mask {tuple(mask.shape)} does not match the tokens of features {tuple(features.shape)}")
    w = mask.to(features.dtype).unsqueeze(-1)
    return (features * w).sum(dim=-2, keepdim=True) / w.sum(dim=-2, keepdim=True).clamp_min(1.0)
