"""Token containers of the AeroJEPA components and the conversions between their single and batched forms.

Parity: ``physicsnemo/experimental/models/aerojepa/layers/types.py`` (``TokenSet`` ``:34``,
``EncoderOutput`` ``:147``) and ``layers/token_utils.py`` (``trim_batched_tokens`` ``:38``,
``pad_token_sets`` ``:79``, ``flatten_valid_token_features`` ``:138``,
``reshape_token_features_for_sigreg`` ``:184``).  ``FlatTokens`` has no reference counterpart: every
component here runs on one flat list of tokens with batch ids, and a single cloud is the batch of one.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Iterable, Optional

import torch

from ...nn.point_utils import compute_batch_offset_step, masked_mean


@dataclass
class TokenSet:
    """Latent tokens: ``features`` ``(T, C)`` / ``(B, T, C)``, ``coords`` ``(T, 3)`` / ``(B, T, 3)``, optional validity ``mask``."""

    features: torch.Tensor
    coords: torch.Tensor
    mask: Optional[torch.Tensor] = None
    global_token: Optional[torch.Tensor] = None
    aux: dict = field(default_factory=dict)

    @property
    def is_batched(self) -> bool:
        return self.features.ndim == 3

    @property
    def token_dim(self) -> int:
        return int(self.features.shape[-1])

    def with_updates(self, *, features=None, coords=None, mask=None, global_token=None, aux=None) -> "TokenSet":
        pick = lambda new, old: old if new is None else new  # noqa: E731
        return TokenSet(pick(features, self.features), pick(coords, self.coords), pick(mask, self.mask),
                        pick(global_token, self.global_token), dict(self.aux) if aux is None else aux)


@dataclass
class EncoderOutput:
    tokens: TokenSet
    global_token: Optional[torch.Tensor] = None
    aux: dict = field(default_factory=dict)


@dataclass
class FlatTokens:
    """Valid tokens of a batch in one list.

    ``coords`` are the true positions; ``search`` are the same shifted per batch item along the first
    axis so that a neighbour search never crosses items; ``batch`` holds the item of every token and
    ``mask`` ``(B, T)`` is the padded layout the list came from.
    """

    coords: torch.Tensor
    search: torch.Tensor
    batch: torch.Tensor
    mask: torch.Tensor

    @classmethod
    def from_padded(cls, coords: torch.Tensor, mask: Optional[torch.Tensor], offset_step: Optional[float] = None) -> "FlatTokens":
        if coords.ndim == 2:
            coords = coords.unsqueeze(0)
            mask = None if mask is None else mask.reshape(1, -1)
        if mask is None:
            mask = torch.ones(coords.shape[:2], dtype=torch.bool, device=coords.device)
        if offset_step is None:
            offset_step = compute_batch_offset_step(coords, mask)
        flat = coords[mask]
        batch = mask.nonzero()[:, 0]
        shift = torch.zeros_like(flat)
        shift[:, 0] = batch.to(flat.dtype) * float(offset_step)
        return cls(flat, flat + shift, batch, mask)

    def gather(self, padded: torch.Tensor) -> torch.Tensor:
        """Rows of a ``(B, T, …)`` (or, for one cloud, ``(T, …)``) tensor in this list's order."""
        if tuple(padded.shape[:2]) != tuple(self.mask.shape):      # (T, …) of a single cloud
            padded = padded.unsqueeze(0)
        return padded[self.mask]

    def per_item(self, values: torch.Tensor) -> torch.Tensor:
        """Broadcast one row per batch item ``(B, C)`` to every token ``(n, C)``."""
        return values[self.batch]

    def scatter(self, flat: torch.Tensor) -> torch.Tensor:
        out = flat.new_zeros(tuple(self.mask.shape) + tuple(flat.shape[1:]))
        out[self.mask] = flat
        return out


def shared_offset_step(*pairs) -> float:
    """One shift that separates the batch items of several padded coordinate sets ``(coords, mask)``."""
    return max(compute_batch_offset_step(c if c.ndim == 3 else c.unsqueeze(0),
                                         None if m is None else (m if m.ndim == 2 else m.reshape(1, -1)))
               for c, m in pairs)


def trim_batched_tokens(tokens: TokenSet, index: int, count: int) -> TokenSet:
    """Item ``index`` of a batched set, cut to its first ``count`` tokens."""
    if not tokens.is_batched:
        raise ValueError("trim_batched_tokens expects a batched TokenSet.")
    return TokenSet(features=tokens.features[index, :count], coords=tokens.coords[index, :count],
                    mask=None if tokens.mask is None else tokens.mask[index, :count],
                    global_token=None if tokens.global_token is None else tokens.global_token[index:index + 1],
                    aux=dict(tokens.aux))


def pad_token_sets(token_sets: Iterable[TokenSet]) -> TokenSet:
    """Stack unbatched sets into one padded set; missing global tokens become the mean of the set's tokens."""
    sets = list(token_sets)
    if not sets:
        raise ValueError("pad_token_sets expects at least one TokenSet.")
    sizes = [s.features.shape[0] for s in sets]
    first = sets[0]
    feats = first.features.new_zeros(len(sets), max(sizes), first.features.shape[-1])
    coords = first.coords.new_zeros(len(sets), max(sizes), first.coords.shape[-1])
    for i, (s, n) in enumerate(zip(sets, sizes)):
        feats[i, :n], coords[i, :n] = s.features, s.coords
    sizes_t = torch.tensor(sizes, device=feats.device)
    mask = torch.arange(max(sizes), device=feats.device)[None, :] < sizes_t[:, None]
    glob = [(s.global_token if s.global_token is not None else masked_mean(s.features, None)).reshape(1, -1) for s in sets]
    return TokenSet(features=feats, coords=coords, mask=mask, global_token=torch.cat(glob, dim=0))


def flatten_valid_token_features(features: torch.Tensor, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``(T, C)`` unchanged; ``(B, T, C)`` → the valid rows ``(n, C)``."""
    if features.ndim == 2:
        return features
    if features.ndim != 3:
        raise ValueError(f"Expected rank-2 or rank-3 features, got {tuple(features.shape)}")
    if mask is None:
        return features.reshape(-1, features.shape[-1])
    if mask.shape != features.shape[:2]:
        raise ValueError(f"mask must match features.shape[:2], got {tuple(mask.shape)} vs {tuple(features.shape[:2])}")
    return features[mask]


def reshape_token_features_for_sigreg(features: torch.Tensor, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Valid token features as one ``(1, n, C)`` sample set for a distribution-matching regulariser."""
    flat = flatten_valid_token_features(features, mask)
    return flat.unsqueeze(0) if flat.shape[0] else flat.new_zeros(1, 0, flat.shape[-1])
