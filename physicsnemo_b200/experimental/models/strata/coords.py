"""Token coordinates for the rotary embeddings of the Strata transformers.

Counterpart of ``physicsnemo/experimental/models/strata/coords.py`` (``build_axial_token_coords`` :39,
``build_stereographic_token_coords`` :70).  Tokens are ordered ``(d, h, w)``; the rotary phase depends on the
horizontal position only, so all levels of a column share their coordinates.
"""

from __future__ import annotations

from typing import Optional, Tuple, Union

import torch

from ...nn.rope import spherical_centroid, stereographic_projection

__all__ = ["build_axial_token_coords", "build_stereographic_token_coords"]


def build_axial_token_coords(d: int, h: int, w: int, device: Optional[torch.device] = None) -> torch.Tensor:
    """``[d*h*w, 2]`` integer-valued ``(row, column)`` coordinates, repeated over the ``d`` levels."""
    ij = torch.stack(torch.meshgrid(torch.arange(h, dtype=torch.float32, device=device),
                                    torch.arange(w, dtype=torch.float32, device=device), indexing="ij"), dim=-1)
    return ij.reshape(1, h * w, 2).expand(d, -1, -1).reshape(d * h * w, 2)


def build_stereographic_token_coords(pos: torch.Tensor, patch_hw: Union[int, Tuple[int, int]], d_patch: int,
                                     length_scale: float) -> torch.Tensor:
    """``[B, d_patch*h*w, 2]`` stereographic coordinates of the patch centroids about the centroid of each tile.

    ``pos`` is ``[B, 2, H, W]`` latitude / longitude in degrees; coordinates are divided by ``length_scale``.
    """
    if length_scale <= 0:
        raise ValueError(f"length_scale must be > 0, got {length_scale}")
    ph, pw = (patch_hw, patch_hw) if isinstance(patch_hw, int) else patch_hw
    lat, lon = pos[:, 0], pos[:, 1]
    B, H, W = lat.shape
    lat0, lon0 = spherical_centroid(lat, lon, reduce_dims=(1, 2))
    patches = lambda t: t.reshape(B, H // ph, ph, W // pw, pw).permute(0, 1, 3, 2, 4)  # noqa: E731
    lat_p, lon_p = spherical_centroid(patches(lat), patches(lon), reduce_dims=(3, 4))
    x, y = stereographic_projection(lat_p.squeeze((-2, -1)), lon_p.squeeze((-2, -1)), lat0, lon0)
    xy = torch.stack([x, y], dim=-1).reshape(B, 1, -1, 2) / length_scale
    return xy.expand(-1, d_patch, -1, -1).reshape(B, -1, 2)
