"""Continuous-position rotary embeddings and the sphere → plane projection that feeds them.

Parity: ``physicsnemo/experimental/nn/rope.py`` (``stereographic_projection``, ``spherical_centroid``,
``build_rope_cos_sin_1d_continuous``, ``build_axial_rope_cos_sin_2d_continuous``); ``apply_rope`` rotates adjacent
channel pairs with the tables those builders return.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

__all__ = ["apply_rope", "build_axial_rope_cos_sin_2d_continuous", "build_rope_cos_sin_1d_continuous", "spherical_centroid",
           "stereographic_projection"]


def stereographic_projection(lat, lon, lat0, lon0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Plane coordinates of (lat, lon) [rad] under the stereographic projection centred at (lat0, lon0)."""
    dlon = lon - lon0
    cos_c = torch.sin(lat0) * torch.sin(lat) + torch.cos(lat0) * torch.cos(lat) * torch.cos(dlon)
    k = 2.0 / (1.0 + cos_c).clamp_min(1e-6)
    return k * torch.cos(lat) * torch.sin(dlon), k * (torch.cos(lat0) * torch.sin(lat) - torch.sin(lat0) * torch.cos(lat) * torch.cos(dlon))


def spherical_centroid(lat, lon, reduce_dims: Tuple[int, ...] = (-2, -1)) -> Tuple[torch.Tensor, torch.Tensor]:
    """Direction of the mean unit vector of the points, as (lat0, lon0)."""
    c = lat.cos()
    x, y, z = (c * lon.cos()).mean(reduce_dims, keepdim=True), (c * lon.sin()).mean(reduce_dims, keepdim=True), lat.sin().mean(reduce_dims, keepdim=True)
    return torch.atan2(z, torch.hypot(x, y)), torch.atan2(y, x)


def build_rope_cos_sin_1d_continuous(positions, dim: int, theta: float = 10000.0, device: Optional[torch.device] = None):
    if dim % 2:
        raise ValueError(f"dim={dim} must be even (rotation acts on adjacent channel pairs).")
    if device is not None:
        positions = positions.to(device)
    freqs = theta ** (-torch.arange(0, dim, 2, dtype=torch.float32, device=positions.device) / dim)
    ang = positions.float().unsqueeze(-1) * freqs
    return ang.cos().repeat_interleave(2, dim=-1).contiguous(), ang.sin().repeat_interleave(2, dim=-1).contiguous()


def build_axial_rope_cos_sin_2d_continuous(x_pos, y_pos, head_dim: int, theta: float = 10000.0, device: Optional[torch.device] = None):
    if head_dim % 4:
        raise ValueError(f"head_dim={head_dim} must be divisible by 4 for axial 2D RoPE (half per axis, then adjacent pairs within each half).")
    cx, sx = build_rope_cos_sin_1d_continuous(x_pos, head_dim // 2, theta, device)
    cy, sy = build_rope_cos_sin_1d_continuous(y_pos, head_dim // 2, theta, device)
    return torch.cat([cx, cy], dim=-1), torch.cat([sx, sy], dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate adjacent channel pairs ``(x0, x1) -> (x0 c − x1 s, x1 c + x0 s)``; tables broadcast against ``x``."""
    pairs = x.reshape(*x.shape[:-1], -1, 2)
    rot = torch.stack((-pairs[..., 1], pairs[..., 0]), dim=-1).reshape(x.shape)
    return x * cos.to(x.dtype) + rot * sin.to(x.dtype)
