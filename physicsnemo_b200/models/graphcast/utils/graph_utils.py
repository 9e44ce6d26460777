"""Spherical geometry helpers of the GraphCast graphs.

Parity: ``physicsnemo/models/graphcast/utils/graph_utils.py`` (``latlon2xyz``, ``xyz2latlon``,
``geospatial_rotation``, ``azimuthal_angle``, ``polar_angle``, ``deg2rad`` / ``rad2deg``,
``cell_to_adj``, ``max_edge_length``, ``get_face_centroids``).  Array arguments are processed as
whole tensors (no per-face Python loops).
"""
from __future__ import annotations

import math

import numpy as np
import torch
from torch import Tensor


def deg2rad(deg):
    return deg * math.pi / 180


def rad2deg(rad):
    return rad * 180 / math.pi


def latlon2xyz(latlon: Tensor, radius: float = 1, unit: str = "deg") -> Tensor:
    if unit not in ("deg", "rad"):
        raise ValueError("Not a valid unit")
    if unit == "deg":
        latlon = deg2rad(latlon)
    lat, lon = latlon[:, 0], latlon[:, 1]
    return torch.stack((radius * torch.cos(lat) * torch.cos(lon), radius * torch.cos(lat) * torch.sin(lon),
                        radius * torch.sin(lat)), dim=1)


def xyz2latlon(xyz: Tensor, radius: float = 1, unit: str = "deg") -> Tensor:
    if unit not in ("deg", "rad"):
        raise ValueError("Not a valid unit")
    lat, lon = torch.arcsin(xyz[:, 2] / radius), torch.arctan2(xyz[:, 1], xyz[:, 0])
    return torch.stack((rad2deg(lat), rad2deg(lon)) if unit == "deg" else (lat, lon), dim=1)


def rotation_matrices(theta: Tensor, axis: str) -> Tensor:
    """``[N, 3, 3]`` right-handed rotations by ``theta`` about a coordinate axis."""
    c, s = torch.cos(theta), torch.sin(theta)
    o, z = torch.ones_like(c), torch.zeros_like(c)
    rows = {"x": (o, z, z, z, c, -s, z, s, c), "y": (c, z, s, z, o, z, -s, z, c), "z": (c, -s, z, s, c, z, z, z, o)}
    if axis not in rows:
        raise ValueError("Invalid axis")
    return torch.stack(rows[axis], dim=-1).reshape(-1, 3, 3)


def geospatial_rotation(invar: Tensor, theta: Tensor, axis: str, unit: str = "rad") -> Tensor:
    if unit not in ("deg", "rad"):
        raise ValueError("Not a valid unit")
    if unit == "deg":
        invar = rad2deg(invar)
    return torch.matmul(rotation_matrices(theta, axis).to(invar.dtype), invar.unsqueeze(-1)).squeeze(-1)


def azimuthal_angle(lon: Tensor) -> Tensor:
    return torch.where(lon >= 0.0, 2 * math.pi - lon, -lon)


def polar_angle(lat: Tensor) -> Tensor:
    return torch.where(lat >= 0.0, lat, 2 * math.pi + lat)


def cell_to_adj(cells):
    c = np.asarray(cells)
    return c[:, [0, 1, 2]].reshape(-1).tolist(), c[:, [1, 2, 0]].reshape(-1).tolist()


def max_edge_length(vertices, source_nodes, destination_nodes) -> float:
    v = np.asarray(vertices)
    return float(np.sqrt(((v[np.asarray(source_nodes)] - v[np.asarray(destination_nodes)]) ** 2).sum(1).max()))


def get_face_centroids(vertices, faces) -> np.ndarray:
    v = np.asarray(vertices)
    return v[np.asarray(faces)].mean(axis=1)
