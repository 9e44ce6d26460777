"""Monte-Carlo volume fraction of a triangle mesh on a voxel grid.

Parity: ``physicsnemo/nn/functional/geometry/mesh_to_voxel_fraction/mesh_to_voxel_fraction.py`` — voxels that no
triangle can touch take the inside/outside class of their centre, the others the mean of ``n_samples`` uniformly
placed inside tests; output ``[nz, ny, nx]`` float32, flat index ``i + j·nx + k·nx·ny``; points farther than
``voxel_size · max(grid_dims)`` from the surface count as outside; ``open_mesh`` classifies by generalized winding
number against ``winding_number_threshold``.

Two passes over the BVH closest-point kernel (``csrc/bvh.cu``) on CUDA, the brute-force search on CPU: pass one
queries every voxel centre with the search radius capped at the voxel half-diagonal — a centre farther than that
from the surface owns a voxel no triangle intersects — and pass two queries only the samples of the surface band,
so the work scales with the surface area in voxels, not with the grid volume. The sample positions come from a
counter-based hash of ``(seed + voxel index, sample)``, which makes the result independent of the launch order.
"""
from __future__ import annotations

from typing import Sequence

import torch

from ....core.function_spec import FunctionSpec
from .sdf import _faces, signed_distance_field


def _hash_uniform(voxel: torch.Tensor, n_samples: int, seed: int) -> torch.Tensor:
    """Uniform numbers ``[V, n_samples, 3]`` in [0, 1) from an integer hash of (seed + voxel, sample, axis)."""
    key = (voxel.long() + seed)[:, None, None] * 0x9E3779B1 + torch.arange(n_samples * 3, device=voxel.device).reshape(1, n_samples, 3) * 0x85EBCA77
    x = key & 0xFFFFFFFF
    for mul in (0x7FEB352D, 0x846CA68B):                       # two xorshift-multiply rounds on 32 bits
        x = ((x ^ (x >> 16)) * mul) & 0xFFFFFFFF
    x = x ^ (x >> 16)
    return (x >> 8).to(torch.float32) * (1.0 / (1 << 24))


def _inside(vertices, faces, pts, max_dist, open_mesh, threshold, implementation):
    if pts.shape[0] == 0:
        return torch.zeros(0, dtype=torch.bool, device=pts.device)
    if open_mesh:
        if pts.is_cuda and implementation != "torch":
            from .sdf import _winding_cuda

            wn = _winding_cuda(vertices, faces, pts)
        else:
            from ....mesh.spatial import winding_number

            tri = vertices[faces]
            wn = torch.cat([winding_number(pts[s:s + 4096], tri) for s in range(0, pts.shape[0], 4096)])
        d, _, _ = signed_distance_field(vertices, faces, pts, max_dist=max_dist, implementation=implementation)
        return (wn > threshold) & torch.isfinite(d)
    d, _, _ = signed_distance_field(vertices, faces, pts, max_dist=max_dist, implementation=implementation)
    return d < 0                                                # NaN (beyond max_dist) compares false: outside


class MeshToVoxelFraction(FunctionSpec):
    @staticmethod
    def _run(mesh_vertices, mesh_indices, origin, voxel_size, grid_dims, n_samples, seed, open_mesh,
             winding_number_threshold, winding_number_accuracy, implementation):
        if mesh_vertices.ndim != 2 or mesh_vertices.shape[-1] != 3:
            raise ValueError("mesh_vertices must have shape (n_vertices, 3)")
        if voxel_size <= 0.0:
            raise ValueError("voxel_size must be strictly positive")
        dims = [int(d) for d in (grid_dims.tolist() if isinstance(grid_dims, torch.Tensor) else grid_dims)]
        if len(dims) != 3 or min(dims) <= 0:
            raise ValueError("grid_dims must be three strictly positive integers (nx, ny, nz)")
        if n_samples <= 0:
            raise ValueError("n_samples must be strictly positive")
        if winding_number_accuracy <= 0.0:
            raise ValueError("winding_number_accuracy must be strictly positive")
        nx, ny, nz = dims
        dev = mesh_vertices.device
        v = mesh_vertices.detach().float().contiguous()
        faces = _faces(v, mesh_indices.to(dev))
        o = torch.as_tensor(origin, dtype=torch.float32, device=dev).reshape(3)
        h = float(voxel_size)
        k, j, i = torch.meshgrid(torch.arange(nz, device=dev), torch.arange(ny, device=dev), torch.arange(nx, device=dev), indexing="ij")
        low = o + torch.stack((i, j, k), dim=-1).reshape(-1, 3).float() * h
        max_dist = h * max(dims)
        centre = low + 0.5 * h
        d, _, _ = signed_distance_field(v, faces, centre, max_dist=max_dist, implementation=implementation)
        band = (d.abs() <= 0.5 * 3 ** 0.5 * h * (1 + 1e-5)).nonzero().squeeze(1)
        if open_mesh:
            out = _inside(v, faces, centre, max_dist, True, winding_number_threshold, implementation).float()
        else:
            out = (d < 0).float()
        if band.numel():
            u = _hash_uniform(band, n_samples, seed)
            samples = (low[band][:, None, :] + u * h).reshape(-1, 3)
            inside = _inside(v, faces, samples, max_dist, open_mesh, winding_number_threshold, implementation)
            out[band] = inside.reshape(-1, n_samples).float().mean(dim=1)
        return out.reshape(nz, ny, nx)

    @FunctionSpec.register(name="cuda", rank=0, device_types=("cuda",))
    def cuda_forward(mesh_vertices, mesh_indices, origin, voxel_size, grid_dims, n_samples=64, seed=42, open_mesh=False,
                     winding_number_threshold=0.5, winding_number_accuracy=2.0):
        return MeshToVoxelFraction._run(mesh_vertices, mesh_indices, origin, voxel_size, grid_dims, n_samples, seed, open_mesh,
                                        winding_number_threshold, winding_number_accuracy, "cuda")

    @FunctionSpec.register(name="torch", rank=1, baseline=True)
    def torch_forward(mesh_vertices, mesh_indices, origin, voxel_size, grid_dims, n_samples=64, seed=42, open_mesh=False,
                      winding_number_threshold=0.5, winding_number_accuracy=2.0):
        return MeshToVoxelFraction._run(mesh_vertices, mesh_indices, origin, voxel_size, grid_dims, n_samples, seed, open_mesh,
                                        winding_number_threshold, winding_number_accuracy, "torch")


mesh_to_voxel_fraction = MeshToVoxelFraction.make_function("mesh_to_voxel_fraction")
