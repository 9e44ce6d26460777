"""Uniform / density-adapted surface remeshing by mass-weighted centroidal vertex clustering.

Parity: ``physicsnemo/nn/functional/geometry/remeshing/remeshing.py`` — ``remeshing(mesh_vertices, mesh_indices,
n_clusters, max_iterations=4, vertex_density=None, vertex_density_exponent=1.0, …) -> (vertices, indices)``: the
input vertices carry an integration mass (a third of the area of their incident triangles times
``density ** exponent``), are grouped into ``n_clusters`` clusters by Lloyd relaxation of mass-weighted centroids,
the centroids are projected onto the source surface, and the output triangles are the input triangles whose three
corners fall into three different clusters (deduplicated, orientation kept, unused clusters dropped). The result
is not differentiable. Clusters are seeded by farthest-point sampling up to ``farthest_point_threshold`` clusters
(from a mass-weighted candidate pool ``farthest_point_oversampling`` times larger) and by mass-weighted sampling
without replacement above it.

The nearest-centroid assignment is the 1-nearest-neighbour kernel on CUDA and the projection the BVH
closest-point kernel; both fall back to tensor operations on CPU. Work happens in float32 on coordinates centred
and scaled to the unit box, and the result is mapped back to the input frame and dtype.
"""
from __future__ import annotations

import torch

from ....core.function_spec import FunctionSpec
from ..neighbors import knn
from .farthest_point_sampling import farthest_point_sampling
from .sdf import signed_distance_field


def _validate(v, f, n_clusters, density, max_iterations):
    if not isinstance(v, torch.Tensor) or not isinstance(f, torch.Tensor):
        raise TypeError("mesh_vertices and mesh_indices must be torch.Tensors")
    if v.ndim != 2 or v.shape[1] != 3:
        raise ValueError("mesh_vertices must have shape (n_vertices, 3)")
    if f.ndim != 2 or f.shape[1] != 3:
        raise ValueError("mesh_indices must have shape (n_faces, 3)")
    if v.shape[0] < 3 or f.shape[0] < 1:
        raise ValueError("the mesh needs at least three vertices and one triangle")
    if not torch.is_floating_point(v):
        raise TypeError(f"mesh_vertices must use a floating-point dtype, got {v.dtype}")
    if torch.is_floating_point(f) or f.dtype == torch.bool:
        raise TypeError(f"mesh_indices must use an integer dtype, got {f.dtype}")
    if v.device != f.device:
        raise ValueError("mesh_vertices and mesh_indices must be on the same device")
    if isinstance(n_clusters, bool) or not isinstance(n_clusters, int):
        raise TypeError(f"n_clusters must be an integer, got {type(n_clusters).__name__}")
    if n_clusters < 3:
        raise ValueError(f"n_clusters must be at least 3, got {n_clusters}")
    if n_clusters > v.shape[0]:
        raise ValueError(f"n_clusters cannot exceed the input vertex count. Got n_clusters={n_clusters} and n_vertices={v.shape[0]}")
    if max_iterations < 0:
        raise ValueError("max_iterations must be non-negative")
    if density is not None:
        if not isinstance(density, torch.Tensor):
            raise TypeError("vertex_density must be a torch.Tensor or None")
        if density.ndim != 1 or density.shape[0] != v.shape[0]:
            raise ValueError(f"vertex_density must have shape (n_vertices,). Got {tuple(density.shape)} for n_vertices={v.shape[0]}")
        if not torch.is_floating_point(density):
            raise TypeError(f"vertex_density must use a real floating-point dtype, got {density.dtype}")
        if density.device != v.device:
            raise ValueError("vertex_density and mesh_vertices must be on the same device")
        if not bool((torch.isfinite(density) & (density > 0)).all()):
            raise ValueError("vertex_density must be finite and strictly positive")
    if int(f.min()) < 0 or int(f.max()) >= v.shape[0]:
        raise ValueError("mesh_indices must index existing vertices")
    if not bool(torch.isfinite(v).all()):
        raise ValueError("mesh_vertices must be finite")


def cluster_surface_vertices(x, mass, n_clusters, max_iterations, fps_threshold, fps_oversampling, generator):
    """Lloyd relaxation of mass-weighted centroids; returns ``(centroids [K, 3], labels [V])``."""
    V = x.shape[0]
    p = (mass / mass.sum()).double()
    if n_clusters <= fps_threshold:
        pool = min(V, max(n_clusters, fps_oversampling * n_clusters))
        cand = torch.multinomial(p, pool, replacement=False, generator=generator) if pool < V else torch.arange(V, device=x.device)
        pick = farthest_point_sampling(x[cand].unsqueeze(0), n_clusters)
        pick = pick[0] if isinstance(pick, (tuple, list)) else pick
        seeds = cand[pick.reshape(-1).long()]
    else:
        seeds = torch.multinomial(p, n_clusters, replacement=False, generator=generator)
    c = x[seeds].clone()
    labels = None
    for it in range(max_iterations + 1):
        labels = knn(c, x, 1)[0].reshape(-1).long()
        if it == max_iterations:
            break
        msum = torch.zeros(n_clusters, device=x.device).index_add_(0, labels, mass)
        csum = torch.zeros(n_clusters, 3, device=x.device).index_add_(0, labels, x * mass.unsqueeze(1))
        filled = msum > 0
        new_c = torch.where(filled.unsqueeze(1), csum / msum.clamp_min(1e-30).unsqueeze(1), c)
        if torch.allclose(new_c, c, atol=1e-7, rtol=0):
            c = new_c
            labels = knn(c, x, 1)[0].reshape(-1).long()
            break
        c = new_c
    return c, labels


class Remeshing(FunctionSpec):
    @FunctionSpec.register(name="torch", rank=0, baseline=True)
    def torch_forward(mesh_vertices, mesh_indices, n_clusters, *, max_iterations=4, vertex_density=None,
                      vertex_density_exponent=1.0, search_radius_scale=1.6, voxel_width_scale=1.15, hash_grid_resolution=128,
                      farthest_point_threshold=256, farthest_point_oversampling=4):
        _validate(mesh_vertices, mesh_indices, n_clusters, vertex_density, max_iterations)
        if search_radius_scale <= 0 or voxel_width_scale <= 0:
            raise ValueError("search_radius_scale and voxel_width_scale must be strictly positive")
        if not 0 < hash_grid_resolution <= 256:
            raise ValueError("hash_grid_resolution must be in [1, 256]")
        if farthest_point_threshold < 0 or farthest_point_oversampling < 1:
            raise ValueError("farthest_point_threshold must be >= 0 and farthest_point_oversampling >= 1")
        with torch.no_grad():
            f = mesh_indices.long()
            centre = 0.5 * (mesh_vertices.min(0).values + mesh_vertices.max(0).values)
            scale = (mesh_vertices.max(0).values - mesh_vertices.min(0).values).max().clamp_min(torch.finfo(mesh_vertices.dtype).tiny)
            x = ((mesh_vertices - centre) / scale).float()
            tri = x[f]
            area = 0.5 * torch.linalg.cross(tri[:, 1] - tri[:, 0], tri[:, 2] - tri[:, 0]).norm(dim=-1)
            if not bool((area.sum() > 0) & torch.isfinite(area.sum())):
                raise ValueError("the surface has no area")
            mass = torch.zeros(x.shape[0], device=x.device).index_add_(0, f.reshape(-1), (area / 3).repeat_interleave(3))
            if vertex_density is not None:
                mass = mass * vertex_density.float().pow(vertex_density_exponent)
            used = mass > 0
            gen = torch.Generator(device=x.device).manual_seed(0)
            ids = used.nonzero().squeeze(1)
            if ids.numel() < n_clusters:
                raise ValueError("n_clusters exceeds the number of vertices that belong to a triangle of positive area")
            c, lab_used = cluster_surface_vertices(x[ids], mass[ids], n_clusters, int(max_iterations), int(farthest_point_threshold),
                                                   int(farthest_point_oversampling), gen)
            labels = torch.full((x.shape[0],), -1, dtype=torch.long, device=x.device)
            labels[ids] = lab_used
            _, on_surface, _ = signed_distance_field(x, f, c)
            c = torch.where(torch.isfinite(on_surface), on_surface, c)
            t = labels[f]
            t = t[(t >= 0).all(1) & (t[:, 0] != t[:, 1]) & (t[:, 1] != t[:, 2]) & (t[:, 0] != t[:, 2])]
            if t.shape[0] == 0:
                raise RuntimeError("remeshing could not reconstruct a nonempty surface; lower n_clusters or refine the input")
            first = t.argmin(dim=1, keepdim=True)                                # rotate the smallest label to the front
            t = torch.gather(t, 1, (first + torch.arange(3, device=t.device)) % 3)
            t = torch.unique(t, dim=0)
            keep = torch.unique(t)
            remap = torch.full((n_clusters,), -1, dtype=torch.long, device=x.device)
            remap[keep] = torch.arange(keep.numel(), device=x.device)
            out_v = (c[keep].to(mesh_vertices.dtype) * scale + centre)
            return out_v, remap[t]


remeshing = Remeshing.make_function("remeshing")
