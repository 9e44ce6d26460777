"""Blue-noise point sets on triangle surfaces: parallel dart throwing and weighted sample elimination.

Parity: ``physicsnemo/nn/functional/geometry/mesh_poisson_disk_sample/mesh_poisson_disk_sample.py``.

* ``dart_throwing`` — every iteration draws ``batch_size`` area-weighted candidates (uniform barycentric
  coordinates; the radius is ``min_distance`` or the barycentric interpolation of ``per_vertex_radius``), drops
  those closer than their radius to an accepted sample, lets conflicting candidates (closer than the smaller of
  the two radii) compete by random priority so that only local winners survive, and commits the winners.
* ``weighted_sample_elimination`` — draws an oversampled pool, then removes samples of largest weight
  ``Σ_j (1 − d̂_ij / 2 r_max)^8`` (``r_max = sqrt(A / (2√3 n))``, ``d̂`` clamped from below at
  ``r_min = r_max (1 − (n/m)^1.5)·0.65``) until ``target_num_points`` remain. The removal is done in rounds:
  every sample that carries the largest weight of its neighbourhood leaves at once and its contributions are
  subtracted from its neighbours, which keeps the greedy order locally and runs as a few tensor passes.

All pair searches are fixed-radius queries: the hash-grid kernel of ``radius_search`` on CUDA, a sort-based
cell hash in tensor operations on CPU; nothing ever forms an all-pairs distance matrix.
"""
from __future__ import annotations

import math
from typing import Sequence

import torch

from ....core.function_spec import FunctionSpec
from .sdf import _faces


def _pairs_within(a: torch.Tensor, b: torch.Tensor, radius: float, implementation=None):
    """All index pairs ``(i, j)`` with ``|a_i − b_j| <= radius`` as ``[2, P]``."""
    if a.shape[0] == 0 or b.shape[0] == 0:
        return torch.zeros(2, 0, dtype=torch.long, device=a.device)
    if a.is_cuda and implementation != "torch":
        from ..neighbors import radius_search

        return radius_search(b, a, radius, max_points=None).long()
    lo = torch.minimum(a.min(0).values, b.min(0).values)
    ca, cb = ((a - lo) / radius).floor().long(), ((b - lo) / radius).floor().long()
    dims = torch.maximum(ca.max(0).values, cb.max(0).values) + 3
    key = lambda c: ((c[:, 0] + 1) * dims[1] + (c[:, 1] + 1)) * dims[2] + (c[:, 2] + 1)  # noqa: E731
    kb, order = key(cb).sort()
    out_i, out_j = [], []
    for dx in (-1, 0, 1):
        for dy in (-1, 0, 1):
            # the three z-neighbours are contiguous in the key: one range lookup covers them
            k0 = key(ca + torch.tensor([dx, dy, -1], device=a.device))
            start, stop = torch.searchsorted(kb, k0), torch.searchsorted(kb, k0 + 2, right=True)
            cnt = stop - start
            if int(cnt.sum()) == 0:
                continue
            i = torch.repeat_interleave(torch.arange(a.shape[0], device=a.device), cnt)
            offs = torch.arange(i.shape[0], device=a.device) - torch.repeat_interleave(cnt.cumsum(0) - cnt, cnt)
            j = order[torch.repeat_interleave(start, cnt) + offs]
            keep = (a[i] - b[j]).square().sum(-1) <= radius * radius
            out_i.append(i[keep]); out_j.append(j[keep])
    if not out_i:
        return torch.zeros(2, 0, dtype=torch.long, device=a.device)
    return torch.stack((torch.cat(out_i), torch.cat(out_j)))


def _surface_candidates(v, faces, cdf, n, gen, per_vertex_radius, constant_radius):
    u = torch.rand(n, 3, generator=gen, device=v.device)
    f = torch.searchsorted(cdf, u[:, 0] * cdf[-1]).clamp_max(faces.shape[0] - 1)
    s = u[:, 1].sqrt()
    bary = torch.stack((1 - s, s * (1 - u[:, 2]), s * u[:, 2]), dim=-1)
    idx = faces[f]
    pos = (v[idx] * bary.unsqueeze(-1)).sum(1)
    rad = (per_vertex_radius[idx] * bary).sum(1) if per_vertex_radius is not None else torch.full((n,), constant_radius, device=v.device)
    return pos, rad


def _dart_throwing(v, faces, cdf, min_distance, per_vertex_radius, batch_size, max_points, max_iterations, gen, implementation):
    acc_p = torch.zeros(0, 3, device=v.device)
    acc_r = torch.zeros(0, device=v.device)
    r_search = float(per_vertex_radius.max()) if per_vertex_radius is not None else float(min_distance)
    for _ in range(max_iterations):
        if acc_p.shape[0] >= max_points:
            break
        pos, rad = _surface_candidates(v, faces, cdf, batch_size, gen, per_vertex_radius, min_distance)
        alive = torch.ones(batch_size, dtype=torch.bool, device=v.device)
        pr = _pairs_within(pos, acc_p, r_search, implementation)
        if pr.shape[1]:
            d = (pos[pr[0]] - acc_p[pr[1]]).norm(dim=-1)
            alive[pr[0][d < rad[pr[0]]]] = False                                # too close to an accepted sample
        ids = alive.nonzero().squeeze(1)
        cp, cr = pos[ids], rad[ids]
        prio = torch.rand(ids.shape[0], generator=gen, device=v.device)
        pr = _pairs_within(cp, cp, r_search, implementation)
        i, j = pr[0], pr[1]
        close = (i != j) & ((cp[i] - cp[j]).norm(dim=-1) < torch.minimum(cr[i], cr[j]))
        i, j = i[close], j[close]
        lose = (prio[j] > prio[i]) | ((prio[j] == prio[i]) & (j < i))           # a neighbour outranks me
        win = torch.ones(ids.shape[0], dtype=torch.bool, device=v.device)
        win[i[lose]] = False
        room = max_points - acc_p.shape[0]
        keep = win.nonzero().squeeze(1)[:room]
        if keep.numel() == 0 and ids.numel() == 0 and acc_p.shape[0]:
            break                                                               # surface is saturated
        acc_p, acc_r = torch.cat((acc_p, cp[keep])), torch.cat((acc_r, cr[keep]))
    return acc_p


def _sample_elimination(pool, target, area, implementation):
    m = pool.shape[0]
    if m <= target:
        return pool
    r_max = math.sqrt(area / (2.0 * math.sqrt(3.0) * target))
    r_min = r_max * (1.0 - (target / m) ** 1.5) * 0.65
    pr = _pairs_within(pool, pool, 2.0 * r_max, implementation)
    i, j = pr[0], pr[1]
    off = i != j
    i, j = i[off], j[off]
    d = (pool[i] - pool[j]).norm(dim=-1).clamp_min(r_min)
    w_ij = (1.0 - d / (2.0 * r_max)).clamp_min(0).pow(8)
    weight = torch.zeros(m, device=pool.device, dtype=w_ij.dtype).index_add_(0, i, w_ij)
    alive = torch.ones(m, dtype=torch.bool, device=pool.device)
    remaining = m
    while remaining > target:
        live = alive[i] & alive[j]
        neigh_max = torch.zeros(m, device=pool.device, dtype=weight.dtype).scatter_reduce_(0, i[live], weight[j[live]], "amax", include_self=True)
        peak = alive & (weight >= neigh_max)
        ties = live & peak[i] & peak[j] & (weight[i] == weight[j]) & (j < i)    # equal peaks: the lower index goes first
        peak[i[ties]] = False
        ids = peak.nonzero().squeeze(1)
        if ids.numel() > remaining - target:
            ids = ids[weight[ids].topk(remaining - target).indices]
        if ids.numel() == 0:
            ids = torch.where(alive, weight, weight.new_full((), -1.0)).argmax().reshape(1)
        gone = torch.zeros(m, dtype=torch.bool, device=pool.device)
        gone[ids] = True
        sel = live & gone[j]
        weight.index_add_(0, i[sel], -w_ij[sel])
        alive &= ~gone
        remaining -= int(ids.numel())
    return pool[alive]


class MeshPoissonDiskSample(FunctionSpec):
    @FunctionSpec.register(name="torch", rank=0, baseline=True)
    def torch_forward(mesh_vertices, mesh_indices, min_distance=0.02, per_vertex_radius=None, batch_size=131072,
                      max_points=2_000_000, max_iterations=64, random_seed=42, hash_grid_resolution=128,
                      mode="dart_throwing", target_num_points=None, implementation=None):
        if mesh_vertices.ndim != 2 or mesh_vertices.shape[-1] != 3:
            raise ValueError("mesh_vertices must have shape (n_vertices, 3)")
        if mode not in ("dart_throwing", "weighted_sample_elimination"):
            raise ValueError(f"mode must be 'dart_throwing' or 'weighted_sample_elimination', got {mode!r}")
        if min_distance <= 0:
            raise ValueError("min_distance must be strictly positive")
        if batch_size <= 0 or max_points <= 0 or max_iterations <= 0:
            raise ValueError("batch_size, max_points and max_iterations must be strictly positive")
        v = mesh_vertices.detach().float()
        faces = _faces(v, mesh_indices.to(v.device))
        if per_vertex_radius is not None:
            per_vertex_radius = per_vertex_radius.to(v).reshape(-1)
            if per_vertex_radius.shape[0] != v.shape[0]:
                raise ValueError("per_vertex_radius must have shape (n_vertices,)")
            if bool((per_vertex_radius <= 0).any()):
                raise ValueError("per_vertex_radius must be strictly positive")
        tri = v[faces]
        areas = 0.5 * torch.linalg.cross(tri[:, 1] - tri[:, 0], tri[:, 2] - tri[:, 0]).norm(dim=-1)
        if not bool((areas > 0).any()):
            raise ValueError("the mesh has no triangle of positive area")
        cdf = areas.double().cumsum(0).float()
        gen = torch.Generator(device=v.device).manual_seed(int(random_seed))
        if mode == "dart_throwing":
            return _dart_throwing(v, faces, cdf, float(min_distance), per_vertex_radius, int(batch_size), int(max_points),
                                  int(max_iterations), gen, implementation)
        target = int(target_num_points if target_num_points is not None else max_points)
        if target <= 0:
            raise ValueError("target_num_points must be strictly positive")
        area = float(areas.sum())
        # pool: a dart-throwing set at a radius that packs about five times the target count
        r_pool = max(math.sqrt(area / (2.0 * math.sqrt(3.0) * 5 * target)) * 0.75, 1e-12)
        pool = _dart_throwing(v, faces, cdf, r_pool, None, max(int(batch_size), 8 * target), 5 * target, int(max_iterations), gen, implementation)
        if pool.shape[0] < target:
            extra, _ = _surface_candidates(v, faces, cdf, target - pool.shape[0], gen, None, 0.0)
            pool = torch.cat((pool, extra))
        return _sample_elimination(pool, target, area, implementation)


mesh_poisson_disk_sample = MeshPoissonDiskSample.make_function("mesh_poisson_disk_sample")
