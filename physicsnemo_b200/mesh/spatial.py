"""Spatial queries on triangle meshes: bounding-volume hierarchy, closest point / signed distance, ray casting.

Parity: ``physicsnemo/mesh/spatial/{bvh,_lbvh,sdf}.py``.  The hierarchy is a complete binary tree over the
Morton-sorted triangles (leaves padded to a power of two), stored as flat ``[2·L − 1, 2, 3]`` bounds built bottom-up
with one min / max per level — every construction step is a tensor operation, so the build runs on any device.
Queries here are tensor formulations (all-pairs in chunks, used on CPU and as the oracle); the CUDA traversal
kernels live in the ``signed_distance_field`` / ``ray_mesh_intersect`` functionals.
"""
from __future__ import annotations

import torch

from .mesh import Mesh


def _expand_bits(v: torch.Tensor) -> torch.Tensor:
    v = (v | (v << 16)) & 0x030000FF
    v = (v | (v << 8)) & 0x0300F00F
    v = (v | (v << 4)) & 0x030C30C3
    return (v | (v << 2)) & 0x09249249


def morton_codes(points: torch.Tensor, lo: torch.Tensor, hi: torch.Tensor) -> torch.Tensor:
    q = ((points - lo) / (hi - lo).clamp_min(1e-30) * 1023.0).clamp(0, 1023).long()
    return (_expand_bits(q[:, 0]) << 2) | (_expand_bits(q[:, 1]) << 1) | _expand_bits(q[:, 2])


class BVH:
    """``order``: triangle index stored at every leaf (−1 for padding); ``bounds[node] = (min, max)``; children of
    node ``i`` are ``2i+1, 2i+2``; leaves start at ``n_leaves − 1``."""

    def __init__(self, vertices: torch.Tensor, faces: torch.Tensor):
        tri = vertices[faces]                                                  # [F, 3, 3]
        lo, hi = tri.amin(1), tri.amax(1)
        codes = morton_codes(tri.mean(1), vertices.amin(0), vertices.amax(0))
        order = torch.argsort(codes)
        F = faces.shape[0]
        L = 1 << max(F - 1, 0).bit_length() if F > 1 else 1
        pad = L - F
        big = torch.finfo(vertices.dtype).max
        leaf_lo = torch.cat([lo[order], lo.new_full((pad, 3), big)])
        leaf_hi = torch.cat([hi[order], hi.new_full((pad, 3), -big)])
        levels_lo, levels_hi = [leaf_lo], [leaf_hi]
        while levels_lo[0].shape[0] > 1:
            a, b = levels_lo[0], levels_hi[0]
            levels_lo.insert(0, torch.minimum(a[0::2], a[1::2]))
            levels_hi.insert(0, torch.maximum(b[0::2], b[1::2]))
        self.bounds = torch.stack([torch.cat(levels_lo), torch.cat(levels_hi)], dim=1).contiguous()
        self.order = torch.cat([order, order.new_full((pad,), -1)]).int().contiguous()
        self.n_leaves, self.n_faces = L, F
        self.triangles = tri.contiguous()


def closest_point_on_triangles(p: torch.Tensor, tri: torch.Tensor) -> torch.Tensor:
    """Closest point of triangles ``tri [..., 3, 3]`` to points ``p [..., 3]`` (Ericson's region tests, vectorised)."""
    a, b, c = tri[..., 0, :], tri[..., 1, :], tri[..., 2, :]
    ab, ac, ap = b - a, c - a, p - a
    d1, d2 = (ab * ap).sum(-1), (ac * ap).sum(-1)
    bp = p - b
    d3, d4 = (ab * bp).sum(-1), (ac * bp).sum(-1)
    cp = p - c
    d5, d6 = (ab * cp).sum(-1), (ac * cp).sum(-1)
    vc, vb, va = d1 * d4 - d3 * d2, d5 * d2 - d1 * d6, d3 * d6 - d5 * d4
    eps = 1e-30
    denom = (va + vb + vc).abs().clamp_min(eps) * torch.sign(va + vb + vc + eps)
    v, w = vb / denom, vc / denom
    res = a + ab * v[..., None] + ac * w[..., None]
    t_ab = (d1 / (d1 - d3).abs().clamp_min(eps) / torch.sign(d1 - d3 + eps))[..., None]
    t_ac = (d2 / (d2 - d6).abs().clamp_min(eps) / torch.sign(d2 - d6 + eps))[..., None]
    t_bc = ((d4 - d3) / ((d4 - d3) + (d5 - d6)).abs().clamp_min(eps) / torch.sign((d4 - d3) + (d5 - d6) + eps))[..., None]
    res = torch.where(((va <= 0) & (d4 - d3 >= 0) & (d5 - d6 >= 0))[..., None], b + (c - b) * t_bc, res)
    res = torch.where(((vb <= 0) & (d2 >= 0) & (d6 <= 0))[..., None], a + ac * t_ac, res)
    res = torch.where(((vc <= 0) & (d1 >= 0) & (d3 <= 0))[..., None], a + ab * t_ab, res)
    res = torch.where(((d6 >= 0) & (d5 <= d6))[..., None], c, res)
    res = torch.where(((d3 >= 0) & (d4 <= d3))[..., None], b, res)
    res = torch.where(((d1 <= 0) & (d2 <= 0))[..., None], a, res)
    return res


def winding_number(p: torch.Tensor, tri: torch.Tensor) -> torch.Tensor:
    """Generalised winding number of points ``p [N, 3]`` with respect to triangles ``tri [F, 3, 3]`` (solid angles)."""
    a, b, c = (tri[None, :, k] - p[:, None] for k in range(3))
    la, lb, lc = a.norm(dim=-1), b.norm(dim=-1), c.norm(dim=-1)
    num = (a * torch.linalg.cross(b, c)).sum(-1)
    den = la * lb * lc + (a * b).sum(-1) * lc + (b * c).sum(-1) * la + (c * a).sum(-1) * lb
    return (2 * torch.atan2(num, den)).sum(1) / (4 * torch.pi)


def closest_point_bruteforce(vertices, faces, queries, chunk: int = 2048):
    """(distance, closest point, face index) of every query, all pairs in chunks."""
    tri = vertices[faces]
    d_out, c_out, f_out = [], [], []
    for s in range(0, queries.shape[0], chunk):
        q = queries[s:s + chunk]
        cp = closest_point_on_triangles(q[:, None, :], tri[None])
        d2 = ((cp - q[:, None]) ** 2).sum(-1)
        best = d2.argmin(dim=1)
        rows = torch.arange(q.shape[0], device=q.device)
        d_out.append(d2[rows, best].clamp_min(0).sqrt()), c_out.append(cp[rows, best]), f_out.append(best)
    return torch.cat(d_out), torch.cat(c_out), torch.cat(f_out)


def ray_triangle_bruteforce(vertices, faces, origins, directions, chunk: int = 1024):
    """First hit of every ray (Möller–Trumbore): (t or inf, face index or −1, barycentric u, v)."""
    tri = vertices[faces]
    v0, e1, e2 = tri[:, 0], tri[:, 1] - tri[:, 0], tri[:, 2] - tri[:, 0]
    T, Fi, U, V = [], [], [], []
    for s in range(0, origins.shape[0], chunk):
        o, d = origins[s:s + chunk, None], directions[s:s + chunk, None]
        pv = torch.linalg.cross(d.expand(-1, tri.shape[0], -1), e2[None].expand(o.shape[0], -1, -1))
        det = (e1[None] * pv).sum(-1)
        ok = det.abs() > 1e-12
        inv = 1.0 / torch.where(ok, det, torch.ones_like(det))
        tv = o - v0[None]
        u = (tv * pv).sum(-1) * inv
        qv = torch.linalg.cross(tv, e1[None].expand_as(tv))
        v = (d * qv).sum(-1) * inv
        t = (e2[None] * qv).sum(-1) * inv
        hit = ok & (u >= 0) & (v >= 0) & (u + v <= 1) & (t > 1e-9)
        t = torch.where(hit, t, torch.full_like(t, float("inf")))
        best = t.argmin(dim=1)
        rows = torch.arange(o.shape[0], device=o.device)
        tb = t[rows, best]
        T.append(tb), Fi.append(torch.where(torch.isfinite(tb), best, torch.full_like(best, -1)))
        U.append(u[rows, best]), V.append(v[rows, best])
    return torch.cat(T), torch.cat(Fi), torch.cat(U), torch.cat(V)


def signed_distance(mesh: Mesh, queries: torch.Tensor, use_winding_number: bool = True):
    """Signed distance (negative inside) and closest points of ``queries`` to a closed triangle surface."""
    from ..nn.functional.geometry.sdf import signed_distance_field

    return signed_distance_field(mesh.points, mesh.cells, queries, use_sign_winding_number=use_winding_number)[:2]
