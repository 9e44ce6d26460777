"""Implicit-function helpers and isosurface extraction.

Parity: ``physicsnemo/mesh/generate/{implicit_functions,marching_cubes}.py`` (``sdf_sphere``, ``sdf_box``, ``sdf_union``,
``sdf_intersection``, ``sdf_difference``, ``project_to_zero_set``, ``marching_cubes(field, threshold, coords) -> Mesh``).

The isosurface is extracted by marching *tetrahedra* on the Kuhn subdivision of every grid cell (six tetrahedra around the
main diagonal, identical on shared faces), written as a tensor program: all tetrahedra are classified at once, edge
crossings are de-duplicated by their grid-edge key, so the surface is watertight and needs no lookup tables; it runs on
whatever device the field lives on.  Triangles are oriented with their normals towards increasing field values (outward
for a signed distance).
"""
from __future__ import annotations

import itertools
from typing import Callable, Sequence

import torch

from .mesh import Mesh

ImplicitFunction = Callable[[torch.Tensor], torch.Tensor]


def sdf_sphere(center, radius: float) -> ImplicitFunction:
    def phi(x):
        return (x - torch.as_tensor(center, dtype=x.dtype, device=x.device)).norm(dim=-1) - radius

    return phi


def sdf_box(lo, hi) -> ImplicitFunction:
    def phi(x):
        a, b = torch.as_tensor(lo, dtype=x.dtype, device=x.device), torch.as_tensor(hi, dtype=x.dtype, device=x.device)
        q = (x - 0.5 * (a + b)).abs() - 0.5 * (b - a)
        return q.clamp_min(0).norm(dim=-1) + q.amax(dim=-1).clamp_max(0)

    return phi


def sdf_union(*phis: ImplicitFunction) -> ImplicitFunction:
    return lambda x: torch.stack([p(x) for p in phis]).amin(0)


def sdf_intersection(*phis: ImplicitFunction) -> ImplicitFunction:
    return lambda x: torch.stack([p(x) for p in phis]).amax(0)


def sdf_difference(phi_a: ImplicitFunction, *phis_b: ImplicitFunction) -> ImplicitFunction:
    return lambda x: torch.stack([phi_a(x), *[-p(x) for p in phis_b]]).amax(0)


def project_to_zero_set(phi: ImplicitFunction, points: torch.Tensor, iterations: int = 10, tol: float = 1e-6) -> torch.Tensor:
    """Newton steps ``x ← x − φ ∇φ / |∇φ|²`` onto the zero level set (gradient by autograd)."""
    x = points.detach().clone()
    for _ in range(iterations):
        x.requires_grad_(True)
        with torch.enable_grad():
            val = phi(x)
            (g,) = torch.autograd.grad(val.sum(), x)
        x = (x - val.unsqueeze(-1) * g / g.square().sum(-1, keepdim=True).clamp_min(1e-30)).detach()
        if float(val.abs().max()) < tol:
            break
    return x


_KUHN = [[(0, 0, 0), tuple(int(k == p[0]) for k in range(3)), tuple(int(k in p[:2]) for k in range(3)), (1, 1, 1)]
         for p in itertools.permutations(range(3))]


def marching_cubes(field: torch.Tensor, threshold: float = 0.0, coords: Sequence[torch.Tensor] | None = None) -> Mesh:
    if field.ndim != 3:
        raise ValueError(f"field must have shape (nx, ny, nz), got {tuple(field.shape)}")
    if min(field.shape) < 2:
        raise ValueError("every grid dimension needs at least two nodes")
    dev = field.device
    f = field.float() - threshold
    nx, ny, nz = f.shape
    if coords is not None:
        if len(coords) != 3 or any(c.ndim != 1 or c.shape[0] != n for c, n in zip(coords, f.shape)):
            raise ValueError("coords must be three 1-D tensors of lengths nx, ny, nz")
        axes = [c.to(dev, torch.float32) for c in coords]
    else:
        axes = [torch.arange(n, device=dev, dtype=torch.float32) for n in f.shape]
    node_pos = torch.stack(torch.meshgrid(*axes, indexing="ij"), dim=-1).reshape(-1, 3)
    fv = f.reshape(-1)
    i, j, k = torch.meshgrid(torch.arange(nx - 1, device=dev), torch.arange(ny - 1, device=dev), torch.arange(nz - 1, device=dev), indexing="ij")
    base = ((i * ny + j) * nz + k).reshape(-1)
    corner = lambda d: base + (d[0] * ny + d[1]) * nz + d[2]  # noqa: E731
    tets = torch.cat([torch.stack([corner(d) for d in tet], dim=1) for tet in _KUHN], dim=0)            # [T, 4] node ids
    vals = fv[tets]
    inside = vals < 0
    n_in = inside.sum(1)
    crossing = (n_in > 0) & (n_in < 4)
    tets, vals, inside, n_in = tets[crossing], vals[crossing], inside[crossing], n_in[crossing]
    if tets.shape[0] == 0:
        return Mesh(torch.zeros(0, 3, device=dev), torch.zeros(0, 3, dtype=torch.long, device=dev))
    order = torch.argsort((~inside).to(torch.int8), dim=1, stable=True)                                  # inside vertices first
    v = torch.gather(tets, 1, order)
    a, b, c, d = v.unbind(1)
    tri_edges = []                                                                                       # (inside node, outside node) per corner
    m1, m3, m2 = n_in == 1, n_in == 3, n_in == 2
    tri_edges.append(torch.stack([torch.stack([a, b], -1), torch.stack([a, c], -1), torch.stack([a, d], -1)], 1)[m1])
    tri_edges.append(torch.stack([torch.stack([a, d], -1), torch.stack([b, d], -1), torch.stack([c, d], -1)], 1)[m3])
    ac, ad, bd, bc = torch.stack([a, c], -1), torch.stack([a, d], -1), torch.stack([b, d], -1), torch.stack([b, c], -1)
    tri_edges.append(torch.stack([ac, ad, bd], 1)[m2])
    tri_edges.append(torch.stack([ac, bd, bc], 1)[m2])
    E = torch.cat(tri_edges, 0)                                                                          # [F, 3, 2]
    lo, hi = E.amin(-1), E.amax(-1)
    keys, inv = torch.unique(lo.reshape(-1) * fv.shape[0] + hi.reshape(-1), return_inverse=True)
    p0, p1 = keys // fv.shape[0], keys % fv.shape[0]
    t = (fv[p0] / (fv[p0] - fv[p1])).clamp(0, 1).unsqueeze(1)
    points = node_pos[p0] * (1 - t) + node_pos[p1] * t
    cells = inv.reshape(-1, 3)
    tri = points[cells]
    normal = torch.linalg.cross(tri[:, 1] - tri[:, 0], tri[:, 2] - tri[:, 0])
    outward = node_pos[E[:, 0, 1]] - node_pos[E[:, 0, 0]]                                                # inside → outside node of one crossing
    flip = (normal * outward).sum(-1) < 0
    cells = torch.where(flip.unsqueeze(1), cells[:, [0, 2, 1]], cells)
    area2 = normal.norm(dim=-1)
    return Mesh(points, cells[area2 > 0].long())
