"""Mesh generators.

Parity: ``physicsnemo/mesh/primitives`` (basic simplices, curves, planar regions, surfaces, volumes, procedural
noise).  Every generator returns a ``Mesh``; resolutions are counts of segments.
"""
from __future__ import annotations

import math

import torch

from .mesh import Mesh


# --------------------------------------------------------------------- basic
def single_point(dim: int = 3) -> Mesh:
    return Mesh(torch.zeros(1, dim))


def single_edge(dim: int = 3) -> Mesh:
    p = torch.zeros(2, dim)
    p[1, 0] = 1.0
    return Mesh(p, torch.tensor([[0, 1]]))


def single_triangle(dim: int = 3) -> Mesh:
    p = torch.zeros(3, dim)
    p[1, 0] = 1.0
    p[2, 1] = 1.0
    return Mesh(p, torch.tensor([[0, 1, 2]]))


def single_tetrahedron() -> Mesh:
    return Mesh(torch.tensor([[0.0, 0, 0], [1, 0, 0], [0, 1, 0], [0, 0, 1]]), torch.tensor([[0, 1, 2, 3]]))


def two_triangles(dim: int = 3) -> Mesh:
    p = torch.zeros(4, dim)
    p[1, 0] = p[2, 0] = p[2, 1] = p[3, 1] = 1.0
    return Mesh(p, torch.tensor([[0, 1, 2], [0, 2, 3]]))


def two_tetrahedra() -> Mesh:
    return Mesh(torch.tensor([[0.0, 0, 0], [1, 0, 0], [0, 1, 0], [0, 0, 1], [1, 1, 1]]), torch.tensor([[0, 1, 2, 3], [1, 2, 3, 4]]))


# -------------------------------------------------------------------- curves
def polyline(points: torch.Tensor, closed: bool = False) -> Mesh:
    n = points.shape[0]
    idx = torch.arange(n)
    cells = torch.stack([idx[:-1], idx[1:]], 1)
    if closed:
        cells = torch.cat([cells, torch.tensor([[n - 1, 0]])])
    return Mesh(points, cells)


def straight_line(n_segments: int = 10, dim: int = 2, length: float = 1.0) -> Mesh:
    p = torch.zeros(n_segments + 1, dim)
    p[:, 0] = torch.linspace(0, length, n_segments + 1)
    return polyline(p)


def circle(n_segments: int = 64, radius: float = 1.0, dim: int = 2) -> Mesh:
    t = torch.arange(n_segments) * (2 * math.pi / n_segments)
    p = torch.zeros(n_segments, dim)
    p[:, 0], p[:, 1] = radius * torch.cos(t), radius * torch.sin(t)
    return polyline(p, closed=True)


def ellipse(n_segments: int = 64, a: float = 2.0, b: float = 1.0) -> Mesh:
    m = circle(n_segments, 1.0)
    return m.scale(torch.tensor([a, b]))


def helix(n_segments: int = 128, radius: float = 1.0, pitch: float = 0.5, turns: float = 3.0) -> Mesh:
    t = torch.linspace(0, 2 * math.pi * turns, n_segments + 1)
    return polyline(torch.stack([radius * torch.cos(t), radius * torch.sin(t), pitch * t / (2 * math.pi)], 1))


def spiral(n_segments: int = 128, turns: float = 3.0, growth: float = 0.2) -> Mesh:
    t = torch.linspace(0, 2 * math.pi * turns, n_segments + 1)
    r = growth * t
    return polyline(torch.stack([r * torch.cos(t), r * torch.sin(t)], 1))


def trefoil_knot(n_segments: int = 200) -> Mesh:
    t = torch.arange(n_segments) * (2 * math.pi / n_segments)
    p = torch.stack([torch.sin(t) + 2 * torch.sin(2 * t), torch.cos(t) - 2 * torch.cos(2 * t), -torch.sin(3 * t)], 1)
    return polyline(p, closed=True)


# -------------------------------------------------------------------- planar
def structured_grid(nx: int = 10, ny: int = 10, x_range=(0.0, 1.0), y_range=(0.0, 1.0), dim: int = 2) -> Mesh:
    """Rectangle split into ``2·nx·ny`` triangles."""
    xs, ys = torch.linspace(*x_range, nx + 1), torch.linspace(*y_range, ny + 1)
    X, Y = torch.meshgrid(xs, ys, indexing="ij")
    p = torch.zeros((nx + 1) * (ny + 1), dim)
    p[:, 0], p[:, 1] = X.reshape(-1), Y.reshape(-1)
    i, j = torch.meshgrid(torch.arange(nx), torch.arange(ny), indexing="ij")
    a = (i * (ny + 1) + j).reshape(-1)
    b, c, d = a + (ny + 1), a + (ny + 1) + 1, a + 1
    return Mesh(p, torch.cat([torch.stack([a, b, c], 1), torch.stack([a, c, d], 1)]))


def unit_square(n: int = 10) -> Mesh:
    return structured_grid(n, n)


def rectangle(width: float = 2.0, height: float = 1.0, nx: int = 20, ny: int = 10) -> Mesh:
    return structured_grid(nx, ny, (0, width), (0, height))


def disk(n_radial: int = 8, n_angular: int = 32, radius: float = 1.0, inner_radius: float = 0.0) -> Mesh:
    """Disk (``inner_radius = 0``) or annulus as triangle fan rings."""
    if inner_radius > 0:
        r = torch.linspace(inner_radius, radius, n_radial + 1)
        t = torch.arange(n_angular) * (2 * math.pi / n_angular)
        R, T = torch.meshgrid(r, t, indexing="ij")
        p = torch.stack([(R * torch.cos(T)).reshape(-1), (R * torch.sin(T)).reshape(-1)], 1)
        i, j = torch.meshgrid(torch.arange(n_radial), torch.arange(n_angular), indexing="ij")
        a = (i * n_angular + j).reshape(-1)
        b = (i * n_angular + (j + 1) % n_angular).reshape(-1)
        c, d = b + n_angular, a + n_angular
        return Mesh(p, torch.cat([torch.stack([a, d, c], 1), torch.stack([a, c, b], 1)]))
    r = torch.linspace(0, radius, n_radial + 1)[1:]
    t = torch.arange(n_angular) * (2 * math.pi / n_angular)
    R, T = torch.meshgrid(r, t, indexing="ij")
    p = torch.cat([torch.zeros(1, 2), torch.stack([(R * torch.cos(T)).reshape(-1), (R * torch.sin(T)).reshape(-1)], 1)])
    j = torch.arange(n_angular)
    cells = [torch.stack([torch.zeros_like(j), 1 + j, 1 + (j + 1) % n_angular], 1)]
    for i in range(n_radial - 1):
        a, b = 1 + i * n_angular + j, 1 + i * n_angular + (j + 1) % n_angular
        cells += [torch.stack([a, a + n_angular, b + n_angular], 1), torch.stack([a, b + n_angular, b], 1)]
    return Mesh(p, torch.cat(cells))


def regular_polygon(n_sides: int = 6, radius: float = 1.0) -> Mesh:
    return disk(1, n_sides, radius)


def l_shape(n: int = 8) -> Mesh:
    full = structured_grid(2 * n, 2 * n, (0, 2), (0, 2))
    keep = ~((full.cell_centroids[:, 0] > 1) & (full.cell_centroids[:, 1] > 1))
    return full.slice_cells(keep).clean(merge_points=False)


# ------------------------------------------------------------------ surfaces
def icosphere(subdivisions: int = 2, radius: float = 1.0) -> Mesh:
    t = (1 + math.sqrt(5)) / 2
    p = torch.tensor([[-1, t, 0], [1, t, 0], [-1, -t, 0], [1, -t, 0], [0, -1, t], [0, 1, t], [0, -1, -t], [0, 1, -t],
                      [t, 0, -1], [t, 0, 1], [-t, 0, -1], [-t, 0, 1]], dtype=torch.float32)
    f = torch.tensor([[0, 11, 5], [0, 5, 1], [0, 1, 7], [0, 7, 10], [0, 10, 11], [1, 5, 9], [5, 11, 4], [11, 10, 2], [10, 7, 6],
                      [7, 1, 8], [3, 9, 4], [3, 4, 2], [3, 2, 6], [3, 6, 8], [3, 8, 9], [4, 9, 5], [2, 4, 11], [6, 2, 10],
                      [8, 6, 7], [9, 8, 1]])
    m = Mesh(p / p.norm(dim=1, keepdim=True), f)
    for _ in range(subdivisions):
        m = m.subdivide(1)
        m = m._with_points(m.points / m.points.norm(dim=1, keepdim=True))
    return m._with_points(m.points * radius)


def uv_sphere(n_lat: int = 16, n_lon: int = 32, radius: float = 1.0) -> Mesh:
    th = torch.linspace(0, math.pi, n_lat + 1)[1:-1]
    ph = torch.arange(n_lon) * (2 * math.pi / n_lon)
    T, P = torch.meshgrid(th, ph, indexing="ij")
    ring = torch.stack([torch.sin(T) * torch.cos(P), torch.sin(T) * torch.sin(P), torch.cos(T)], -1).reshape(-1, 3)
    p = torch.cat([torch.tensor([[0.0, 0, 1]]), ring, torch.tensor([[0.0, 0, -1]])]) * radius
    j = torch.arange(n_lon)
    last = p.shape[0] - 1
    cells = [torch.stack([torch.zeros_like(j), 1 + j, 1 + (j + 1) % n_lon], 1)]
    for i in range(n_lat - 2):
        a, b = 1 + i * n_lon + j, 1 + i * n_lon + (j + 1) % n_lon
        cells += [torch.stack([a, a + n_lon, b + n_lon], 1), torch.stack([a, b + n_lon, b], 1)]
    base = 1 + (n_lat - 2) * n_lon
    cells.append(torch.stack([base + j, torch.full_like(j, last), base + (j + 1) % n_lon], 1))
    return Mesh(p, torch.cat(cells))


def torus(n_major: int = 32, n_minor: int = 16, major_radius: float = 1.0, minor_radius: float = 0.3) -> Mesh:
    u = torch.arange(n_major) * (2 * math.pi / n_major)
    v = torch.arange(n_minor) * (2 * math.pi / n_minor)
    U, V = torch.meshgrid(u, v, indexing="ij")
    r = major_radius + minor_radius * torch.cos(V)
    p = torch.stack([r * torch.cos(U), r * torch.sin(U), minor_radius * torch.sin(V)], -1).reshape(-1, 3)
    i, j = torch.meshgrid(torch.arange(n_major), torch.arange(n_minor), indexing="ij")
    a = (i * n_minor + j).reshape(-1)
    b = (((i + 1) % n_major) * n_minor + j).reshape(-1)
    c = (((i + 1) % n_major) * n_minor + (j + 1) % n_minor).reshape(-1)
    d = (i * n_minor + (j + 1) % n_minor).reshape(-1)
    return Mesh(p, torch.cat([torch.stack([a, b, c], 1), torch.stack([a, c, d], 1)]))


def cylinder(n_angular: int = 32, n_height: int = 8, radius: float = 1.0, height: float = 2.0, capped: bool = True) -> Mesh:
    t = torch.arange(n_angular) * (2 * math.pi / n_angular)
    z = torch.linspace(-height / 2, height / 2, n_height + 1)
    Z, T = torch.meshgrid(z, t, indexing="ij")
    p = torch.stack([radius * torch.cos(T), radius * torch.sin(T), Z], -1).reshape(-1, 3)
    i, j = torch.meshgrid(torch.arange(n_height), torch.arange(n_angular), indexing="ij")
    a = (i * n_angular + j).reshape(-1)
    b = (i * n_angular + (j + 1) % n_angular).reshape(-1)
    c, d = b + n_angular, a + n_angular
    cells = [torch.stack([a, b, c], 1), torch.stack([a, c, d], 1)]
    if capped:
        lo, hi = p.shape[0], p.shape[0] + 1
        p = torch.cat([p, torch.tensor([[0, 0, -height / 2], [0, 0, height / 2]])])
        jj = torch.arange(n_angular)
        top = n_height * n_angular
        cells += [torch.stack([torch.full_like(jj, lo), (jj + 1) % n_angular, jj], 1),
                  torch.stack([torch.full_like(jj, hi), top + jj, top + (jj + 1) % n_angular], 1)]
    return Mesh(p, torch.cat(cells))


def cube_surface(n: int = 4, size: float = 1.0) -> Mesh:
    """Closed box surface, outward-oriented, with shared edges welded."""
    face = structured_grid(n, n, (-0.5, 0.5), (-0.5, 0.5), dim=3)
    half = torch.tensor([0, 0, 0.5])
    parts = []
    for axis in range(3):
        for sign in (1, -1):
            f = face.translate(half)
            pts = f.points.clone()
            if axis == 0:
                pts = pts[:, [2, 0, 1]]
            elif axis == 1:
                pts = pts[:, [1, 2, 0]]
            cells = f.cells
            if sign < 0:                       # point reflection reverses orientation: restore outward winding
                pts, cells = -pts, cells.flip(1)
            parts.append(Mesh(pts * size, cells))
    return Mesh.merge(parts).clean(tolerance=1e-6 * size)


def plane(nx: int = 10, ny: int = 10, size: float = 1.0) -> Mesh:
    return structured_grid(nx, ny, (-size / 2, size / 2), (-size / 2, size / 2), dim=3)


# ------------------------------------------------------------------- volumes
def box_volume(nx: int = 4, ny: int = 4, nz: int = 4, bounds=((0.0, 1.0), (0.0, 1.0), (0.0, 1.0))) -> Mesh:
    """Box filled with ``6·nx·ny·nz`` tetrahedra (Kuhn subdivision of every hexahedron: conforming)."""
    axes = [torch.linspace(lo, hi, n + 1) for (lo, hi), n in zip(bounds, (nx, ny, nz))]
    X, Y, Z = torch.meshgrid(*axes, indexing="ij")
    p = torch.stack([X.reshape(-1), Y.reshape(-1), Z.reshape(-1)], 1)
    i, j, k = torch.meshgrid(torch.arange(nx), torch.arange(ny), torch.arange(nz), indexing="ij")
    sy, sx = nz + 1, (ny + 1) * (nz + 1)
    base = (i * sx + j * sy + k).reshape(-1)
    corner = lambda dx, dy, dz: base + dx * sx + dy * sy + dz  # noqa: E731
    tets = []
    from itertools import permutations

    for perm in permutations(range(3)):
        verts = [(0, 0, 0)]
        cur = [0, 0, 0]
        for ax in perm:
            cur = list(cur)
            cur[ax] = 1
            verts.append(tuple(cur))
        tets.append(torch.stack([corner(*v) for v in verts], 1))
    cells = torch.cat(tets)
    m = Mesh(p, cells)
    neg = torch.linalg.det(m.points[m.cells[:, 1:]] - m.points[m.cells[:, :1]]) < 0
    cells = torch.where(neg[:, None], cells[:, [0, 2, 1, 3]], cells)
    return Mesh(p, cells)


def ball_volume(subdivisions: int = 2, radius: float = 1.0) -> Mesh:
    """Tetrahedra fanning from the centre to an icosphere."""
    s = icosphere(subdivisions, radius)
    p = torch.cat([s.points, torch.zeros(1, 3)])
    c = torch.cat([s.cells, torch.full((s.n_cells, 1), s.n_points)], 1)
    return Mesh(p, c)


# ---------------------------------------------------------------- procedural
def perturb(mesh: Mesh, amplitude: float = 0.05, generator=None, fix_boundary: bool = True) -> Mesh:
    noise = torch.randn(mesh.points.shape, generator=generator) * amplitude
    if fix_boundary and mesh.n_cells and mesh.n_manifold_dims >= 1:
        b = mesh.get_boundary_mesh(data_source="none").cells.reshape(-1)
        noise[b] = 0
    return mesh._with_points(mesh.points + noise.to(mesh.points))


def lumpy_sphere(subdivisions: int = 3, amplitude: float = 0.2, n_modes: int = 6, generator=None) -> Mesh:
    s = icosphere(subdivisions)
    dirs = torch.randn(n_modes, 3, generator=generator)
    dirs = dirs / dirs.norm(dim=1, keepdim=True)
    amp = torch.rand(n_modes, generator=generator) * amplitude
    bump = (amp[None] * torch.cos(3.0 * s.points @ dirs.T)).sum(1)
    return s._with_points(s.points * (1 + bump)[:, None])


# ------------------------------------------------- further basic shapes, curves
def three_points(dim: int = 3) -> Mesh:
    """Three isolated points (a 0-manifold)."""
    p = torch.zeros(3, dim)
    p[1, 0], p[2, min(1, dim - 1)] = 1.0, 1.0
    return Mesh(p, torch.arange(3)[:, None])


def three_edges(dim: int = 3) -> Mesh:
    """An open chain of three unit-ish segments that bends in the plane."""
    xy = torch.tensor([[0.0, 0.0], [1.0, 0.0], [1.5, 0.8], [2.5, 1.0]])
    return polyline(torch.nn.functional.pad(xy, (0, dim - 2)))


def line_segments_1d(n_segments: int = 8, x_range=(0.0, 1.0)) -> Mesh:
    """A partition of an interval: 1-manifold in one spatial dimension."""
    return polyline(torch.linspace(x_range[0], x_range[1], n_segments + 1)[:, None])


def circular_arc(n_segments: int = 32, radius: float = 1.0, start_angle: float = 0.0, end_angle: float = math.pi / 2) -> Mesh:
    a = torch.linspace(start_angle, end_angle, n_segments + 1)
    return polyline(radius * torch.stack([a.cos(), a.sin()], 1))


def spline(control_points: torch.Tensor | None = None, n_segments: int = 64, closed: bool = False) -> Mesh:
    """Catmull–Rom curve through the control points (default: a 3-D zig-zag), sampled uniformly in parameter."""
    if control_points is None:
        control_points = torch.tensor([[0.0, 0, 0], [1, 1, 0], [2, 0, 1], [3, 1, 1], [4, 0, 0]])
    c = torch.as_tensor(control_points, dtype=torch.float32)
    n = c.shape[0]
    if n < 2:
        raise ValueError("a spline needs at least two control points")
    spans = n if closed else n - 1
    t = torch.linspace(0, spans, n_segments + (0 if closed else 1) + (1 if closed else 0))[: n_segments + (0 if closed else 1)]
    i = t.floor().clamp(max=spans - 1).long()
    u = (t - i)[:, None]

    def pick(k):
        return c[(i + k) % n] if closed else c[(i + k).clamp(0, n - 1)]

    p0, p1, p2, p3 = pick(-1), pick(0), pick(1), pick(2)
    pts = 0.5 * (2 * p1 + (p2 - p0) * u + (2 * p0 - 5 * p1 + 4 * p2 - p3) * u ** 2 + (3 * p1 - p0 - 3 * p2 + p3) * u ** 3)
    return polyline(pts, closed=closed)


# ------------------------------------------------------ further planar regions
def annulus(n_radial: int = 4, n_angular: int = 32, inner_radius: float = 0.5, outer_radius: float = 1.0) -> Mesh:
    return disk(n_radial=n_radial, n_angular=n_angular, radius=outer_radius, inner_radius=inner_radius)


def equilateral_triangle(side: float = 1.0, subdivisions: int = 0) -> Mesh:
    p = torch.tensor([[0.0, 0.0], [side, 0.0], [side / 2, side * math.sqrt(3) / 2]])
    m = Mesh(p, torch.tensor([[0, 1, 2]]))
    return m.subdivide(subdivisions) if subdivisions else m


def perturbed_grid(nx: int = 10, ny: int = 10, amplitude: float = 0.2, generator=None) -> Mesh:
    """Structured triangle grid whose interior vertices move by at most ``amplitude`` (< 0.5) cell widths per axis."""
    g = structured_grid(nx, ny)
    cell = torch.tensor([1.0 / nx, 1.0 / ny])
    jitter = (torch.rand(g.points.shape, generator=generator) * 2 - 1) * amplitude * cell
    jitter[g.get_boundary_mesh(data_source="none").cells.reshape(-1)] = 0
    return g._with_points(g.points + jitter)


# ------------------------------------------------------------ further surfaces
def _platonic(points, faces, radius: float, subdivisions: int) -> Mesh:
    p = torch.tensor(points, dtype=torch.float32)
    m = Mesh(radius * p / p.norm(dim=1, keepdim=True), torch.tensor(faces))
    return m.subdivide(subdivisions) if subdivisions else m


def tetrahedron_surface(radius: float = 1.0, subdivisions: int = 0) -> Mesh:
    return _platonic([[1, 1, 1], [1, -1, -1], [-1, 1, -1], [-1, -1, 1]], [[0, 1, 2], [0, 3, 1], [0, 2, 3], [1, 3, 2]],
                     radius, subdivisions)


def octahedron_surface(radius: float = 1.0, subdivisions: int = 0) -> Mesh:
    return _platonic([[1, 0, 0], [-1, 0, 0], [0, 1, 0], [0, -1, 0], [0, 0, 1], [0, 0, -1]],
                     [[0, 2, 4], [2, 1, 4], [1, 3, 4], [3, 0, 4], [2, 0, 5], [1, 2, 5], [3, 1, 5], [0, 3, 5]], radius, subdivisions)


def icosahedron_surface(radius: float = 1.0) -> Mesh:
    return icosphere(0, radius)


def hemisphere(n_lat: int = 8, n_lon: int = 32, radius: float = 1.0) -> Mesh:
    """Upper half of a latitude / longitude sphere, open at the equator."""
    th = torch.linspace(0, math.pi / 2, n_lat + 1)[1:]
    ph = torch.arange(n_lon) * (2 * math.pi / n_lon)
    T, P = torch.meshgrid(th, ph, indexing="ij")
    ring = torch.stack([T.sin() * P.cos(), T.sin() * P.sin(), T.cos()], -1).reshape(-1, 3)
    pts = radius * torch.cat([torch.tensor([[0.0, 0.0, 1.0]]), ring])
    j = torch.arange(n_lon)
    jn = (j + 1) % n_lon
    cells = [torch.stack([torch.zeros_like(j), 1 + j, 1 + jn], 1)]
    for r in range(n_lat - 1):
        a, b = 1 + r * n_lon, 1 + (r + 1) * n_lon
        cells += [torch.stack([a + j, b + j, b + jn], 1), torch.stack([a + j, b + jn, a + jn], 1)]
    return Mesh(pts, torch.cat(cells))


def cone(n_angular: int = 32, n_height: int = 8, radius: float = 1.0, height: float = 2.0, capped: bool = True) -> Mesh:
    """Lateral surface from the base circle (z = 0) to the apex (z = height), optionally with the base disk."""
    ph = torch.arange(n_angular) * (2 * math.pi / n_angular)
    levels = torch.linspace(0, 1, n_height + 1)[:-1]
    rings = [torch.stack([(1 - s) * radius * ph.cos(), (1 - s) * radius * ph.sin(), torch.full_like(ph, float(s) * height)], 1)
             for s in levels]
    pts = torch.cat(rings + [torch.tensor([[0.0, 0.0, height]])])
    apex = n_height * n_angular
    j = torch.arange(n_angular)
    jn = (j + 1) % n_angular
    cells = []
    for r in range(n_height - 1):
        a, b = r * n_angular, (r + 1) * n_angular
        cells += [torch.stack([a + j, a + jn, b + jn], 1), torch.stack([a + j, b + jn, b + j], 1)]
    top = (n_height - 1) * n_angular
    cells.append(torch.stack([top + j, top + jn, torch.full_like(j, apex)], 1))
    if capped:
        pts = torch.cat([pts, torch.zeros(1, 3)])
        cells.append(torch.stack([jn, j, torch.full_like(j, apex + 1)], 1))
    return Mesh(pts, torch.cat(cells))


def cylinder_open(n_angular: int = 32, n_height: int = 8, radius: float = 1.0, height: float = 2.0) -> Mesh:
    return cylinder(n_angular=n_angular, n_height=n_height, radius=radius, height=height, capped=False)


def mobius_strip(n_around: int = 64, n_across: int = 4, radius: float = 1.0, width: float = 0.4) -> Mesh:
    """One-sided band: the cross-section turns by half a revolution around the loop, and the seam joins flipped."""
    u = torch.arange(n_around) * (2 * math.pi / n_around)
    v = torch.linspace(-width / 2, width / 2, n_across + 1)
    U, V = torch.meshgrid(u, v, indexing="ij")
    r = radius + V * (U / 2).cos()
    pts = torch.stack([r * U.cos(), r * U.sin(), V * (U / 2).sin()], -1).reshape(-1, 3)
    w = n_across + 1
    cells = []
    for i in range(n_around):
        last = i == n_around - 1
        for k in range(n_across):
            a, b = i * w + k, i * w + k + 1
            c, d = ((n_across - k), (n_across - k - 1)) if last else ((i + 1) * w + k, (i + 1) * w + k + 1)
            cells += [[a, c, d], [a, d, b]]
    return Mesh(pts, torch.tensor(cells))


# ------------------------------------------------------------- further volumes
def sphere_volume(subdivisions: int = 2, radius: float = 1.0) -> Mesh:
    return ball_volume(subdivisions, radius)


def tetrahedron_volume(subdivisions: int = 0) -> Mesh:
    m = single_tetrahedron()
    return m.subdivide(subdivisions) if subdivisions else m


def cylinder_volume(n_radial: int = 3, n_angular: int = 16, n_height: int = 4, radius: float = 1.0, height: float = 2.0) -> Mesh:
    """Tetrahedral solid cylinder: a triangulated disk swept along ``z`` in ``n_height`` layers."""
    from .projections import extrude

    layer = disk(n_radial=n_radial, n_angular=n_angular, radius=radius)
    step = height / n_height
    slabs = []
    for k in range(n_height):
        base = Mesh(torch.nn.functional.pad(layer.points, (0, 1), value=k * step), layer.cells)
        slabs.append(extrude(base, [0.0, 0.0, step]))
    return Mesh.merge(slabs).clean()


# ---------------------------------------------------------- further procedural
def value_noise(points: torch.Tensor, frequency: float = 2.0, octaves: int = 3, seed: int = 0) -> torch.Tensor:
    """Smooth pseudo-random scalar field: a sum of randomly oriented, randomly phased cosines per octave."""
    g = torch.Generator().manual_seed(int(seed))
    out = torch.zeros(points.shape[0], dtype=points.dtype)
    for o in range(octaves):
        k = torch.randn(8, points.shape[1], generator=g)
        k = k / k.norm(dim=1, keepdim=True) * frequency * 2 ** o
        phase = torch.rand(8, generator=g) * 2 * math.pi
        out = out + (torch.cos(points.cpu() @ k.T.to(points.dtype) + phase.to(points.dtype))).mean(1) / 2 ** o
    return out.to(points.device)


def noisy_mesh(mesh: Mesh, amplitude: float = 0.05, frequency: float = 2.0, octaves: int = 3, seed: int = 0) -> Mesh:
    """Displace a codimension-1 mesh along its point normals (any other mesh: along the first axis) by smooth noise."""
    field = value_noise(mesh.points, frequency, octaves, seed)
    if mesh.n_cells and mesh.codimension == 1:
        direction = mesh.point_normals
    else:
        direction = torch.zeros_like(mesh.points)
        direction[:, 0] = 1.0
    return mesh._with_points(mesh.points + amplitude * field[:, None] * direction)


def lumpy_ball(subdivisions: int = 2, amplitude: float = 0.2, n_modes: int = 6, generator=None) -> Mesh:
    """Tetrahedral solid bounded by :func:`lumpy_sphere`."""
    s = lumpy_sphere(subdivisions, amplitude, n_modes, generator)
    return Mesh(torch.cat([s.points, torch.zeros(1, 3)]), torch.cat([s.cells, torch.full((s.n_cells, 1), s.n_points)], 1))
