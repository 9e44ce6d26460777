"""Headless renderers: analytic checks of the PyTorch implementations (CPU) and kernel-vs-oracle checks (GPU)."""
import math

import pytest
import torch

from physicsnemo_b200.mesh import primitives as P
from physicsnemo_b200.nn.functional.rendering import (isosurface_render, line_integral_convolution, mesh_raycast,
                                                     point_cloud_render, scalar_field_to_rgba, vector_field_to_rgba,
                                                     volume_render, wireframe_render)

CAM = dict(eye=[0.0, 0.0, -2.5], center=[0.0, 0.0, 0.0], up=[0.0, 1.0, 0.0], fov_y_degrees=45.0)
BOX = dict(bounds_min=[-1.0, -1.0, -1.0], bounds_max=[1.0, 1.0, 1.0])


def _cube_volume(dev="cpu"):
    v = torch.zeros(24, 24, 24, 4, dtype=torch.uint8, device=dev)
    v[..., 0], v[..., 1], v[..., 2] = 96, 192, 255
    v[7:17, 7:17, 7:17, 3] = 96
    return v


def _sphere_field(n=40, dev="cpu"):
    x = torch.linspace(-1, 1, n, device=dev)
    X, Y, Z = torch.meshgrid(x, x, x, indexing="ij")
    return torch.sqrt(X * X + Y * Y + Z * Z) - 0.6


def test_volume_and_isosurface_torch():
    rgba, depth = volume_render(_cube_volume(), 32, 32, **CAM, **BOX, step_size=0.08, max_steps=80)
    assert rgba.shape == (32, 32, 4) and depth.shape == (32, 32)
    assert rgba[16, 16, 3] > 0.8 and torch.isinf(depth[0, 0]) and rgba[0, 0].abs().sum() == 0
    assert torch.allclose(rgba[16, 16, :3], torch.tensor([96, 192, 255.0]) / 255, atol=1e-5)
    assert 1.9 < float(depth[16, 16]) < 2.3                      # cube front face at z = -0.39, eye at -2.5
    rgba, depth, normal = isosurface_render(_sphere_field(), 33, 33, **CAM, **BOX, step_size=0.02, max_steps=300,
                                            surface_color=[1.0, 0.5, 0.25])
    assert abs(float(depth[16, 16]) - 1.9) < 0.02                # sphere of radius 0.6
    assert normal[16, 16, 2] < -0.99 and torch.isinf(depth[0, 0]) and rgba[16, 16, 3] == 1
    assert torch.allclose(rgba[16, 16, :3] / rgba[16, 16, 0], torch.tensor([1.0, 0.5, 0.25]), atol=1e-5)


def test_mesh_raycast_points_wireframe_torch():
    s = P.icosphere(2)
    vc = (s.points + 1) / 2
    rgba, depth, normal = mesh_raycast(s.points, s.cells, 31, 31, **CAM, vertex_colors=vc)
    assert abs(float(depth[15, 15]) - 1.5) < 0.01 and normal[15, 15, 2] < -0.95 and torch.isinf(depth[0, 0])
    pts = torch.tensor([[0.0, 0, 0], [0.0, 0, 1.0], [0.5, 0.5, 0]])
    cols = torch.tensor([[1.0, 0, 0], [0, 1.0, 0], [0, 0, 1.0]])
    rgba, depth = point_cloud_render(pts, 32, 32, **CAM, point_colors=cols, point_size=3)
    assert rgba[16, 16].tolist() == [1, 0, 0, 1] and abs(float(depth[16, 16]) - 2.5) < 1e-5      # nearer point wins
    assert int((rgba[..., 2] == 1).sum()) == 9
    edges = torch.tensor([[[-0.5, 0.0, 0.0], [0.5, 0.0, 0.0]], [[0.0, -0.5, 0.5], [0.0, 0.5, 0.5]]])
    rgba, depth = wireframe_render(edges, 64, 64, **CAM, line_color=[0.0, 1.0, 0.0])
    lit = rgba[..., 3] > 0
    assert lit[32, 20:44].all() and lit[24:40, 32].all() and abs(float(depth[32, 32]) - 2.5) < 1e-3
    assert abs(float(depth[26, 32]) - 3.0) < 1e-3 and not lit[10, 10]


def test_lic_and_colour_maps_torch():
    n = 12
    v = torch.zeros(n, n, n, 3)
    v[..., 0] = 1.0
    seed = torch.rand(n, n, n, generator=torch.Generator().manual_seed(0))
    lic = line_integral_convolution(v, seed, step_size=1.0, num_steps=4, contrast=1.0)
    # along x the texture is a weighted moving average of the seed
    w = [1 - k / 5 for k in range(1, 5)]
    i = 6
    want = (seed[i, 3, 3] + sum(wk * (seed[i + k, 3, 3] + seed[i - k, 3, 3]) for k, wk in zip(range(1, 5), w))) / (1 + 2 * sum(w))
    assert abs(float(lic[i, 3, 3]) - float(want)) < 1e-5
    rgba = scalar_field_to_rgba(torch.linspace(0, 1, 27).reshape(3, 3, 3), 0.0, 1.0)
    assert rgba.dtype == torch.uint8 and rgba[0, 0, 0].tolist() == [0, 0, 127, 0] and rgba[2, 2, 2].tolist() == [127, 0, 0, 204]
    out = vector_field_to_rgba(v * 0.5, lic, 0.0, 1.0)
    assert out.shape == (n, n, n, 4) and int(out[..., 3].max()) <= int(0.5 * 0.8 * 255) + 1
    with pytest.raises(ValueError):
        scalar_field_to_rgba(torch.zeros(3, 3, 3), 1.0, 0.0)


@pytest.mark.gpu
def test_render_kernels_match_oracles():
    dev = "cuda"
    kw = dict(step_size=0.05, max_steps=120)
    a = volume_render(_cube_volume(dev), 48, 64, **CAM, **BOX, **kw, implementation="cuda")
    b = volume_render(_cube_volume(dev), 48, 64, **CAM, **BOX, **kw, implementation="torch")
    assert (a[0] - b[0]).abs().max() < 2e-3 and (torch.nan_to_num(a[1], posinf=0) - torch.nan_to_num(b[1], posinf=0)).abs().max() < 1e-3
    f = _sphere_field(48, dev)
    cf = torch.rand(48, 48, 48, 3, device=dev)
    a = isosurface_render(f, 40, 56, **CAM, **BOX, step_size=0.02, max_steps=300, color_field=cf, implementation="cuda")
    b = isosurface_render(f, 40, 56, **CAM, **BOX, step_size=0.02, max_steps=300, color_field=cf, implementation="torch")
    same = torch.isinf(a[1]) == torch.isinf(b[1])
    assert same.float().mean() > 0.995
    m = same & ~torch.isinf(a[1])
    assert (a[1][m] - b[1][m]).abs().max() < 1e-3 and (a[0][m] - b[0][m]).abs().max() < 5e-3 and (a[2][m] - b[2][m]).abs().max() < 5e-3
    s = P.lumpy_sphere(3, generator=torch.Generator().manual_seed(1)).to(dev)
    fc = torch.rand(s.n_cells, 3, device=dev)
    for extra in (dict(face_colors=fc), dict(vertex_colors=torch.rand(s.n_points, 4, device=dev)), {}):
        a = mesh_raycast(s.points, s.cells, 64, 64, **CAM, **extra, implementation="cuda")
        b = mesh_raycast(s.points, s.cells, 64, 64, **CAM, **extra, implementation="torch")
        same = torch.isinf(a[1]) == torch.isinf(b[1])
        assert same.float().mean() > 0.998
        m = same & ~torch.isinf(a[1])
        assert (a[1][m] - b[1][m]).abs().max() < 1e-3
        assert ((a[0][m] - b[0][m]).abs().amax(-1) < 1e-3).float().mean() > 0.995           # silhouette-edge ties aside
    pts = torch.randn(20000, 3, device=dev) * 0.5
    pc = torch.rand(20000, 3, device=dev)
    a = point_cloud_render(pts, 96, 128, **CAM, point_colors=pc, point_size=2, implementation="cuda")
    b = point_cloud_render(pts, 96, 128, **CAM, point_colors=pc, point_size=2, implementation="torch")
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    e = torch.randn(300, 2, 3, device=dev) * 0.7
    a = wireframe_render(e, 96, 128, **CAM, line_thickness=2, implementation="cuda")
    b = wireframe_render(e, 96, 128, **CAM, line_thickness=2, implementation="torch")
    assert ((a[0] != b[0]).any(-1)).float().mean() < 0.01 and (torch.nan_to_num(a[1], posinf=0) - torch.nan_to_num(b[1], posinf=0)).abs().median() == 0
    v = torch.randn(20, 22, 24, 3, device=dev)
    seed = torch.rand(20, 22, 24, device=dev)
    a = line_integral_convolution(v, seed, implementation="cuda")
    b = line_integral_convolution(v, seed, implementation="torch")
    # streamlines of a random field are chaotic (rounding differences grow every step): compare the bulk
    assert ((a - b).abs() > 1e-4).float().mean() < 0.05
    gx, gy, gz = torch.meshgrid(torch.linspace(-1, 1, 20, device=dev), torch.linspace(-1, 1, 22, device=dev),
                                torch.linspace(-1, 1, 24, device=dev), indexing="ij")
    swirl = torch.stack([-gy, gx, 0.3 + 0 * gz], -1)
    sa = line_integral_convolution(swirl, seed, implementation="cuda")
    sb = line_integral_convolution(swirl, seed, implementation="torch")
    assert ((sa - sb).abs() > 1e-4).float().mean() < 0.002 and (sa - sb).abs().median() < 1e-6
    fld = torch.randn(20, 22, 24, device=dev)
    assert (scalar_field_to_rgba(fld, -1.0, 1.0, implementation="cuda").int() - scalar_field_to_rgba(fld, -1.0, 1.0, implementation="torch").int()).abs().max() <= 1
    assert (vector_field_to_rgba(v, a, 0.0, 2.0, implementation="cuda").int() - vector_field_to_rgba(v, a, 0.0, 2.0, implementation="torch").int()).abs().max() <= 1
