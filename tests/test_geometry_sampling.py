"""mesh_to_voxel_fraction, mesh_poisson_disk_sample and remeshing on analytic shapes (CPU and CUDA paths)."""
import math

import pytest
import torch

from physicsnemo_b200.mesh import primitives
from physicsnemo_b200.nn.functional import mesh_poisson_disk_sample, mesh_to_voxel_fraction, remeshing
from physicsnemo_b200.nn.functional.geometry.mesh_poisson_disk_sample import _pairs_within

DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]


def _sphere(level, device, radius=1.0):
    s = primitives.icosphere(level)
    return (s.points.float() * radius).to(device), s.cells.to(device)


def _min_pair_distance(p):
    d = torch.cdist(p.double(), p.double())
    d.fill_diagonal_(float("inf"))
    return d.min(dim=1).values


@pytest.mark.parametrize("device", DEVICES)
def test_voxel_fraction_of_sphere(device):
    V, F = _sphere(3, device, 0.8)
    h, n = 2.0 / 24, 24
    f = mesh_to_voxel_fraction(V, F, (-1.0, -1.0, -1.0), h, (n, n, n), n_samples=32)
    assert f.shape == (n, n, n) and f.dtype == torch.float32
    assert float(f.min()) == 0.0 and float(f.max()) == 1.0
    exact = float((V[F[:, 0]] * torch.linalg.cross(V[F[:, 1]], V[F[:, 2]])).sum() / 6)
    assert float(f.sum()) * h ** 3 == pytest.approx(exact, rel=0.02)
    assert torch.equal(f, mesh_to_voxel_fraction(V, F, (-1.0, -1.0, -1.0), h, (n, n, n), n_samples=32))   # seeded
    centre = f[n // 2, n // 2, n // 2]
    assert float(centre) == 1.0 and float(f[0, 0, 0]) == 0.0
    # anisotropic grid: output is [nz, ny, nx] and x runs fastest
    g = mesh_to_voxel_fraction(V, F.reshape(-1), torch.tensor([-1.0, -1.0, -1.0]), h, (24, 12, 6), n_samples=8)
    assert g.shape == (6, 12, 24)
    assert torch.allclose(g.sum(dim=(0, 1)) > 0, f[:6, :12].sum(dim=(0, 1)) > 0)


@pytest.mark.parametrize("device", DEVICES)
def test_voxel_fraction_open_mesh_uses_winding_number(device):
    V, F = _sphere(3, device, 0.8)
    keep = V[F].mean(1)[:, 2] < 0.7                         # cut a small cap off: the winding number stays > 0.5 inside
    h, n = 2.0 / 16, 16
    closed = mesh_to_voxel_fraction(V, F, (-1.0, -1.0, -1.0), h, (n, n, n), n_samples=16)
    opened = mesh_to_voxel_fraction(V, F[keep], (-1.0, -1.0, -1.0), h, (n, n, n), n_samples=16, open_mesh=True)
    assert float((closed - opened).abs().mean()) < 0.02


def test_pair_search_matches_bruteforce():
    torch.manual_seed(0)
    a, b = torch.rand(500, 3), torch.rand(700, 3)
    got = set(map(tuple, _pairs_within(a, b, 0.1).t().tolist()))
    want = set(map(tuple, (torch.cdist(a, b) <= 0.1).nonzero().tolist()))
    assert got == want


@pytest.mark.parametrize("device", DEVICES)
def test_poisson_disk_dart_throwing(device):
    V, F = _sphere(3, device)
    p = mesh_poisson_disk_sample(V, F, min_distance=0.1, batch_size=4096, max_iterations=32)
    assert p.dtype == torch.float32 and p.shape[1] == 3
    assert float(_min_pair_distance(p).min()) >= 0.1 - 1e-6
    assert float(p.norm(dim=-1).min()) > 0.99 and float(p.norm(dim=-1).max()) <= 1.0 + 1e-5   # on the surface
    # saturation: disks of radius r/2 do not overlap, so N = packing · 4π / (π r²/4) with packing in (0.4, 0.9069)
    assert 0.4 * 1600 < p.shape[0] < 0.9069 * 1600
    capped = mesh_poisson_disk_sample(V, F, min_distance=0.1, batch_size=4096, max_points=50)
    assert capped.shape[0] == 50
    r = (0.05 + 0.15 * (V[:, 2] > 0)).float()                # coarse on the upper half
    q = mesh_poisson_disk_sample(V, F, per_vertex_radius=r, batch_size=4096, max_iterations=32)
    assert int((q[:, 2] < -0.1).sum()) > 3 * int((q[:, 2] > 0.1).sum())


@pytest.mark.parametrize("device", DEVICES)
def test_poisson_disk_sample_elimination(device):
    V, F = _sphere(3, device)
    q = mesh_poisson_disk_sample(V, F, mode="weighted_sample_elimination", target_num_points=300, batch_size=4096)
    assert q.shape == (300, 3)
    nn = _min_pair_distance(q)
    spacing = 2.0 * math.sqrt(4 * math.pi / (2 * math.sqrt(3.0) * 300))       # hexagonal packing distance
    assert float(nn.mean()) > 0.6 * spacing                                     # white noise gives ≈ 0.27 spacing
    assert float(nn.std() / nn.mean()) < 0.25
    with pytest.raises(ValueError):
        mesh_poisson_disk_sample(V, F, mode="nope")


@pytest.mark.parametrize("device", DEVICES)
def test_remeshing_keeps_a_closed_oriented_sphere(device):
    V, F = _sphere(4, device)
    V = V.double() * 2 + 1
    v, f = remeshing(V, F, 200)
    assert v.dtype == torch.float64 and f.dtype == torch.int64 and v.shape == (200, 3)
    e = torch.cat((f[:, [0, 1]], f[:, [1, 2]], f[:, [2, 0]]))
    und, cnt = torch.unique(e.sort(1).values, dim=0, return_counts=True)
    assert cnt.unique().tolist() == [2]                                          # watertight manifold
    assert v.shape[0] - und.shape[0] + f.shape[0] == 2                           # a sphere
    assert torch.unique(e, dim=0).shape[0] == e.shape[0]                         # consistently oriented
    rad = (v - 1).norm(dim=-1)
    assert float(rad.min()) > 1.99 and float(rad.max()) < 2.0 + 1e-6             # vertices lie on the source surface
    vol = float(((v[f[:, 0]] - 1) * torch.linalg.cross(v[f[:, 1]] - 1, v[f[:, 2]] - 1)).sum() / 6)
    assert vol == pytest.approx(4 / 3 * math.pi * 8, rel=0.06) and vol > 0
    area = 0.5 * torch.linalg.cross(v[f[:, 1]] - v[f[:, 0]], v[f[:, 2]] - v[f[:, 0]]).norm(dim=-1)
    assert float(area.std() / area.mean()) < 0.35                                # near-uniform triangles
    dens = ((V[:, 2] > 1).double() * 3 + 1)
    v2, _ = remeshing(V, F, 600, vertex_density=dens)
    assert int((v2[:, 2] > 1).sum()) > 1.8 * int((v2[:, 2] <= 1).sum())


def test_remeshing_validation():
    V, F = _sphere(1, "cpu")
    with pytest.raises(ValueError):
        remeshing(V, F, 2)
    with pytest.raises(ValueError):
        remeshing(V, F, V.shape[0] + 1)
    with pytest.raises(TypeError):
        remeshing(V, F.float(), 10)
    with pytest.raises(TypeError):
        remeshing(V, F, 10.0)
    with pytest.raises(ValueError):
        remeshing(V, F, 10, vertex_density=torch.ones(3))
